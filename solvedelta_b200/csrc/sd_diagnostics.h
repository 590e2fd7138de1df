/*
 * Entry points of the profiling build only (compiled with -DSD_DIAGNOSTICS into
 * libsolvedelta_b200_diag.so; the shipped library has none of them and none of the
 * clock stamps inside its kernels).  No upstream counterpart.
 */
#ifndef SOLVEDELTA_B200_DIAGNOSTICS_H
#define SOLVEDELTA_B200_DIAGNOSTICS_H
#ifdef SD_DIAGNOSTICS
#include "../../include/solvedelta_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/*
 * Runs sd_forward and, when `bwd` is not NULL, sd_backward, with a CUDA event between
 * launches, waits for the stream and returns the device time of every launch in
 * milliseconds (`count` entries, in launch order; sd_launch_name gives their names).
 * Not thread safe; not for use inside stream capture.
 */
int sd_profile_step(const sd_forward_args *fwd, const sd_backward_args *bwd, void *stream,
                    float *ms, int capacity, int *count);
const char *sd_launch_name(int index);
/*
 * When `device_buffer` (at least 16*16 int64) is not NULL, one CTA of every chunk kernel
 * records the SM clock at each of its phase boundaries into slot [launch index][phase];
 * NULL switches the recording off.  Process-wide, not thread safe.
 */
void sd_debug_timeline(void *device_buffer);

#ifdef __cplusplus
}
#endif
#endif /* SD_DIAGNOSTICS */
#endif
