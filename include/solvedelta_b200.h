/*
 * solvedelta_b200 -- C ABI of the B200 (sm_100a) SolveDelta chunked recurrence.
 *
 * Plain pointers and sizes only.  Every device pointer is memory of the GPU
 * that is current when the call is made; the library allocates nothing
 * (callers pass the `saved` and `scratch` buffers, sized by the query
 * functions), launches only asynchronous work on the stream it is given and
 * never synchronises.  Functions return 0 on success and a negative
 * sd_status otherwise; nothing throws, nothing exits.
 *
 * Upstream interfaces these entry points stand in for (paths inside the
 * SolveDelta project):
 *   sd_forward      causallsso/ops/operator.py:13-55 (solvedelta_native) ->
 *                   causallsso/ops/residual_frame/operator.py:154-304
 *                   (solvedelta_residual_frame_native, dense branch)
 *   sd_backward     the autograd reverse of the same call:
 *                   causallsso/ops/residual_frame/operator.py:74-138
 *                   (_RelativeExterior.backward),
 *                   causallsso/ops/residual_frame/predictor.py:129-282
 *                   (_OjaResidual.backward),
 *                   causallsso/ops/residual_frame/l2norm.py:129-146
 *   sd_decode_step  causallsso/ops/residual_frame/recurrent.py:188-327
 *                   (solvedelta_recurrent_inference, T = 1, no grad)
 *
 * Tensor contract (same as upstream): u, h, q, keys, values, erase_raw,
 * write_raw are BF16 with unit innermost stride and arbitrary outer strides
 * (views into a fused projection row are legal); log_decay and gamma are FP32;
 * the continuation states are FP32, contiguous, C [B,H,r,r] with
 * prediction = C u and S [B,H,r,V].  r and V may be any value in 1..128.
 */
#ifndef SOLVEDELTA_B200_H
#define SOLVEDELTA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    SD_OK = 0,
    SD_ERR_INVALID_ARGUMENT = -1, /* null pointer, non-positive size, bad stride */
    SD_ERR_UNSUPPORTED_SHAPE = -2, /* r or V outside 1..128 */
    SD_ERR_BUFFER_TOO_SMALL = -3,  /* saved / scratch smaller than the query says */
    SD_ERR_LAUNCH_FAILED = -4,     /* the CUDA runtime refused a launch */
    SD_ERR_NO_DEVICE = -5,         /* no CUDA device / wrong architecture */
    SD_ERR_STATIC_WORKSPACE_EXCEEDED = -6 /* sd_forward_static: shape too large, see below */
} sd_status;

/* A strided [B,T,H,width] operand: element strides of batch, token, head. */
typedef struct {
    const void *ptr;
    int64_t stride_b, stride_t, stride_h;
} sd_operand;

typedef struct {
    int32_t B, T, H, r, V;
} sd_shape;

typedef struct {
    sd_shape shape;
    sd_operand u, h, q, keys, values;  /* BF16, widths r,r,r,r,V */
    sd_operand erase_raw, write_raw;    /* BF16 raw gate logits, widths r,V */
    sd_operand log_decay;               /* FP32, width r, values <= 0 */
    sd_operand gamma;                   /* FP32, width 1 (per token; strides may be 0) */
    const float *C0, *S0;               /* initial states or NULL (= zero) */
    void *y;                            /* out: BF16 contiguous [B,T,H,V] */
    float *C_T, *S_T;                   /* out: final states or NULL */
    void *saved;                        /* out: kept for sd_backward (sd_saved_bytes) */
    size_t saved_bytes;
    void *scratch;                      /* temporary (sd_forward_scratch_bytes) */
    size_t scratch_bytes;
    /* Token masks, one byte per token, contiguous [B,T]; either may be NULL.  A token whose
     * valid byte is 0 takes no part: zero output, state and gradients untouched.  A valid token
     * whose reset byte is non-zero starts from the zero state.  Replaces the gather into
     * reset-free segments of causallsso/ops/operator.py:96-193 (semantics:
     * causallsso/reference.py:157-164,216-226); handled inside the kernels, no host work. */
    const unsigned char *valid_mask;
    const unsigned char *reset_mask;
} sd_forward_args;

typedef struct {
    sd_shape shape;
    sd_operand u, h, q, keys, values, erase_raw, write_raw, log_decay, gamma;
    sd_operand dy;                      /* BF16 upstream gradient of y, width V */
    const float *dC_T, *dS_T;           /* gradients of the final states or NULL */
    const void *saved;                  /* what sd_forward wrote */
    size_t saved_bytes;
    void *scratch;                      /* temporary (sd_backward_scratch_bytes) */
    size_t scratch_bytes;
    /* outputs, all contiguous: BF16 [B,T,H,width] ... */
    void *du, *dh, *dq, *dkeys, *dvalues, *derase_raw, *dwrite_raw;
    float *dlog_decay;                  /* FP32 [B,T,H,r] */
    float *dgamma;                      /* FP32 [B,T,H] */
    float *dC0, *dS0;                   /* FP32 or NULL */
    const unsigned char *valid_mask;    /* the masks the forward call was given (or NULL) */
    const unsigned char *reset_mask;
} sd_backward_args;

typedef struct {
    sd_shape shape;                     /* T must be 1 */
    sd_operand u, h, q, keys, values, erase_raw, write_raw, log_decay, gamma;
    float *C, *S;                       /* in/out recurrent cache, updated in place */
    void *y;                            /* out: BF16 [B,1,H,V] */
} sd_decode_args;

/*
 * Glue of the block around the mixer (BF16 rows, contiguous), forward and reverse:
 * sd_add_rmsnorm  sum = x + delta and normed = RMSNorm(sum) * weight in one pass: a residual add and
 *                 the norm that follows it (causallsso/modeling_solvedelta.py:230-255).  delta may be
 *                 NULL (the norm alone: sum is not written) when D is a multiple of 256 up to 2048.
 * sd_add_rmsnorm_backward  the one gradient x and delta share, dsum + d normed / d sum, and the weight
 *                 gradient; D a multiple of 256 up to 2048 (else SD_ERR_UNSUPPORTED_SHAPE)
 * sd_swiglu       out = silu(gate) * value for rows [gate | value] (modeling_solvedelta.py:68-101)
 * sd_swiglu_backward  the gradient row [d gate | d value] from dout
 */
typedef struct {
    int64_t rows;
    int32_t D;
    float eps;
    const void *x, *delta;             /* BF16 [rows][D]; delta may be NULL */
    const float *weight;               /* [D] */
    void *sum, *normed;                /* out BF16 [rows][D]; sum unused when delta is NULL */
} sd_add_rmsnorm_args;

typedef struct {
    int64_t rows;
    int32_t D;
    float eps;
    const void *sum;                   /* BF16 [rows][D]: the forward's sum (x itself when delta was NULL) */
    const float *weight;               /* [D] */
    const void *dsum;                  /* BF16 cotangent of sum, or NULL */
    const void *dnormed;               /* BF16 cotangent of normed */
    void *dx;                          /* out BF16 [rows][D]: gradient of x, and of delta */
    float *dweight;                    /* out [D] */
    void *scratch;                     /* sd_add_rmsnorm_backward_scratch_bytes */
    size_t scratch_bytes;
} sd_add_rmsnorm_backward_args;

typedef struct {
    int64_t rows;
    int32_t I;
    const void *gate_value;            /* BF16 [rows][2 I] */
    void *out;                         /* forward: BF16 [rows][I] */
    const void *dout;                  /* backward: BF16 [rows][I] */
    void *dgate_value;                 /* backward: out BF16 [rows][2 I] */
} sd_swiglu_args;

int sd_add_rmsnorm(const sd_add_rmsnorm_args *args, void *stream);
size_t sd_add_rmsnorm_backward_scratch_bytes(int64_t rows, int32_t D);
int sd_add_rmsnorm_backward(const sd_add_rmsnorm_backward_args *args, void *stream);
int sd_swiglu(const sd_swiglu_args *args, void *stream);
int sd_swiglu_backward(const sd_swiglu_args *args, void *stream);

/*
 * The gradient of the fused projection row (causallsso/model.py:321-332 slices it; autograd upstream
 * adds one zero-filled full row per slice) written in one pass: dst[row] = [piece 0 | piece 1 | ... | zeros].
 * Every piece is a contiguous BF16 matrix [rows][width] (NULL: zeros); widths and row_width are whole groups
 * of eight channels and all pointers 16-byte aligned, else SD_ERR_UNSUPPORTED_SHAPE.
 */
#define SD_PACK_MAX_PIECES 12
typedef struct {
    const void *src;
    int32_t width;
} sd_row_piece;
typedef struct {
    int64_t rows;
    int32_t pieces;
    int32_t row_width;                 /* >= the sum of the widths; the rest of a row is zero-filled */
    sd_row_piece piece[SD_PACK_MAX_PIECES];
    void *dst;                         /* out BF16 [rows][row_width] */
} sd_pack_rows_args;
int sd_pack_rows(const sd_pack_rows_args *args, void *stream);

/*
 * A projection of a cached single-token step: y [M][N] = x [M][K] weight^T (+ bias) for M <= 4 rows
 * (nn.Linear layout, BF16, FP32 accumulation), one warp per output column.  With swiglu != 0 the output is
 * [M][N/2] = silu(y[:, :N/2]) * y[:, N/2:] (the gated MLP's first projection and activation,
 * causallsso/modeling_solvedelta.py:68-101).  K and x_stride multiples of 8, x and weight 16-byte aligned,
 * else SD_ERR_UNSUPPORTED_SHAPE (the caller then runs its library GEMM).
 */
typedef struct {
    int32_t M, N, K;
    int32_t swiglu;
    const void *x;                     /* BF16 [M][K], rows x_stride elements apart */
    int64_t x_stride;
    const void *weight;                /* BF16 [N][K] contiguous */
    const void *bias;                  /* BF16 [N] or NULL */
    void *y;                           /* out BF16, rows y_stride elements apart */
    int64_t y_stride;
} sd_gemv_args;
int sd_gemv(const sd_gemv_args *args, void *stream);

/*
 * Cross entropy over BF16 logits, the owner behind fuse_cross_entropy upstream
 * (FusedCrossEntropyLoss, causallsso/modeling_solvedelta.py:469-470).  Forward: per row the log-sum-exp
 * and -log softmax(label), 0 for rows whose label is ignore_index.  Backward: d logits =
 * (softmax - onehot(label)) * coef, coef a device scalar (upstream gradient / token count); zeros for
 * ignored rows.  The mean over the counted rows is the caller's (a sum of `rows` floats).
 */
typedef struct {
    int64_t rows;
    int32_t V;
    const void *logits;                /* BF16 [rows][V] */
    const int64_t *labels;             /* [rows] */
    int64_t ignore_index;
    float *lse;                        /* [rows]: out of forward, in of backward */
    float *row_loss;                   /* forward: out [rows] */
    const float *coef;                 /* backward: device scalar */
    void *dlogits;                     /* backward: out BF16 [rows][V] */
} sd_cross_entropy_args;
int sd_cross_entropy_forward(const sd_cross_entropy_args *args, void *stream);
int sd_cross_entropy_backward(const sd_cross_entropy_args *args, void *stream);

/*
 * The whole mixer glue of a cached single-token step in the decode kernel: q, k, v come from
 * the conv4 + SiLU of the projection row against the carried window (advanced in place,
 * causallsso/model.py:146-164 at T = 1), the log decay from the decay gate
 * (-exp(A[h]) softplus(raw + bias), model.py:375-390), the geometry rate from
 * sigmoid(raw + bias) (model.py:391-394); then the recurrent step of sd_decode_step
 * (recurrent.py:188-327), optionally followed by the gated RMSNorm of the output row.  One
 * launch instead of conv, gate, three element-wise kernels, the step and the norm.  No upstream counterpart as a single call.
 */
typedef struct {
    sd_shape shape;                     /* T must be 1 */
    sd_operand u, h, erase_raw, write_raw;   /* BF16 views of the projection row, widths r,r,r,V */
    const void *qkv;                    /* BF16 conv input of the token: per batch row 2*H*r + H*V channels (q|k|v) */
    int64_t qkv_stride_b;               /* elements between batch rows */
    const float *conv_weight;           /* [D][4] */
    void *conv_state;                   /* BF16 [B][D][3], in/out */
    const void *decay_raw;              /* BF16 [B][H*r] */
    int64_t decay_stride_b;
    const float *log_rate;              /* [H] */
    const float *decay_bias;            /* [H*r] */
    const void *geometry_raw;           /* BF16 [B][H] */
    int64_t geometry_stride_b;
    const float *geometry_bias;         /* [H] */
    float *C, *S;                       /* in/out recurrent cache */
    void *y;                            /* out: BF16 [B,1,H,V] */
    /* optional: the sigmoid-gated RMSNorm of the output row (causallsso/ops/norm_gate.py:19-43),
     * y <- y rsqrt(mean(y^2) + eps) w sigmoid(gate); norm_weight NULL = off */
    const float *norm_weight;           /* [V] or NULL */
    float norm_eps;
    const void *output_gate;            /* BF16 [B][H*V] */
    int64_t output_gate_stride_b;
    /* optional, both or neither (then decay_raw / output_gate above may be NULL): the two small
     * projections in front of the gates, raw = BF16(W hidden (+ bias)) (causallsso/model.py:369-374);
     * gate_rank a multiple of 16, at most 128; weights 16-byte aligned; needs the fused norm */
    int32_t gate_rank;
    const void *decay_hidden;           /* BF16 [B][gate_rank] */
    int64_t decay_hidden_stride_b;
    const void *decay_proj_weight;      /* BF16 [H*r][gate_rank] */
    const void *gate_hidden;            /* BF16 [B][gate_rank] */
    int64_t gate_hidden_stride_b;
    const void *gate_proj_weight;       /* BF16 [H*V][gate_rank] */
    const void *gate_proj_bias;         /* BF16 [H*V] or NULL */
} sd_mixer_decode_args;

int sd_mixer_decode_step(const sd_mixer_decode_args *args, void *stream);

/* Bytes of the buffer sd_forward fills for sd_backward. */
size_t sd_saved_bytes(const sd_shape *shape);
size_t sd_forward_scratch_bytes(const sd_shape *shape);
size_t sd_backward_scratch_bytes(const sd_shape *shape);

/* `stream` is a cudaStream_t passed as void* (NULL = legacy default stream). */
int sd_forward(const sd_forward_args *args, void *stream);
int sd_backward(const sd_backward_args *args, void *stream);
int sd_decode_step(const sd_decode_args *args, void *stream);

/*
 * Predictor only: the sub-owner entry oja_residual(target, source, beta, log_decay, query,
 * initial_state) of causallsso/ops/residual_frame/predictor.py:285-305 (forward :32-87,
 * reverse :129-282).  `source` and `query` are taken as they are (the reference passes the
 * L2-normalised panels; nothing is normalised here and their gradients are the gradients of
 * the rows themselves).  Outputs: frame_action = C_t^T query accumulated through the chunk
 * (what the operator adds to k^ to form the primal address) and update = Delta, both BF16
 * contiguous [B,T,H,r], and the final predictor state.  Workspace sizes are those of the
 * full operator for the same shape with V = r (sd_saved_bytes, sd_forward_scratch_bytes,
 * sd_backward_scratch_bytes); shape.V is ignored.
 */
typedef struct {
    sd_shape shape;
    sd_operand target, source, query;   /* BF16, width r */
    sd_operand beta;                    /* FP32, width 1 (geometry rate per token) */
    sd_operand log_decay;               /* FP32, width r */
    const float *C0;                    /* [B,H,r,r] or NULL */
    void *frame_action, *update;        /* out BF16 [B,T,H,r] contiguous */
    float *C_T;                         /* out or NULL */
    void *saved;  size_t saved_bytes;
    void *scratch; size_t scratch_bytes;
    const unsigned char *valid_mask, *reset_mask;
} sd_predictor_forward_args;

typedef struct {
    sd_shape shape;
    sd_operand target, source, query, beta, log_decay;
    const void *frame_action;           /* what the forward call returned */
    const void *d_frame_action;         /* BF16 [B,T,H,r] contiguous or NULL */
    const void *d_update;               /* BF16 [B,T,H,r] contiguous or NULL */
    const float *dC_T;                  /* or NULL */
    const void *saved; size_t saved_bytes;
    void *scratch; size_t scratch_bytes;
    void *dtarget, *dsource, *dquery;   /* out BF16 [B,T,H,r] contiguous */
    float *dbeta;                       /* out FP32 [B,T,H] */
    float *dlog_decay;                  /* out FP32 [B,T,H,r] */
    float *dC0;                         /* out or NULL */
    const unsigned char *valid_mask, *reset_mask;
} sd_predictor_backward_args;

int sd_predictor_forward(const sd_predictor_forward_args *args, void *stream);
int sd_predictor_backward(const sd_predictor_backward_args *args, void *stream);

/*
 * sd_forward_static -- forward pass for callers that are not allowed to
 * allocate device memory.  It has no counterpart in the upstream project.
 *
 * Who needs it: a serving loop that has handed all device memory to its own
 * arena, code that runs while a stream is being captured, or a plugin host
 * whose rules forbid cudaMalloc inside an operator -- such callers cannot
 * produce the `saved` and `scratch` buffers sd_forward asks for.  Here the
 * library brings its own: one fixed device array of SD_STATIC_WORKSPACE_BYTES
 * that every GPU loading the library holds until the process exits.  The
 * caller passes inputs, outputs and states exactly as for sd_forward; the
 * fields `saved`, `saved_bytes`, `scratch`, `scratch_bytes` are ignored.
 *
 * Limit: sd_saved_bytes(shape) + sd_forward_scratch_bytes(shape) must not
 * exceed SD_STATIC_WORKSPACE_BYTES, i.e. B*H*ceil(T/64) <= 54 chunk tasks of
 * about 600 KiB each (for example B=1, H=8, T<=384).  Larger shapes are refused with
 * SD_ERR_STATIC_WORKSPACE_EXCEEDED before anything is launched.
 *
 * The call itself never calls cudaMalloc, cudaFree or any allocating routine.
 * The first call on each device looks up the array's device address (with
 * that device current); make that first call before starting a stream
 * capture.  All calls on a device share the one array: two calls whose
 * kernels may overlap on the GPU (different streams) race on it -- keep them
 * on one stream or order them yourself.  Nothing in the array needs zeroing
 * between calls, and what it holds afterwards is not a usable `saved` buffer
 * for sd_backward once another call has run.
 */
#define SD_STATIC_WORKSPACE_BYTES (32u * 1024u * 1024u)
int sd_forward_static(const sd_forward_args *args, void *stream);

/* Number of kernels one call launches for this shape (for accounting). */
int sd_forward_launches(const sd_shape *shape);
int sd_backward_launches(const sd_shape *shape);

/*
 * Device fault word.  Every wait inside the kernels is bounded; a wait that runs out does
 * not hang the GPU: it stores a code here, the kernel walks to its end, and the results of
 * that launch are undefined.  Codes 1-5 come from the tensor-memory state scan: 1 = the first
 * contraction of a step (X = P + Q St) never completed, 2 = the second (state update),
 * 3 = a step's Q panel never landed, 4 = its R / P panels never landed, 5 = the slot of
 * the R / P panels was never released; codes 6-7 from the tensor-memory output contraction:
 * 6 = its panels never landed, 7 = the contraction never completed.  No upstream counterpart.
 *
 * sd_device_fault waits for the device and returns the word (0 = no fault, -1 = the device
 * could not be read); the word stays set until sd_device_fault_clear() (which also waits
 * for the device) puts it back to 0.  Callers that already synchronise -- the end of a
 * training step, of a generation loop, of a benchmark -- should read it there.
 */
int sd_device_fault(void);
int sd_device_fault_clear(void);

/*
 * Introspection for tests: offset and size of a named intermediate panel
 * inside the saved (which = 0), forward-scratch (1) or backward-scratch (2)
 * buffer.  Returns SD_ERR_INVALID_ARGUMENT for an unknown name.
 */
int sd_panel_info(const sd_shape *shape, int which, const char *name,
                  size_t *offset, size_t *bytes);
/* Element layout of that panel: FP32 0 = [64][128] panel, 1 = [64][64] matrix,
 * 2 = [128][128] state, 3 = [128] vector; BF16 4 = panel, 5 = matrix, 6 = state.
 * Negative = unknown name. */
int sd_panel_kind(const sd_shape *shape, int which, const char *name);

/* ------------------------------------------------------------------------
 * Mixer glue on either side of the recurrence (all device pointers, BF16
 * activations, FP32 parameters; every call is asynchronous on `stream`).
 *
 * sd_conv4_silu_*   depthwise causal convolution of width 4 + SiLU with a carried
 *                   [B,D,3] state: causallsso/model.py:110-164 (_packed_conv; the
 *                   CUDA branch calls the causal-conv1d extension, :119-136)
 * sd_kda_gate_*     log_decay = -exp(A[h]) * softplus(raw + bias[h][c]):
 *                   causallsso/model.py:375-390 (fused_kda_gate / its CPU formula)
 * sd_norm_gate_*    y = x * rsqrt(mean(x^2)+eps) * w * sigmoid(gate) over rows of
 *                   width V <= 128: causallsso/ops/norm_gate.py:19-43,162-217
 */
typedef struct {
    int32_t B, T, D;
    const void *x;                 /* BF16 [B,T,D] view, unit inner stride */
    int64_t x_stride_b, x_stride_t;
    const float *weight;           /* [D][4], tap 3 multiplies the current token */
    const void *initial_state;     /* BF16 [B][D][3] or NULL (= zeros) */
    void *y;                       /* out BF16 [B,T,D] contiguous */
    void *final_state;             /* out BF16 [B][D][3] or NULL */
    /* one byte per (batch, token), either may be NULL: an invalid token gives zero output and
     * leaves the window untouched, a reset on a valid token empties the window first
     * (the masked loop of causallsso/model.py:146-164; upstream's CUDA branch repacks the
     * batch into segments instead, model.py:166-273) */
    const unsigned char *valid_mask;
    const unsigned char *reset_mask;
} sd_conv4_forward_args;

typedef struct {
    int32_t B, T, D;
    const void *x;
    int64_t x_stride_b, x_stride_t;
    const float *weight;
    const void *initial_state;
    const void *dy;                /* BF16 [B,T,D] contiguous */
    void *dx;                      /* out BF16 [B,T,D] contiguous */
    float *dweight;                /* out [D][4] */
    void *dinitial_state;          /* out BF16 [B][D][3] or NULL */
    void *scratch;                 /* sd_conv4_backward_scratch_bytes */
    size_t scratch_bytes;
    const unsigned char *valid_mask;   /* as in the forward call */
    const unsigned char *reset_mask;
} sd_conv4_backward_args;

size_t sd_conv4_backward_scratch_bytes(int32_t B, int32_t T, int32_t D);
int sd_conv4_silu_forward(const sd_conv4_forward_args *args, void *stream);
int sd_conv4_silu_backward(const sd_conv4_backward_args *args, void *stream);

typedef struct {
    int64_t rows;                  /* B*T */
    int32_t H, r;                  /* H*r <= 1024 */
    const void *raw;               /* BF16 [rows][H][r] contiguous */
    const float *log_rate;         /* A [H] */
    const float *bias;             /* [H][r] */
    float *log_decay;              /* out (forward) FP32 [rows][H][r] */
    const float *dlog_decay;       /* backward input */
    void *draw;                    /* backward out BF16 [rows][H][r] */
    float *dlog_rate;              /* backward out [H] */
    float *dbias;                  /* backward out [H][r] */
    void *scratch;                 /* backward: sd_kda_gate_backward_scratch_bytes */
    size_t scratch_bytes;
} sd_kda_gate_args;

size_t sd_kda_gate_backward_scratch_bytes(int64_t rows, int32_t H, int32_t r);
int sd_kda_gate_forward(const sd_kda_gate_args *args, void *stream);
int sd_kda_gate_backward(const sd_kda_gate_args *args, void *stream);

typedef struct {
    int64_t rows;                  /* B*T*H */
    int32_t V;                     /* <= 128 */
    float eps;
    const void *x, *gate;          /* BF16 [rows][V] contiguous */
    const float *weight;           /* [V] */
    void *y;                       /* out (forward) BF16 [rows][V] */
    const void *dy;                /* backward input BF16 */
    void *dx, *dgate;              /* backward out BF16 */
    float *dweight;                /* backward out [V] */
    void *scratch;                 /* backward: sd_norm_gate_backward_scratch_bytes */
    size_t scratch_bytes;
} sd_norm_gate_args;

size_t sd_norm_gate_backward_scratch_bytes(int64_t rows, int32_t V);
int sd_norm_gate_forward(const sd_norm_gate_args *args, void *stream);
int sd_norm_gate_backward(const sd_norm_gate_args *args, void *stream);

const char *sd_status_string(int status);
int sd_version(void);
/* Tokens per chunk of the chunked scan (a private tuning constant upstream). */
int sd_chunk_tokens(void);

#ifdef __cplusplus
}
#endif
#endif /* SOLVEDELTA_B200_H */
