// The forward chunk-state scan on the fifth-generation tensor cores (tcgen05).
//
// Same recurrence, ScanParams and launch grid as k_state_scan:
//     X  = P + Q * St ;  checkpoint St ;  St = diag(lam) St + R^T X
// A CTA carries a [DP][NS] column slice of one stream's state.  The slice
// lives in tensor memory as the accumulator of the update contraction (lane =
// state row p, column = slice column c); the step's X is a second
// accumulator, held transposed (lane = slice column, column = token):
//     X^T[c][tok] = sum_p St[p][c] * Q[tok][p]       M=128 (64 used) N=64 K=128
//     St [p][c]  += sum_t R[tok][p] * X[tok][c]      M=128           N=64 K=64
// All four operands are K-major in shared memory, in the unswizzled canonical
// layout of 8 x 16-byte core matrices (the first contraction's M is padded to
// 128: rows 64..127 of its A operand alias whatever follows in shared memory
// and only feed accumulator lanes nobody reads).  Q [tok][p] arrives by ONE
// tiled TMA load per chunk (cp.async.bulk.tensor.4d, completion counted on an
// mbarrier): the tensor map lists the 16-byte K-chunk as a dimension of its own,
// so the panel lands as [K-chunk][row][4 elements], which is the canonical layout.  X^T is written by the thread that holds the row after
// tcgen05.ld, four consecutive tokens to a 16-byte chunk.  The state, held by
// rows, is written element by element into the transposed operand, with the
// K-chunk pitch padded to 144 bytes so that a warp's 32 rows hit 32 banks.
// R [tok][p], whose contraction index is the slow one in global memory, is
// landed as it lies by a tiled TMA load (with the CTA's slice of P) and turned
// through registers: a thread reads columns of it, one lane per column, and
// writes each as 16-byte chunks of one operand row (the warps without X^T
// rows do this, two columns per thread).  The decay
// diag(lam) is one scalar per thread, applied on the way back into tensor
// memory; checkpoints and X go to global memory from the same registers.
// Operands are rounded to TF32 (round to nearest) before the tensor core,
// which would truncate, sees them: the state, X and R in registers here, Q by
// the kernels that write the Q panels.
//
// Every mbarrier wait is bounded: a wait that runs out raises the fault word
// the host reads back, the thread stops waiting for the rest of the launch,
// and the kernel still walks to its end and frees its tensor memory.
#pragma once
#include <cuda.h>   // CUtensorMap (types only: the encoder is reached through the runtime's driver entry point)

#include "sd_scan.cuh"

namespace sd {

constexpr int TC_PARTS = 2;               // warps per lane quarter: each takes 64/TC_PARTS columns (or tokens)
constexpr int TC_N = 64 / TC_PARTS;        // columns of the state slice, or tokens of X^T, per thread
constexpr int TC_THREADS = 128 * TC_PARTS; // lane quarter = warp % 4, part = warp / 4
constexpr int TC_TMEM_COLS = 128;         // 64 state-slice columns + 64 X^T columns
constexpr int TC_X_COL = SCAN_NS;         // first tensor-memory column of X^T
constexpr unsigned TC_CORE = 128;         // bytes of one 8 x 16-byte core matrix
constexpr unsigned TC_Q_LBO = CL * 16;               // Q landed by TMA: K-chunk pitch (all 64 rows of one 16-byte chunk)
constexpr unsigned TC_Q_SBO = 8 * 16;                // ... and the pitch of its 8-row groups
constexpr unsigned TC_KT_SBO = (CL / 4) * TC_CORE;  // K = tokens (X, R): bytes between 8-row groups
constexpr unsigned TC_PANEL_BYTES = CL * DP * 4;    // one [CL][DP] or [DP][CL] operand
constexpr unsigned TC_S_LBO = TC_CORE + 16;         // padded K-chunk pitch of the transposed state operand
constexpr unsigned TC_S_SBO = (DP / 4) * TC_S_LBO;  // its bytes between 8-row groups
constexpr unsigned TC_S_BYTES = (SCAN_NS / 8) * TC_S_SBO;   // the 64 rows that are written
constexpr unsigned TC_X_BYTES = SCAN_NS * CL * 4;
// Q ring, state operand, X operand, R operand.  The padded A operand of the first contraction reaches
// 2 * TC_S_BYTES past the start of the state operand, which must stay inside this allocation.
constexpr size_t SCAN_TC_OPERAND_BYTES = size_t(2) * TC_PANEL_BYTES + TC_S_BYTES + TC_X_BYTES + TC_PANEL_BYTES;
constexpr unsigned TC_RAW_P_BYTES = CL * SCAN_NS * 4;   // the P slice as it lies, [CL][NS]
// ... followed by R as it lies ([CL][DP]) and the P slice, both landed by TMA one step ahead
constexpr size_t SCAN_TC_SMEM_BYTES = SCAN_TC_OPERAND_BYTES + TC_PANEL_BYTES + TC_RAW_P_BYTES;
static_assert(2 * TC_S_BYTES <= TC_S_BYTES + TC_X_BYTES + TC_PANEL_BYTES, "padded operand rows leave the allocation");
constexpr int TC_WAIT_LIMIT = 1 << 20;    // polls of one mbarrier before the wait is given up

__device__ __forceinline__ unsigned tc_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// Shared-memory matrix descriptor, no swizzle: start address, leading and stride byte offsets in 16-byte units.
__device__ __forceinline__ unsigned long long tc_desc(unsigned addr, unsigned lbo, unsigned sbo) {
    return (unsigned long long)((addr >> 4) & 0x3FFF) | ((unsigned long long)((lbo >> 4) & 0x3FFF) << 16) |
           ((unsigned long long)((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
// Instruction descriptor: FP32 accumulator, TF32 operands, both K-major, M = 128.
__device__ __forceinline__ unsigned tc_idesc(int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(n >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void tc_mma(unsigned d_tmem, unsigned long long da, unsigned long long db, unsigned idesc,
                                       unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Bounded wait on one phase of an mbarrier; false when the limit ran out.
__device__ __forceinline__ bool tc_wait(unsigned bar, unsigned parity) {
    for (int it = 0; it < TC_WAIT_LIMIT; ++it) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// 32 consecutive 32-bit tensor-memory columns of this thread's lane.
__device__ __forceinline__ void tc_ld32(unsigned taddr, float* r) {
    unsigned* u = reinterpret_cast<unsigned*>(r);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31}, [%32];"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
          "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
          "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
          "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tc_st32(unsigned taddr, const float* r) {
    const unsigned* u = reinterpret_cast<const unsigned*>(r);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31};" ::"r"(u[0]),
        "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]), "r"(u[8]), "r"(u[9]), "r"(u[10]),
        "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]), "r"(u[16]), "r"(u[17]), "r"(u[18]), "r"(u[19]),
        "r"(u[20]), "r"(u[21]), "r"(u[22]), "r"(u[23]), "r"(u[24]), "r"(u[25]), "r"(u[26]), "r"(u[27]), "r"(u[28]),
        "r"(u[29]), "r"(u[30]), "r"(u[31]), "r"(taddr)
        : "memory");
}
// 16-column forms of the two moves above
__device__ __forceinline__ void tc_ld16(unsigned taddr, float* r) {
    unsigned* u = reinterpret_cast<unsigned*>(r);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
          "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tc_st16(unsigned taddr, const float* r) {
    const unsigned* u = reinterpret_cast<const unsigned*>(r);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};" ::"r"(u[0]),
        "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]), "r"(u[8]), "r"(u[9]), "r"(u[10]),
        "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]), "r"(taddr)
        : "memory");
}
template <int N>
__device__ __forceinline__ void tc_ld(unsigned taddr, float* r) {
    static_assert(N == 16 || N == 32, "16 or 32 columns per move");
    if (N == 32) tc_ld32(taddr, r); else tc_ld16(taddr, r);
}
template <int N>
__device__ __forceinline__ void tc_st(unsigned taddr, const float* r) {
    static_assert(N == 16 || N == 32, "16 or 32 columns per move");
    if (N == 32) tc_st32(taddr, r); else tc_st16(taddr, r);
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// One full 32-byte sector per thread (256-bit store; the address is 32-byte aligned).
__device__ __forceinline__ void tc_store32(void* g, const unsigned (&w)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(g), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                 "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
}

__device__ __forceinline__ float tc_round(float x) { return __uint_as_float(f2tf32(x)); }

// One tiled TMA load lands the [CL][DP] panel Q of chunk `chunk` as a K-major unswizzled operand:
// the map's dimensions are (4 elements, CL rows, DP/4 K-chunks, chunks), so shared memory receives
// [K-chunk][row][4 elements].  Completion is counted in bytes on `bar`.
__device__ __forceinline__ void tc_load_q(unsigned char* sm, const CUtensorMap* map, int chunk, unsigned bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(TC_PANEL_BYTES) : "memory");
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
            tc_smem(sm)),
        "l"(reinterpret_cast<unsigned long long>(map)), "r"(0), "r"(0), "r"(0), "r"(chunk), "r"(bar)
        : "memory");
}

// Row-major tiled loads (map dimensions: DP columns, CL rows, chunks): all of R, and the CTA's
// NS-column slice of P, both counted on `bar`.
__device__ __forceinline__ void tc_load_rp(unsigned char* sR_raw, unsigned char* sP_raw, const CUtensorMap* rmap,
                                           const CUtensorMap* pmap, int chunk, int col0, unsigned bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                 "r"(TC_PANEL_BYTES + TC_RAW_P_BYTES)
                 : "memory");
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            tc_smem(sR_raw)),
        "l"(reinterpret_cast<unsigned long long>(rmap)), "r"(0), "r"(0), "r"(chunk), "r"(bar)
        : "memory");
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            tc_smem(sP_raw)),
        "l"(reinterpret_cast<unsigned long long>(pmap)), "r"(col0), "r"(0), "r"(chunk), "r"(bar)
        : "memory");
}

// Profiling build only: thread 0 of the first CTA records the SM clock at the phase boundaries of its ninth step.
#ifdef SD_DIAGNOSTICS
#define TC_STAMP(k)                                                                              \
    do {                                                                                         \
        if (dbg != nullptr && blockIdx.x == 0 && tid == 0 && step == 8)                          \
            dbg[k] = clock64();                                                                  \
    } while (0)
#else
#define TC_STAMP(k) do { } while (0)
#endif

__global__ void __launch_bounds__(TC_THREADS, 1) k_state_scan_tc(ScanParams p, const __grid_constant__ CUtensorMap qmap,
                                                                  const __grid_constant__ CUtensorMap rmap,
                                                                  const __grid_constant__ CUtensorMap pmap, int* fault,
                                                                  long long* dbg) {
    extern __shared__ __align__(128) unsigned char tsm[];
    unsigned char* sQ = tsm;                          // [2] B of the first contraction (rows = tokens, K = state rows)
    unsigned char* sS = sQ + 2 * TC_PANEL_BYTES;      // A of the first: slice^T        (rows = slice columns, K = state rows)
    unsigned char* sX = sS + TC_S_BYTES;              // B of the second: X^T           (rows = slice columns, K = tokens)
    unsigned char* sR = sX + TC_X_BYTES;              // A of the second: R^T           (rows = state rows, K = tokens)
    unsigned char* sRraw = tsm + SCAN_TC_OPERAND_BYTES;   // R as it lies, [CL][DP]
    unsigned char* sPraw = sRraw + TC_PANEL_BYTES;        // the P slice as it lies, [CL][NS]
    __shared__ __align__(8) unsigned long long bars[6];   // two contractions, two Q slots, R/P landed, R/P taken
    __shared__ unsigned s_tmem;

    // grid.x = stream * (DP / NS) + column slice (the x dimension has no 65535 limit)
    const int col0 = (blockIdx.x % (DP / SCAN_NS)) * SCAN_NS;
    const int s = blockIdx.x / (DP / SCAN_NS);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quarter = warp & 3, part = warp >> 2;
    // This thread's tensor-memory lane: state row p for the state accumulator and for the R column
    // it turns; slice column c for the X^T accumulator (lanes 0..63 only).
    const int row = quarter * 32 + lane;
    const bool has_x = quarter < 2;
    const long long base = (long long)s * p.NC;

    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&bars[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&bars[1])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&bars[2])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&bars[3])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&bars[4])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tc_smem(&bars[5])), "r"(TC_THREADS));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&s_tmem)),
                     "r"(TC_TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    auto chunk_at = [&](int step) { return base + (p.reverse ? (p.NC - 1 - step) : step); };
    // thread 0 alone moves Q: one tiled load per chunk into the two-slot ring
    auto issue = [&](int step) {
        if (tid == 0 && step < p.NC)
            tc_load_q(sQ + (step & 1) * TC_PANEL_BYTES, &qmap, (int)chunk_at(step), tc_smem(&bars[2 + (step & 1)]));
    };

    // this thread's part of the slice: state row `row`, slice columns [TC_N*part, TC_N*part+TC_N)
    float st[TC_N];
    const int c0 = part * TC_N;
#pragma unroll
    for (int j = 0; j < TC_N; ++j) {
        float v = 0.f;
        int cc = col0 + c0 + j;
        if (p.init != nullptr && row < p.nrows && cc < p.ncols) {
            const float* src = p.init + (long long)s * p.nrows * p.ncols;
            v = p.transposed_io ? src[(long long)cc * p.nrows + row] : src[(long long)row * p.ncols + cc];
        }
        st[j] = v;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tbase = s_tmem;
    const unsigned t_state = tbase + ((unsigned)(quarter * 32) << 16) + c0;
    const unsigned t_x = tbase + ((unsigned)(quarter * 32) << 16) + TC_X_COL + part * TC_N;
    const unsigned bar1 = tc_smem(&bars[0]), bar2 = tc_smem(&bars[1]);
    const unsigned idesc = tc_idesc(SCAN_NS);   // N = 64 for both: tokens, then slice columns
    const unsigned own_row = (row >> 3) * TC_KT_SBO + (row & 7) * 16;                 // this thread's row of sR (and sX)
    const unsigned own_col = (row >> 2) * TC_S_LBO + (row & 3) * 4;                   // its K position in the state operand
    bool alive = true;   // cleared by the first wait that runs out
    issue(0);
    auto issue_rp = [&](int step) {   // single slot: called once every thread is past its reads of the previous one
        if (tid == 0 && step < p.NC)
            tc_load_rp(sRraw, sPraw, &rmap, &pmap, (int)chunk_at(step), col0, tc_smem(&bars[4]));
    };
    issue_rp(0);

    for (int step = 0; step < p.NC; ++step) {
        const long long gi = chunk_at(step);
        const int b = step & 1;
        TC_STAMP(0);
        // next step's Q: its ring slot was last read by the first contraction of the previous step, which every
        // thread has seen complete, so the load gets a whole step to land
        issue(step + 1);
        const float lam = p.lam[gi * DP + row];
        // the slice, transposed and rounded, as this step's A operand
#pragma unroll
        for (int j = 0; j < TC_N; ++j) {
            const int c = c0 + j;
            *reinterpret_cast<float*>(sS + (c >> 3) * TC_S_SBO + (c & 7) * 16 + own_col) = tc_round(st[j]);
        }
        if (alive && !tc_wait(tc_smem(&bars[2 + b]), (step >> 1) & 1)) {   // this step's Q has landed
            alive = false;
            atomicExch(fault, 3);
        }
        tc_fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            const unsigned aS = tc_smem(sS), bQ = tc_smem(sQ + b * TC_PANEL_BYTES);
#pragma unroll
            for (int ks = 0; ks < DP / 8; ++ks)
                tc_mma(tbase + TC_X_COL, tc_desc(aS + ks * 2 * TC_S_LBO, TC_S_LBO, TC_S_SBO),
                       tc_desc(bQ + ks * 2 * TC_Q_LBO, TC_Q_LBO, TC_Q_SBO), idesc, ks > 0);
            tc_commit(bar1);
        }
        __syncwarp();
        TC_STAMP(1);
        // behind the first contraction: this thread's R (and P) values, checkpoints, decay
        // The warps that own X^T rows (lane quarters 0 and 1) take their P values and later run the X
        // epilogue; the other two quarters turn R, for two state rows each (their own and the one 64
        // below).  Both read the panels as TMA landed them: rows of consecutive columns, one lane each.
        if (alive && !tc_wait(tc_smem(&bars[4]), step & 1)) {
            alive = false;
            atomicExch(fault, 4);
        }
        float rv[TC_N], rv2[TC_N], pv[TC_N];
        if (has_x) {
            const float* ps = reinterpret_cast<const float*>(sPraw) + (part * TC_N) * SCAN_NS + row;
#pragma unroll
            for (int j = 0; j < TC_N; ++j) pv[j] = ps[j * SCAN_NS];
        } else {
            const float* rs = reinterpret_cast<const float*>(sRraw) + (part * TC_N) * DP + row;
#pragma unroll
            for (int j = 0; j < TC_N; ++j) rv[j] = rs[j * DP];
#pragma unroll
            for (int j = 0; j < TC_N; ++j) rv2[j] = rs[j * DP - 64];
        }
        // every thread reports that it holds its values; thread 0 then refills the slot for the next step
        // right away instead of after the second barrier (the load gets most of a step to land)
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem(&bars[5])) : "memory");
        if (tid == 0) {
            if (alive && !tc_wait(tc_smem(&bars[5]), step & 1)) {
                alive = false;
                atomicExch(fault, 5);
            }
            issue_rp(step + 1);
        }
        __syncwarp();
        TC_STAMP(2);
        if (p.ckb != nullptr) {
            bf16* ck = p.ckb + gi * (long long)(DP * DP) + row * DP + col0 + c0;
#pragma unroll
            for (int j16 = 0; j16 < TC_N / 16; ++j16) {
                unsigned w[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(st[16 * j16 + 2 * e], st[16 * j16 + 2 * e + 1]);
                    w[e] = *reinterpret_cast<unsigned*>(&h2);
                }
                tc_store32(ck + 16 * j16, w);
            }
        }
        if (p.ck != nullptr) {
            float* ck = state_ptr(p.ck, gi) + row * DP + col0 + c0;
#pragma unroll
            for (int j8 = 0; j8 < TC_N / 8; ++j8) {
                unsigned w[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) w[e] = __float_as_uint(st[8 * j8 + e]);
                tc_store32(ck + 8 * j8, w);
            }
        }
#pragma unroll
        for (int j = 0; j < TC_N; ++j) st[j] *= lam;
        TC_STAMP(3);
        tc_st<TC_N>(t_state, st);
        tc_wait_st();
        TC_STAMP(4);
        // R^T as the second contraction's A operand (the previous step's second contraction has completed)
        if (!has_x) {
#pragma unroll
            for (int j4 = 0; j4 < TC_N / 4; ++j4) {
                float4 v = make_float4(tc_round(rv[4 * j4]), tc_round(rv[4 * j4 + 1]), tc_round(rv[4 * j4 + 2]),
                                       tc_round(rv[4 * j4 + 3]));
                *reinterpret_cast<float4*>(sR + own_row + (part * (TC_N / 4) + j4) * TC_CORE) = v;
                float4 w = make_float4(tc_round(rv2[4 * j4]), tc_round(rv2[4 * j4 + 1]), tc_round(rv2[4 * j4 + 2]),
                                       tc_round(rv2[4 * j4 + 3]));
                *reinterpret_cast<float4*>(sR + own_row - 8 * TC_KT_SBO + (part * (TC_N / 4) + j4) * TC_CORE) = w;
            }
        }

        TC_STAMP(5);
        if (alive && !tc_wait(bar1, step & 1)) {
            alive = false;
            atomicExch(fault, 1);
        }
        tc_fence_after();
        TC_STAMP(6);
        if (has_x) {   // warp-uniform: lanes 0..63 of the X^T accumulator
            float x[TC_N];
            tc_ld<TC_N>(t_x, x);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < TC_N; ++j) x[j] += pv[j];
            if (p.Xb != nullptr) {
                bf16* xb = bpanel_ptr(p.Xb, gi) + (part * TC_N) * DP + col0 + row;
#pragma unroll
                for (int j = 0; j < TC_N; ++j) xb[j * DP] = __float2bfloat16_rn(x[j]);
            } else {
                float* xg = panel_ptr(p.X, gi) + (part * TC_N) * DP + col0 + row;
#pragma unroll
                for (int j = 0; j < TC_N; ++j) __stcg(xg + j * DP, x[j]);
            }
#pragma unroll
            for (int j4 = 0; j4 < TC_N / 4; ++j4) {
                float4 v = make_float4(tc_round(x[4 * j4]), tc_round(x[4 * j4 + 1]), tc_round(x[4 * j4 + 2]),
                                       tc_round(x[4 * j4 + 3]));
                *reinterpret_cast<float4*>(sX + own_row + (part * (TC_N / 4) + j4) * TC_CORE) = v;
            }
        }
        tc_fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            const unsigned aR = tc_smem(sR), bX = tc_smem(sX);
#pragma unroll
            for (int ks = 0; ks < CL / 8; ++ks)
                tc_mma(tbase, tc_desc(aR + ks * 2 * TC_CORE, TC_CORE, TC_KT_SBO),
                       tc_desc(bX + ks * 2 * TC_CORE, TC_CORE, TC_KT_SBO), idesc, 1u);
            tc_commit(bar2);
        }
        __syncwarp();
        TC_STAMP(7);
        TC_STAMP(8);
        if (alive && !tc_wait(bar2, step & 1)) {
            alive = false;
            atomicExch(fault, 2);
        }
        tc_fence_after();
        tc_ld<TC_N>(t_state, st);
        tc_wait_ld();
        TC_STAMP(9);
    }

    if (p.fin != nullptr) {
        float* dst = p.fin + (long long)s * p.nrows * p.ncols;
#pragma unroll
        for (int j = 0; j < TC_N; ++j) {
            int cc = col0 + c0 + j;
            if (row < p.nrows && cc < p.ncols) {
                if (p.transposed_io)
                    dst[(long long)cc * p.nrows + row] = st[j];
                else
                    dst[(long long)row * p.ncols + cc] = st[j];
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(TC_TMEM_COLS));
}

}  // namespace sd
