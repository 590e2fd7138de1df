// Shared device helpers of the SolveDelta chunk kernels (sm_100a).
//
// A "panel" is the FP32 image of one chunk of one (batch, head) stream:
// CL token rows by DP channels.  In global memory panels are dense
// [CL][DP]; in shared memory rows are padded to LDP floats.  r and V may be
// smaller than DP: the extra channels are zero on load and skipped on store,
// so one instantiation serves every width up to 128.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sd {

constexpr int CL = 64;        // tokens per chunk
constexpr int DP = 128;       // padded channel width
constexpr int LDP = DP + 4;   // shared-memory row pitch of a panel
constexpr int LDA = CL + 4;   // row pitch of a CL x CL matrix
constexpr int LDH = CL + 4;   // row pitch of a [DP][CL] half state (transposed read)
constexpr int NTHREADS = 512;            // threads of a chunk CTA (16 warps)
constexpr int ROWS_PER_PASS = NTHREADS / 16;  // token rows covered by one row-wise pass
constexpr int ROW_PASSES = CL / ROWS_PER_PASS;
constexpr int NT128 = DP / 32;            // 8-column MMA tiles per warp for a CL x DP output
constexpr int NT64 = CL / 32;             // ... for a CL x CL output
constexpr float RHO = 0.625f; // radius of the residual-local frame

constexpr int SLOT_FLOATS = (CL * LDP > DP * LDH) ? CL * LDP : DP * LDH;
constexpr int MAT_FLOATS = CL * LDA;
constexpr size_t SLOT_BYTES = size_t(SLOT_FLOATS) * 4;
constexpr size_t MAT_BYTES = size_t(MAT_FLOATS) * 4;

struct Operand {
    const void* ptr;
    long long sb, st, sh;  // element strides
    int vec;               // 1 when 16-byte vector access is legal
};

// A reset token starts from the zero state.  It is carried as RESET_NATS of extra forgetting in
// the token's log decay: exp(-RESET_NATS) is exactly zero in FP32, so every decay-weighted term
// that would cross the reset vanishes -- pair entries, the carried-in state, the carried-out
// contributions of earlier tokens, the chunk's retention -- while terms inside one segment only
// see differences of the prefix, in which the offset cancels.
constexpr float RESET_NATS = 128.f;

struct Geometry {
    int B, T, H, r, V, NC;  // NC = chunks per stream
    const unsigned char* valid;  // [B][T] bytes, 0 = token takes no part (null: every token is valid)
    const unsigned char* reset;  // [B][T] bytes, 1 = token starts from the zero state (null: none)
#ifdef SD_DIAGNOSTICS
    long long* dbg;         // phase clock stamps of one CTA (null = off); profiling build only
    int dbg_block;
#endif
};

// Profiling build (-DSD_DIAGNOSTICS): thread 0 of one chosen CTA records the SM clock at a phase
// boundary.  The shipped build compiles the stamps out.
#ifdef SD_DIAGNOSTICS
#define SD_PHASE(g, ph)                                                                   \
    do {                                                                                  \
        if ((g).dbg != nullptr && (int)blockIdx.x == (g).dbg_block && threadIdx.x == 0 && \
            (ph) < 16)                                                                    \
            (g).dbg[(ph)] = clock64();                                                    \
        ++(ph);                                                                           \
    } while (0)
#else
#define SD_PHASE(g, ph) do { (void)(ph); } while (0)
#endif

// The chunk a CTA works on.  MASKED selects, at compile time, whether token masks exist at all: the
// unmasked instantiation of every kernel tests `i < nvalid` and carries no mask words.
template <bool MASKED>
struct ChunkT {
    int s, c, b, hh, t0, nvalid;
    long long gi;  // global chunk index s * NC + c
    unsigned long long vm;  // MASKED: bit i = token row i exists and is valid
    unsigned long long rm;  // MASKED: bit i = token row i is a (valid) reset token
    __device__ __forceinline__ unsigned long long valid_rows() const {
        return MASKED ? vm : (nvalid >= CL ? ~0ull : ((1ull << nvalid) - 1ull));
    }
    __device__ __forceinline__ unsigned long long reset_rows() const { return MASKED ? rm : 0ull; }
    __device__ __forceinline__ bool ok(int i) const { return MASKED ? ((vm >> i) & 1ull) != 0ull : i < nvalid; }
    __device__ __forceinline__ bool rst(int i) const { return MASKED ? ((rm >> i) & 1ull) != 0ull : false; }
    // what the exclusive prefix E_i = G_{i-1} of a reset row still lacks: the reset belongs to row i itself
    __device__ __forceinline__ float eoff(int i) const { return rst(i) ? RESET_NATS : 0.f; }
};
typedef ChunkT<false> Chunk;

template <bool MASKED>
__device__ __forceinline__ ChunkT<MASKED> chunk_of(const Geometry& g, int idx) {
    ChunkT<MASKED> ch;
    ch.gi = idx;
    ch.s = idx / g.NC;
    ch.c = idx - ch.s * g.NC;
    ch.b = ch.s / g.H;
    ch.hh = ch.s - ch.b * g.H;
    ch.t0 = ch.c * CL;
    int left = g.T - ch.t0;
    ch.nvalid = left < CL ? left : CL;
    ch.vm = 0ull;
    ch.rm = 0ull;
    if (MASKED) {
        // every warp reads the chunk's 64 mask bytes (all threads call chunk_of together); the ballots are
        // warp-uniform values
        const int lane = threadIdx.x & 31;
        const unsigned char* vp = g.valid ? g.valid + (long long)ch.b * g.T + ch.t0 : nullptr;
        const unsigned char* rp = g.reset ? g.reset + (long long)ch.b * g.T + ch.t0 : nullptr;
        const bool v0 = lane < ch.nvalid && (vp == nullptr || vp[lane] != 0);
        const bool v1 = lane + 32 < ch.nvalid && (vp == nullptr || vp[lane + 32] != 0);
        const bool r0 = v0 && rp != nullptr && rp[lane] != 0;
        const bool r1 = v1 && rp != nullptr && rp[lane + 32] != 0;
        ch.vm = (unsigned long long)__ballot_sync(0xffffffffu, v0) |
                ((unsigned long long)__ballot_sync(0xffffffffu, v1) << 32);
        ch.rm = (unsigned long long)__ballot_sync(0xffffffffu, r0) |
                ((unsigned long long)__ballot_sync(0xffffffffu, r1) << 32);
    }
    return ch;
}

__device__ __forceinline__ float* panel_ptr(float* base, long long gi) {
    return base + gi * (long long)(CL * DP);
}
__device__ __forceinline__ const float* panel_ptr(const float* base, long long gi) {
    return base + gi * (long long)(CL * DP);
}
__device__ __forceinline__ float* mat_ptr(float* base, long long gi) {
    return base + gi * (long long)(CL * CL);
}
__device__ __forceinline__ const float* mat_ptr(const float* base, long long gi) {
    return base + gi * (long long)(CL * CL);
}
__device__ __forceinline__ float* state_ptr(float* base, long long gi) {
    return base + gi * (long long)(DP * DP);
}
__device__ __forceinline__ const float* state_ptr(const float* base, long long gi) {
    return base + gi * (long long)(DP * DP);
}

// 1 / (1 + exp(-x)) with the fast reciprocal (2 ulp): exp(-x) = inf gives exactly 0.
__device__ __forceinline__ float sigmoidf_(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// ---- half-warp (16 lanes = one token row) reductions ---------------------
__device__ __forceinline__ float row_sum16(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v;
}

// ---- strided BF16 / FP32 row access --------------------------------------
template <class CH>
__device__ __forceinline__ const __nv_bfloat16* row_bf16(const Operand& op, const CH& ch, int i) {
    return reinterpret_cast<const __nv_bfloat16*>(op.ptr) + ch.b * op.sb + (long long)(ch.t0 + i) * op.st +
           ch.hh * op.sh;
}
template <class CH>
__device__ __forceinline__ const float* row_f32(const Operand& op, const CH& ch, int i) {
    return reinterpret_cast<const float*>(op.ptr) + ch.b * op.sb + (long long)(ch.t0 + i) * op.st + ch.hh * op.sh;
}

// Eight consecutive channels of a BF16 row; channels >= width read as zero.
// FAST: every operand is 16-byte aligned and the widths are multiples of 8, so the
// access is one predicated vector load with no control flow around it -- the
// compiler can then keep many independent loads in flight.
template <bool FAST>
__device__ __forceinline__ void load8_bf16(const __nv_bfloat16* row, int c0, int width, int vec, bool valid,
                                           float (&x)[8]) {
    if (FAST) {
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (valid && c0 < width) raw = *reinterpret_cast<const uint4*>(row + c0);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float2 f = __bfloat1622float2(p[e]);
            x[2 * e] = f.x;
            x[2 * e + 1] = f.y;
        }
        return;
    }
    if (!valid || c0 >= width) {
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = 0.f;
        return;
    }
    if (vec && c0 + 8 <= width) {
        uint4 raw = *reinterpret_cast<const uint4*>(row + c0);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float2 f = __bfloat1622float2(p[e]);
            x[2 * e] = f.x;
            x[2 * e + 1] = f.y;
        }
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = (c0 + e < width) ? __bfloat162float(row[c0 + e]) : 0.f;
    }
}

template <bool FAST>
__device__ __forceinline__ void load8_f32(const float* row, int c0, int width, int vec, bool valid, float (&x)[8]) {
    if (FAST) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (valid && c0 < width) {
            a = *reinterpret_cast<const float4*>(row + c0);
            b = *reinterpret_cast<const float4*>(row + c0 + 4);
        }
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
        x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        return;
    }
    if (!valid || c0 >= width) {
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = 0.f;
        return;
    }
    if (vec && c0 + 8 <= width) {
        float4 a = *reinterpret_cast<const float4*>(row + c0);
        float4 b = *reinterpret_cast<const float4*>(row + c0 + 4);
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
        x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = (c0 + e < width) ? row[c0 + e] : 0.f;
    }
}

// Contiguous outputs [B,T,H,width]: eight channels of one row.
template <bool FAST, class CH>
__device__ __forceinline__ void store8_bf16(void* base, const Geometry& g, const CH& ch, int i, int c0,
                                            int width, const float (&x)[8]) {
    if (FAST) {
        __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(base) +
                             (((long long)ch.b * g.T + ch.t0 + i) * g.H + ch.hh) * (long long)width;
        uint4 raw;
        __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) p[e] = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
        if (!ch.ok(i)) raw = make_uint4(0u, 0u, 0u, 0u);   // a masked token: exact zeros
        if (i < ch.nvalid && c0 < width) *reinterpret_cast<uint4*>(row + c0) = raw;
        return;
    }
    if (i >= ch.nvalid || c0 >= width) return;
    if (!ch.ok(i)) {
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (c0 + e < width)
                (reinterpret_cast<__nv_bfloat16*>(base) +
                 (((long long)ch.b * g.T + ch.t0 + i) * g.H + ch.hh) * (long long)width)[c0 + e] = __float2bfloat16_rn(0.f);
        return;
    }
    __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(base) +
                         (((long long)ch.b * g.T + ch.t0 + i) * g.H + ch.hh) * (long long)width;
    if ((width & 7) == 0) {
        uint4 raw;
        __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) p[e] = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
        *reinterpret_cast<uint4*>(row + c0) = raw;
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (c0 + e < width) row[c0 + e] = __float2bfloat16_rn(x[e]);
    }
}

// ---- L2 prefetch of what a later phase of the same CTA reads from HBM --------
__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
// a dense region of `bytes` bytes (128-byte lines), all threads of the CTA
__device__ __forceinline__ void prefetch_region(const void* base, int bytes) {
    const char* b = reinterpret_cast<const char*>(base);
    for (int off = threadIdx.x * 128; off < bytes; off += NTHREADS * 128) prefetch_l2(b + off);
}
// the CL token rows of a strided operand chunk (row_bytes per row)
template <class CH>
__device__ __forceinline__ void prefetch_rows(const Operand& op, const CH& ch, int elem_bytes, int row_bytes) {
    const int lines = (row_bytes + 127) / 128;
    for (int idx = threadIdx.x; idx < CL * lines; idx += NTHREADS) {
        const int i = idx / lines, l = idx - i * lines;
        if (ch.ok(i)) {
            const char* row = reinterpret_cast<const char*>(op.ptr) +
                              (ch.b * op.sb + (long long)(ch.t0 + i) * op.st + ch.hh * op.sh) * elem_bytes;
            prefetch_l2(row + l * 128);
        }
    }
}

// ---- dense panel movement -------------------------------------------------
__device__ __forceinline__ void s2g_panel(float* g, const float* sm) {
    for (int idx = threadIdx.x; idx < CL * (DP / 4); idx += NTHREADS) {
        int i = idx >> 5, c4 = (idx & 31) << 2;
        *reinterpret_cast<float4*>(g + i * DP + c4) = *reinterpret_cast<const float4*>(sm + i * LDP + c4);
    }
}
// ---- TF32 tensor-core contraction on shared-memory operands --------------
__device__ __forceinline__ uint32_t f2tf32(float x) {
    uint32_t y;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float round_tf32(float x) { return __uint_as_float(f2tf32(x)); }
// a [CL][DP] shared panel to global memory, rounded to TF32 on the way
__device__ __forceinline__ void s2g_panel_tf32(float* g, const float* sm) {
    for (int idx = threadIdx.x; idx < CL * (DP / 4); idx += NTHREADS) {
        int i = idx >> 5, c4 = (idx & 31) << 2;
        float4 v = *reinterpret_cast<const float4*>(sm + i * LDP + c4);
        *reinterpret_cast<float4*>(g + i * DP + c4) =
            make_float4(round_tf32(v.x), round_tf32(v.y), round_tf32(v.z), round_tf32(v.w));
    }
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NTW>
__device__ __forceinline__ void acc_zero(float (&acc)[NTW][4]) {
#pragma unroll
    for (int n = 0; n < NTW; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
}

// acc[16 x 8*NTW] += A[r0.., kbeg..kend) * B[kbeg..kend), n0..), one warp.
// fa(i, k) and fb(k, n) return floats (any shared-memory indexing).
template <int NTW, class FA, class FB>
__device__ __forceinline__ void warp_mma(float (&acc)[NTW][4], int r0, int n0, int kbeg, int kend, FA fa, FB fb) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll 2
    for (int kk = kbeg; kk < kend; kk += 8) {
        uint32_t a0 = f2tf32(fa(r0 + g, kk + t));
        uint32_t a1 = f2tf32(fa(r0 + g + 8, kk + t));
        uint32_t a2 = f2tf32(fa(r0 + g, kk + t + 4));
        uint32_t a3 = f2tf32(fa(r0 + g + 8, kk + t + 4));
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
            uint32_t b0 = f2tf32(fb(kk + t, n0 + nt * 8 + g));
            uint32_t b1 = f2tf32(fb(kk + t + 4, n0 + nt * 8 + g));
            mma_tf32(acc[nt], a0, a1, a2, a3, b0, b1);
        }
    }
}

// fe(i, j, v0, v1): element (i, j) = v0 and (i, j + 1) = v1, j even.
template <int NTW, class FE>
__device__ __forceinline__ void warp_epi(float (&acc)[NTW][4], int r0, int n0, FE fe) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nt = 0; nt < NTW; ++nt) {
        int j = n0 + nt * 8 + 2 * t;
        fe(r0 + g, j, acc[nt][0], acc[nt][1]);
        fe(r0 + g + 8, j, acc[nt][2], acc[nt][3]);
    }
}

// Warp tiling of a CL x N output over the 16 warps of a chunk CTA
// (4 row tiles x 4 column quarters).
template <int N>
struct Tile64 {
    static constexpr int NTW = N / 32;
    __device__ static __forceinline__ int r0() { return ((threadIdx.x >> 5) & 3) * 16; }
    __device__ static __forceinline__ int n0() { return (threadIdx.x >> 7) * (N / 4); }
};

// ---- chunk-local gate algebra ----------------------------------------------
// In place: sG[i][c] <- sum_{j<=i} g[j][c].  Call with all threads; needs a
// __syncthreads() before and after.
__device__ __forceinline__ void chunk_cumsum(float* sG) {
    if (threadIdx.x < DP) {
        float run = 0.f;
        float* p = sG + threadIdx.x;
#pragma unroll 8
        for (int i = 0; i < CL; ++i) {
            run += p[i * LDP];
            p[i * LDP] = run;
        }
    }
}

// Loads a BF16 operand chunk, L2-normalises every row and stores it as FP32.
// rstd (may be null) receives 1/|x| per row.  UNIT: the rows already are unit vectors and are taken as they
// are (the predictor-only entry, whose caller normalises).
template <bool FAST, bool UNIT = false, class CH>
__device__ __forceinline__ void load_norm_panel(const Operand& op, const CH& ch, int width, float* sm,
                                                float* rstd) {
    const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
#pragma unroll
    for (int p = 0; p < ROW_PASSES; ++p) {
        int i = lr + ROWS_PER_PASS * p;
        float x[8];
        load8_bf16<FAST>(row_bf16(op, ch, i), c0, width, op.vec, ch.ok(i), x);
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(x[e], x[e], ss);
        ss = row_sum16(ss);
        float rs = UNIT ? 1.f : rsqrtf(ss + 1e-24f);
#pragma unroll
        for (int e = 0; e < 8; ++e) sm[i * LDP + c0 + e] = x[e] * rs;
        if (rstd != nullptr && (threadIdx.x & 15) == 0) rstd[i] = rs;
    }
}

template <bool FAST, class CH>
__device__ __forceinline__ void load_raw_panel(const Operand& op, const CH& ch, int width, float* sm) {
    const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
#pragma unroll
    for (int p = 0; p < ROW_PASSES; ++p) {
        int i = lr + ROWS_PER_PASS * p;
        float x[8];
        load8_bf16<FAST>(row_bf16(op, ch, i), c0, width, op.vec, ch.ok(i), x);
#pragma unroll
        for (int e = 0; e < 8; ++e) sm[i * LDP + c0 + e] = x[e];
    }
}

template <bool FAST, class CH>
__device__ __forceinline__ void load_f32_panel(const Operand& op, const CH& ch, int width, float* sm) {
    const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
#pragma unroll
    for (int p = 0; p < ROW_PASSES; ++p) {
        int i = lr + ROWS_PER_PASS * p;
        float x[8];
        load8_f32<FAST>(row_f32(op, ch, i), c0, width, op.vec, ch.ok(i), x);
#pragma unroll
        for (int e = 0; e < 8; ++e) sm[i * LDP + c0 + e] = x[e];
    }
}

template <class CH>
__device__ __forceinline__ void load_gamma(const Operand& op, const CH& ch, float* sg) {
    if (threadIdx.x < CL) {
        int i = threadIdx.x;
        sg[i] = ch.ok(i) ? *row_f32(op, ch, i) : 0.f;
    }
}

}  // namespace sd
