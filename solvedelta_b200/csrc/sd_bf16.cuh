// BF16 tensor-core contractions on shared-memory panels (ldmatrix + mma.sync
// m16n8k16, FP32 accumulation) and the BF16 panel movers that feed them.
//
// BF16 shared panels use a row pitch of LDB (= DP + 8) elements and matrices /
// half states LDM (= CL + 8): both make the eight 16-byte rows of an ldmatrix
// tile fall into distinct banks.
#pragma once
#include "sd_common.cuh"

namespace sd {

typedef __nv_bfloat16 bf16;

constexpr int LDB = DP + 8;  // pitch of a [CL][DP] BF16 panel
constexpr int LDM = CL + 8;  // pitch of a [CL][CL] BF16 matrix or a [DP][CL] half state
constexpr int BSLOT_ELEMS = CL * LDB;  // one [CL][DP] BF16 panel
constexpr int BMAT_ELEMS = CL * LDM;
constexpr size_t BSLOT_BYTES = size_t(BSLOT_ELEMS) * 2;
constexpr size_t BMAT_BYTES = size_t(BMAT_ELEMS) * 2;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// acc[16 x 8*NTW] += A[r0.., kbeg..kend) * B[kbeg..kend), n0..) for one warp.
//   TA == false: A(i,k) = A[i*lda + k]      TA == true: A(i,k) = A[k*lda + i]
//   TB == false: B(k,n) = B[k*ldb + n]      TB == true: B(k,n) = B[n*ldb + k]
// kbeg, kend multiples of 16; r0 multiple of 16; n0 multiple of 8; NTW even.
template <int NTW, bool TA, bool TB>
__device__ __forceinline__ void warp_mma_bf16(float (&acc)[NTW][4], const bf16* A, int lda, const bf16* B, int ldb,
                                              int r0, int n0, int kbeg, int kend) {
    const int lane = threadIdx.x & 31, j = lane >> 3, rr = lane & 7;
#pragma unroll 2
    for (int kk = kbeg; kk < kend; kk += 16) {
        uint32_t a[4];
        if (!TA) {
            ldsm_x4(a, A + (r0 + (lane & 15)) * lda + kk + (lane >> 4) * 8);
        } else {
            ldsm_x4_t(a, A + (kk + rr + (j >> 1) * 8) * lda + r0 + (j & 1) * 8);
        }
#pragma unroll
        for (int nt = 0; nt < NTW; nt += 2) {
            uint32_t b[4];
            if (TB) {
                ldsm_x4(b, B + (n0 + (nt + (j >> 1)) * 8 + rr) * ldb + kk + (j & 1) * 8);
            } else {
                ldsm_x4_t(b, B + (kk + (j & 1) * 8 + rr) * ldb + n0 + (nt + (j >> 1)) * 8);
            }
            mma_bf16(acc[nt], a, b[0], b[1]);
            mma_bf16(acc[nt + 1], a, b[2], b[3]);
        }
    }
}

// Same contraction with the A operand scaled along k by mvec[k] (BF16, one value
// per k; A not transposed): acc += (A .* mvec) * B.
template <int NTW, bool TB>
__device__ __forceinline__ void warp_mma_bf16_kscale(float (&acc)[NTW][4], const bf16* A, int lda, const bf16* B,
                                                     int ldb, int r0, int n0, int kbeg, int kend, const bf16* mvec) {
    const int lane = threadIdx.x & 31, j = lane >> 3, rr = lane & 7, t = lane & 3;
#pragma unroll 2
    for (int kk = kbeg; kk < kend; kk += 16) {
        uint32_t a[4];
        ldsm_x4(a, A + (r0 + (lane & 15)) * lda + kk + (lane >> 4) * 8);
        {
            // fragment registers 0,1 hold k = kk + 2t (+1), registers 2,3 hold k = kk + 8 + 2t (+1)
            const __nv_bfloat162 mlo = *reinterpret_cast<const __nv_bfloat162*>(mvec + kk + 2 * t);
            const __nv_bfloat162 mhi = *reinterpret_cast<const __nv_bfloat162*>(mvec + kk + 8 + 2 * t);
            __nv_bfloat162* af = reinterpret_cast<__nv_bfloat162*>(a);
            af[0] = __hmul2(af[0], mlo);
            af[1] = __hmul2(af[1], mlo);
            af[2] = __hmul2(af[2], mhi);
            af[3] = __hmul2(af[3], mhi);
        }
#pragma unroll
        for (int nt = 0; nt < NTW; nt += 2) {
            uint32_t b[4];
            if (TB) {
                ldsm_x4(b, B + (n0 + (nt + (j >> 1)) * 8 + rr) * ldb + kk + (j & 1) * 8);
            } else {
                ldsm_x4_t(b, B + (kk + (j & 1) * 8 + rr) * ldb + n0 + (nt + (j >> 1)) * 8);
            }
            mma_bf16(acc[nt], a, b[0], b[1]);
            mma_bf16(acc[nt + 1], a, b[2], b[3]);
        }
    }
}

// ---- movers -----------------------------------------------------------------
__device__ __forceinline__ uint4 pack8_bf16(const float (&x)[8]) {
    uint4 raw;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) p[e] = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
    return raw;
}
__device__ __forceinline__ void unpack8_bf16(const uint4& raw, float (&x)[8]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        float2 f = __bfloat1622float2(p[e]);
        x[2 * e] = f.x;
        x[2 * e + 1] = f.y;
    }
}
__device__ __forceinline__ void store8_bsm(bf16* sm, int i, int c0, const float (&x)[8]) {
    *reinterpret_cast<uint4*>(sm + i * LDB + c0) = pack8_bf16(x);
}
__device__ __forceinline__ void load8_bsm(const bf16* sm, int i, int c0, float (&x)[8]) {
    unpack8_bf16(*reinterpret_cast<const uint4*>(sm + i * LDB + c0), x);
}
// dense BF16 panel rows in global memory
__device__ __forceinline__ void store8_bpanel(bf16* panel, int i, int c0, const float (&x)[8]) {
    *reinterpret_cast<uint4*>(panel + i * DP + c0) = pack8_bf16(x);
}
__device__ __forceinline__ void load8_bpanel(const bf16* panel, int i, int c0, float (&x)[8]) {
    unpack8_bf16(*reinterpret_cast<const uint4*>(panel + i * DP + c0), x);
}

__device__ __forceinline__ bf16* bpanel_ptr(bf16* base, long long gi) { return base + gi * (long long)(CL * DP); }
__device__ __forceinline__ const bf16* bpanel_ptr(const bf16* base, long long gi) {
    return base + gi * (long long)(CL * DP);
}
__device__ __forceinline__ bf16* bmat_ptr(bf16* base, long long gi) { return base + gi * (long long)(CL * CL); }
__device__ __forceinline__ const bf16* bmat_ptr(const bf16* base, long long gi) {
    return base + gi * (long long)(CL * CL);
}

__device__ __forceinline__ void cp16(void* smem, const void* gmem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
// 16 bytes, or 16 zero bytes when !valid (nothing is read then; gmem must still be a mapped address)
__device__ __forceinline__ void cp16_zfill(void* smem, const void* gmem, bool valid) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(valid ? 16 : 0));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::); }
template <int N>
__device__ __forceinline__ void cp_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

// dense BF16 global panel [CL][DP] -> shared [CL][LDB], asynchronously
__device__ __forceinline__ void async_bpanel(bf16* sm, const bf16* g) {
    for (int idx = threadIdx.x; idx < CL * (DP / 8); idx += NTHREADS) {
        int i = idx >> 4, c8 = (idx & 15) << 3;
        cp16(sm + i * LDB + c8, g + i * DP + c8);
    }
}
// dense BF16 global matrix [CL][CL] -> shared [CL][LDM]
__device__ __forceinline__ void async_bmat(bf16* sm, const bf16* g) {
    for (int idx = threadIdx.x; idx < CL * (CL / 8); idx += NTHREADS) {
        int i = idx >> 3, c8 = (idx & 7) << 3;
        cp16(sm + i * LDM + c8, g + i * CL + c8);
    }
}
constexpr size_t BSTATE_BYTES = size_t(DP) * LDB * 2;  // a whole state in BF16

// ---- blocked unit-triangular solve -------------------------------------------
// Solves (I + sgn * T) X = RHS in place for the 2*DP columns of two shared panels,
// T strictly triangular and stored by rows of the system in Mr (FP32, pitch LDA):
//   UPPER == false: T lower  (Mr[i][k], k < i), rows solved first to last;
//   UPPER == true : T upper  (Mr[i][k], k > i), rows solved last to first
//                   (this is how a transposed lower system is passed in).
// Entries outside the stated triangle must be exactly zero.  Mr is consumed: its
// 16 x 16 diagonal blocks are replaced by (I + sgn T_II)^-1 - I.
// The 64 rows are cut into four 16-row blocks.  First the four diagonal blocks are
// inverted by substitution (one warp per block, one lane per column of the inverse).
// After that every warp owns 16 of the 256 right-hand-side columns for the whole
// solve and never waits for another warp: per block it subtracts the coupling with the
// blocks already solved and applies the inverted diagonal block, both on the tensor
// cores (TF32; split-TF32 "3x" coupling when SPLIT).  The identity part of the
// inverse is added from the FP32 registers, so only the correction (T_II^-1 - I) r
// sees TF32 operand rounding.
struct PanelF32 {
    float* p0;
    float* p1;
    __device__ __forceinline__ float get(int k, int n) const {
        return (n < DP ? p0 : p1)[k * LDP + (n & (DP - 1))];
    }
    __device__ __forceinline__ float2 get2(int i, int n) const {
        return *reinterpret_cast<const float2*>((n < DP ? p0 : p1) + i * LDP + (n & (DP - 1)));
    }
    __device__ __forceinline__ void put2(int i, int n, float v0, float v1) const {
        *reinterpret_cast<float2*>((n < DP ? p0 : p1) + i * LDP + (n & (DP - 1))) = make_float2(v0, v1);
    }
};
struct PanelBF16 {
    bf16* p0;
    bf16* p1;
    __device__ __forceinline__ float get(int k, int n) const {
        return __bfloat162float((n < DP ? p0 : p1)[k * LDB + (n & (DP - 1))]);
    }
    __device__ __forceinline__ float2 get2(int i, int n) const {
        return __bfloat1622float2(
            *reinterpret_cast<const __nv_bfloat162*>((n < DP ? p0 : p1) + i * LDB + (n & (DP - 1))));
    }
    __device__ __forceinline__ void put2(int i, int n, float v0, float v1) const {
        *reinterpret_cast<__nv_bfloat162*>((n < DP ? p0 : p1) + i * LDB + (n & (DP - 1))) =
            __floats2bfloat162_rn(v0, v1);
    }
};

template <bool UPPER, bool SPLIT, class Panel>
__device__ __forceinline__ void trisolve_blocked(float* Mr, float sgn, Panel P) {
    static_assert(NTHREADS == 2 * DP * 2, "16 warps of 16 right-hand-side columns each");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    constexpr int NB = CL / 16;
    // ---- the four diagonal blocks: D_I <- (I + sgn T_II)^-1 - I, in place -------------
    if (warp < NB) {
        float* D = Mr + (16 * warp) * LDA + 16 * warp;
        const int j = lane & 15;   // column of the inverse (both half-warps compute the same block)
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = (i == j) ? 1.f : 0.f;
        if (!UPPER) {
#pragma unroll
            for (int i = 1; i < 16; ++i) {
                float a0 = 0.f, a1 = 0.f;
#pragma unroll
                for (int k4 = 0; k4 < i; k4 += 4) {
                    const float4 m = *reinterpret_cast<const float4*>(D + i * LDA + k4);
                    a0 = fmaf(m.x, x[k4], a0);
                    a1 = fmaf(m.y, x[k4 + 1], a1);
                    a0 = fmaf(m.z, x[k4 + 2], a0);
                    a1 = fmaf(m.w, x[k4 + 3], a1);
                }
                x[i] = (i > j) ? -sgn * (a0 + a1) : x[i];
            }
        } else {
#pragma unroll
            for (int i = 14; i >= 0; --i) {
                float a0 = 0.f, a1 = 0.f;
#pragma unroll
                for (int k4 = ((i + 1) & ~3); k4 < 16; k4 += 4) {
                    const float4 m = *reinterpret_cast<const float4*>(D + i * LDA + k4);
                    a0 = fmaf(m.x, x[k4], a0);
                    a1 = fmaf(m.y, x[k4 + 1], a1);
                    a0 = fmaf(m.z, x[k4 + 2], a0);
                    a1 = fmaf(m.w, x[k4 + 3], a1);
                }
                x[i] = (i < j) ? -sgn * (a0 + a1) : x[i];
            }
        }
        __syncwarp();   // every lane has read the block before anyone overwrites it
        if (lane < 16) {
#pragma unroll
            for (int i = 0; i < 16; ++i) D[i * LDA + j] = (i == j) ? 0.f : x[i];
        }
    }
    __syncthreads();
    // ---- warp-local sweep over this warp's 16 columns ---------------------------------
    const int n0 = 16 * warp;
    // fully unrolled: every bound below is a compile-time constant, so the operand loads of a block run ahead
    // of the contractions that use them
#pragma unroll
    for (int step = 0; step < NB; ++step) {
        const int I = UPPER ? (NB - 1 - step) : step;
        const int r0 = 16 * I;
        float rr[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int j = n0 + nt * 8 + 2 * t;
            const float2 a = P.get2(r0 + g, j), b = P.get2(r0 + g + 8, j);
            rr[nt][0] = a.x; rr[nt][1] = a.y; rr[nt][2] = b.x; rr[nt][3] = b.y;
        }
        if (step > 0) {
            // r = RHS[I] - sgn * Mr[I rows][solved cols] * X[solved rows]
            const int kbeg = UPPER ? 16 * (I + 1) : 0;
            const int kend = UPPER ? CL : 16 * I;
            float acc[2][4];
            acc_zero<2>(acc);
#pragma unroll
            for (int kk = kbeg; kk < kend; kk += 8) {
                float af[4] = {Mr[(r0 + g) * LDA + kk + t], Mr[(r0 + g + 8) * LDA + kk + t],
                               Mr[(r0 + g) * LDA + kk + t + 4], Mr[(r0 + g + 8) * LDA + kk + t + 4]};
                uint32_t ah[4], al[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    ah[e] = f2tf32(af[e]);
                    if (SPLIT) al[e] = f2tf32(af[e] - __uint_as_float(ah[e]));
                }
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    float b0 = P.get(kk + t, n0 + nt * 8 + g), b1 = P.get(kk + t + 4, n0 + nt * 8 + g);
                    uint32_t bh0 = f2tf32(b0), bh1 = f2tf32(b1);
                    if (SPLIT) {
                        uint32_t bl0 = f2tf32(b0 - __uint_as_float(bh0)), bl1 = f2tf32(b1 - __uint_as_float(bh1));
                        mma_tf32(acc[nt], al[0], al[1], al[2], al[3], bh0, bh1);
                        mma_tf32(acc[nt], ah[0], ah[1], ah[2], ah[3], bl0, bl1);
                    }
                    mma_tf32(acc[nt], ah[0], ah[1], ah[2], ah[3], bh0, bh1);
                }
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) rr[nt][e] = fmaf(-sgn, acc[nt][e], rr[nt][e]);
                const int j = n0 + nt * 8 + 2 * t;
                P.put2(r0 + g, j, rr[nt][0], rr[nt][1]);
                P.put2(r0 + g + 8, j, rr[nt][2], rr[nt][3]);
            }
            __syncwarp();
        }
        {
            // X[I] = r + D_I r : the block's own rows, K = 16 (the identity part stays in FP32 registers)
            float acc[2][4];
            acc_zero<2>(acc);
#pragma unroll
            for (int kk = 0; kk < 16; kk += 8) {
                const uint32_t a0 = f2tf32(Mr[(r0 + g) * LDA + r0 + kk + t]);
                const uint32_t a1 = f2tf32(Mr[(r0 + g + 8) * LDA + r0 + kk + t]);
                const uint32_t a2 = f2tf32(Mr[(r0 + g) * LDA + r0 + kk + t + 4]);
                const uint32_t a3 = f2tf32(Mr[(r0 + g + 8) * LDA + r0 + kk + t + 4]);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const uint32_t b0 = f2tf32(P.get(r0 + kk + t, n0 + nt * 8 + g));
                    const uint32_t b1 = f2tf32(P.get(r0 + kk + t + 4, n0 + nt * 8 + g));
                    mma_tf32(acc[nt], a0, a1, a2, a3, b0, b1);
                }
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int j = n0 + nt * 8 + 2 * t;
                P.put2(r0 + g, j, rr[nt][0] + acc[nt][0], rr[nt][1] + acc[nt][1]);
                P.put2(r0 + g + 8, j, rr[nt][2] + acc[nt][2], rr[nt][3] + acc[nt][3]);
            }
            __syncwarp();
        }
    }
    __syncthreads();
}

}  // namespace sd
