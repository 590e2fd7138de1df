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
// dense FP32 global panel -> BF16 shared panel (through registers)
__device__ __forceinline__ void g2s_panel_f32_to_bf16(bf16* sm, const float* g) {
    for (int idx = threadIdx.x; idx < CL * (DP / 8); idx += NTHREADS) {
        int i = idx >> 4, c8 = (idx & 15) << 3;
        float x[8];
        float4 a = *reinterpret_cast<const float4*>(g + i * DP + c8);
        float4 b = *reinterpret_cast<const float4*>(g + i * DP + c8 + 4);
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
        x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        *reinterpret_cast<uint4*>(sm + i * LDB + c8) = pack8_bf16(x);
    }
}
// whole FP32 state [DP][DP] -> BF16 shared [DP][LDB]
__device__ __forceinline__ void g2s_state_f32_to_bf16(bf16* sm, const float* st) {
    for (int idx = threadIdx.x; idx < DP * (DP / 8); idx += NTHREADS) {
        int i = idx >> 4, c8 = (idx & 15) << 3;
        float x[8];
        float4 a = *reinterpret_cast<const float4*>(st + i * DP + c8);
        float4 b = *reinterpret_cast<const float4*>(st + i * DP + c8 + 4);
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
        x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        *reinterpret_cast<uint4*>(sm + i * LDB + c8) = pack8_bf16(x);
    }
}
constexpr size_t BSTATE_BYTES = size_t(DP) * LDB * 2;  // a whole state in BF16

}  // namespace sd
