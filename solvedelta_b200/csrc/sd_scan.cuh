// The serial chunk-state scan shared by all four state carries.
//
// For every chunk, in forward or reverse chunk order:
//     X  = P + Q * St              (CL x NS, contraction over the DP state rows)
//     checkpoint St
//     St = diag(lam) St + R^T X  (+ R2^T X2)
// St is a [DP][NS] column slice of the carried state (the predictor state is
// carried transposed, St[c][a] = C[a][c], so that both C and S decay by rows).
// Column slices never exchange data, so a stream is split over DP/NS CTAs.
// The two forward scans (FP32 panels, TF32 contractions) run on tensor memory,
// k_state_scan_tc; the two reverse scans (BF16 panels) keep the slice in
// mma.sync accumulator registers, k_state_scan_b below.  In both, panels of the
// next chunk stream in through cp.async while the current contraction runs.
#pragma once
#include "sd_bf16.cuh"
#include "sd_common.cuh"

namespace sd {

constexpr int SCAN_NS = 64;            // state columns per CTA (2 CTAs per stream)
constexpr int SCAN_G1 = SCAN_NS / 16;  // 8-column tiles per warp in X = P + Q St
constexpr int SCAN_THREADS = 256;      // 8 warps: one 16-row strip of the state slice each

struct ScanParams {
    const float* P;    // [chunks][CL][DP]
    const float* Q;
    const float* R;
    const float* lam;  // [chunks][DP]
    float* X;          // out [chunks][CL][DP]            (FP32; or null when Xb is set)
    float* ck;         // out [chunks][DP][DP] state before the chunk's update (or null when ckb is set)
    bf16* Xb;          // BF16 alternatives for consumers that only feed BF16 contractions
    bf16* ckb;
    const float* init; // nullable: true-dimension state [S][rows][cols] (or transposed)
    float* fin;        // nullable
    int NC;            // chunks per stream
    int reverse;       // walk chunks last to first
    int transposed_io; // init/fin hold the transpose (predictor state C[a][c])
    int nrows, ncols;  // true dims of the carried St: rows (<= DP), cols (<= DP)
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

}  // namespace sd

// ---------------------------------------------------------------------------
// BF16-operand variant of the scan, used by the two reverse scans (gradient
// tolerances admit BF16 contraction operands; the carried state itself stays
// FP32 in registers).  Panels P, Q, R, R2, X2 and the outputs X and the state
// checkpoints are BF16 in global memory.
namespace sd {

constexpr int LDTB = SCAN_NS + 8;  // pitch of [*][NS] BF16 shared buffers

struct ScanParamsB {
    const bf16* P;
    const bf16* Q;
    const bf16* R;
    const bf16* R2;   // nullable
    const bf16* X2;   // nullable
    const float* lam; // [chunks][DP]
    bf16* X;          // out [chunks][CL][DP]
    bf16* ck;         // out [chunks][DP][DP]
    const float* init;
    float* fin;
    int NC, reverse, transposed_io, nrows, ncols;
};

__device__ __forceinline__ void async_bpanel_scan(bf16* sm, const bf16* g) {
    for (int idx = threadIdx.x; idx < CL * (DP / 8); idx += SCAN_THREADS) {
        int i = idx >> 4, c8 = (idx & 15) << 3;
        cp16(sm + i * LDB + c8, g + i * DP + c8);
    }
}
__device__ __forceinline__ void async_bslice(bf16* sm, const bf16* g, int col0) {
    for (int idx = threadIdx.x; idx < CL * (SCAN_NS / 8); idx += SCAN_THREADS) {
        int i = idx / (SCAN_NS / 8), c8 = (idx % (SCAN_NS / 8)) << 3;
        cp16(sm + i * LDTB + c8, g + i * DP + col0 + c8);
    }
}

constexpr size_t SCAN_B_SMEM_BYTES = (size_t(6) * CL * LDB + size_t(5) * CL * LDTB + size_t(DP) * LDTB) * 2;

__global__ void __launch_bounds__(SCAN_THREADS, 1) k_state_scan_b(ScanParamsB p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);  // [2][CL][LDB]
    bf16* sR = sQ + 2 * CL * LDB;                  // [2][CL][LDB]
    bf16* sR2 = sR + 2 * CL * LDB;                 // [2][CL][LDB]
    bf16* sP = sR2 + 2 * CL * LDB;                 // [2][CL][LDTB]
    bf16* sX2 = sP + 2 * CL * LDTB;                // [2][CL][LDTB]
    bf16* sX = sX2 + 2 * CL * LDTB;                // [CL][LDTB]
    bf16* sSt = sX + CL * LDTB;                    // [DP][LDTB]

    const int col0 = (blockIdx.x % (DP / SCAN_NS)) * SCAN_NS;   // grid.x = stream * (DP / NS) + column slice
    const int s = blockIdx.x / (DP / SCAN_NS);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const bool has2 = p.R2 != nullptr;
    const long long base = (long long)s * p.NC;

    float st[SCAN_NS / 8][4];
    const int row_a = warp * 16 + g, row_b = row_a + 8;
#pragma unroll
    for (int nt = 0; nt < SCAN_NS / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            int rr = (e < 2) ? row_a : row_b;
            int cc = col0 + nt * 8 + 2 * t + (e & 1);
            float v = 0.f;
            if (p.init != nullptr && rr < p.nrows && cc < p.ncols) {
                const float* src = p.init + (long long)s * p.nrows * p.ncols;
                v = p.transposed_io ? src[(long long)cc * p.nrows + rr] : src[(long long)rr * p.ncols + cc];
            }
            st[nt][e] = v;
        }
    }

    auto chunk_at = [&](int step) { return base + (p.reverse ? (p.NC - 1 - step) : step); };
    auto issue = [&](int step) {
        if (step < p.NC) {
            const long long gi = chunk_at(step);
            const int b = step & 1;
            async_bpanel_scan(sQ + b * CL * LDB, bpanel_ptr(p.Q, gi));
            async_bslice(sP + b * CL * LDTB, bpanel_ptr(p.P, gi), col0);
            async_bpanel_scan(sR + b * CL * LDB, bpanel_ptr(p.R, gi));
            if (has2) {
                async_bpanel_scan(sR2 + b * CL * LDB, bpanel_ptr(p.R2, gi));
                async_bslice(sX2 + b * CL * LDTB, bpanel_ptr(p.X2, gi), col0);
            }
        }
        cp_commit();
    };
    issue(0);

    for (int step = 0; step < p.NC; ++step) {
        const long long gi = chunk_at(step);
        const bf16* bQ = sQ + (step & 1) * CL * LDB;
        const bf16* bR = sR + (step & 1) * CL * LDB;
        const bf16* bR2 = sR2 + (step & 1) * CL * LDB;
        const bf16* bP = sP + (step & 1) * CL * LDTB;
        const bf16* bX2 = sX2 + (step & 1) * CL * LDTB;
        const float* lam = p.lam + gi * DP;
        const float la = lam[row_a], lb = lam[row_b];
        {
            bf16* ck = p.ck + gi * (long long)(DP * DP);
#pragma unroll
            for (int nt = 0; nt < SCAN_NS / 8; ++nt) {
                int cc = nt * 8 + 2 * t;
                __nv_bfloat162 va = __floats2bfloat162_rn(st[nt][0], st[nt][1]);
                __nv_bfloat162 vb = __floats2bfloat162_rn(st[nt][2], st[nt][3]);
                *reinterpret_cast<__nv_bfloat162*>(sSt + row_a * LDTB + cc) = va;
                *reinterpret_cast<__nv_bfloat162*>(sSt + row_b * LDTB + cc) = vb;
                *reinterpret_cast<__nv_bfloat162*>(ck + row_a * DP + col0 + cc) = va;
                *reinterpret_cast<__nv_bfloat162*>(ck + row_b * DP + col0 + cc) = vb;
            }
        }
        cp_wait<0>();
        __syncthreads();
        issue(step + 1);   // the previous step's ring slot is free: prefetch during the whole of this step
        {
            float acc[SCAN_G1][4];
            acc_zero<SCAN_G1>(acc);
            const int r0 = (warp & 3) * 16, n0 = (warp >> 2) * (SCAN_NS / 2);
            warp_mma_bf16<SCAN_G1, false, false>(acc, bQ, LDB, sSt, LDTB, r0, n0, 0, DP);
            bf16* xg = bpanel_ptr(p.X, gi);
            warp_epi<SCAN_G1>(acc, r0, n0, [&](int i, int j, float v0, float v1) {
                float2 pv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(bP + i * LDTB + j));
                __nv_bfloat162 xv = __floats2bfloat162_rn(pv.x + v0, pv.y + v1);
                *reinterpret_cast<__nv_bfloat162*>(sX + i * LDTB + j) = xv;
                *reinterpret_cast<__nv_bfloat162*>(xg + i * DP + col0 + j) = xv;
            });
        }
        __syncthreads();
        {
#pragma unroll
            for (int nt = 0; nt < SCAN_NS / 8; ++nt) {
                st[nt][0] *= la;
                st[nt][1] *= la;
                st[nt][2] *= lb;
                st[nt][3] *= lb;
            }
            warp_mma_bf16<SCAN_NS / 8, true, false>(st, bR, LDB, sX, LDTB, warp * 16, 0, 0, CL);
            if (has2) warp_mma_bf16<SCAN_NS / 8, true, false>(st, bR2, LDB, bX2, LDTB, warp * 16, 0, 0, CL);
        }
    }
    cp_wait<0>();

    if (p.fin != nullptr) {
        float* dst = p.fin + (long long)s * p.nrows * p.ncols;
#pragma unroll
        for (int nt = 0; nt < SCAN_NS / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int rr = (e < 2) ? row_a : row_b;
                int cc = col0 + nt * 8 + 2 * t + (e & 1);
                if (rr < p.nrows && cc < p.ncols) {
                    if (p.transposed_io)
                        dst[(long long)cc * p.nrows + rr] = st[nt][e];
                    else
                        dst[(long long)rr * p.ncols + cc] = st[nt][e];
                }
            }
        }
    }
}

}  // namespace sd
