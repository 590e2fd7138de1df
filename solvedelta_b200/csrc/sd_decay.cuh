// Block-centred decay factors for the intra-chunk contractions.
//
// A chunk of CL tokens is cut into NBLK blocks of BT tokens.  With G the
// inclusive prefix of the log decay inside the chunk, E = G - g the exclusive
// one, and Gprev_I / Gend_I the prefix just before / at the end of block I,
// every decay-weighted term exp(x_i - G_j) (x = G or E, j <= i) is evaluated
// from factors that never exceed one, so no reciprocal retention exp(-G) is
// ever formed and arbitrarily strong forgetting stays exact:
//   rowG_i = exp(G_i - Gprev_I),  rowE_i = exp(E_i - Gprev_I)    row side
//   col_j  = exp(Gend_J - G_j)                                    column side
//   beta_J = exp(Gend_J - Gprev_J)                                a whole block
//   exp(x_i - G_j) = row_i * (prod_{J<K<I} beta_K) * col_j        for J < I
// and inside one block (I == J) the exponent is evaluated directly.
//
// Three contraction forms use this:
//   pair   A[i][j]   = sum_c a[i][c] b[j][c] exp(x_ic - G_jc)
//   causal out[i][c] = sum_{j<=i} P[i][j] b[j][c] exp(x_ic - G_jc)
//   anti   out[j][c] = sum_{i>=j} P[i][j] a[i][c] exp(x_ic - G_jc)
// Off-diagonal blocks run on the tensor cores over row-/column-centred panels
// (pair: the beta product scales the row operand along the contraction; causal
// / anti: the accumulator is multiplied by beta between blocks, Horner-style).
// The helpers here cover the factors and the diagonal blocks.
//
// Upstream counterpart: the centred cross-subchunk factorisation and direct
// diagonal subchunks of causallsso/ops/residual_frame/vector_pair.py:1-16.
#pragma once
#include "sd_bf16.cuh"
#include "sd_common.cuh"

namespace sd {

constexpr int BT = 16;          // tokens per decay block
constexpr int NBLK = CL / BT;   // blocks per chunk

// Fast blocks.  Inside one block the reciprocal form is harmless as long as the block
// forgets less than FAST_BLOCK_NATS in every channel: exp(Gprev_I - G_j) <= e^60 then, and
// the diagonal block is one more tensor-core block (pair: the row operand scaled by
// 1 / beta_I along the contraction; causal / anti: one more Horner step, with the final
// factor referenced to the other end of the block).  A block that forgets more takes the
// direct evaluation.  The choice is per block and uniform over a warp tile.
constexpr float FAST_BLOCK_NATS = 60.f;

// One thread per (block J, channel c): s_beta = exp(Gend_J - Gprev_J), s_ibeta = its
// reciprocal (0 where the block is not fast), s_fastw[warp] = every channel of the warp's
// slice is fast.  Needs a __syncthreads() before the tables are read.
template <class FG>
__device__ __forceinline__ void block_decay_tables(float* s_beta, float* s_ibeta, int* s_fastw, FG fg) {
    static_assert(NTHREADS == NBLK * DP, "one thread per (block, channel)");
    const int J = threadIdx.x >> 7, c = threadIdx.x & (DP - 1);
    const float d = fg(BT * J + BT - 1, c) - (J ? fg(BT * J - 1, c) : 0.f);
    const bool ok = d >= -FAST_BLOCK_NATS;
    if (s_beta != nullptr) s_beta[threadIdx.x] = __expf(d);
    if (s_ibeta != nullptr) s_ibeta[threadIdx.x] = ok ? __expf(-d) : 0.f;
    const int all = __all_sync(0xffffffffu, ok);
    if ((threadIdx.x & 31) == 0) s_fastw[threadIdx.x >> 5] = all;
}
// block I is fast: all four warps of its channel slices agreed
__device__ __forceinline__ bool block_is_fast(const int* s_fastw, int I) {
    return (s_fastw[4 * I] & s_fastw[4 * I + 1] & s_fastw[4 * I + 2] & s_fastw[4 * I + 3]) != 0;
}

// Row-operand scale of an off-diagonal pair block (I, J), I - J >= 2:
//   s_M[0] = beta_1 (blocks (2,0)),  s_M[1] = beta_2 ((3,1)),  s_M[2] = beta_1 beta_2 ((3,0)).
template <class FG>
__device__ __forceinline__ void pair_block_scales(float* s_M, FG fg) {
    static_assert(NBLK == 4, "pair scale table is written for four blocks");
    for (int idx = threadIdx.x; idx < 3 * DP; idx += NTHREADS) {
        const int m = idx >> 7, c = idx & (DP - 1);
        const float e0 = fg(BT - 1, c), e1 = fg(2 * BT - 1, c), e2 = fg(3 * BT - 1, c);
        s_M[idx] = __expf(m == 0 ? e1 - e0 : (m == 1 ? e2 - e1 : e2 - e0));
    }
}
__device__ __forceinline__ int pair_scale_index(int I, int J) {  // -1: adjacent blocks, no scale
    return (I - J < 2) ? -1 : (I - J == 3 ? 2 : J);
}

// acc columns n0 + 8 nt + 2t (+1) *= vec[column]
template <int NTW>
__device__ __forceinline__ void scale_acc(float (&acc)[NTW][4], const float* vec, int n0) {
    const int t = threadIdx.x & 3;
#pragma unroll
    for (int nt = 0; nt < NTW; ++nt) {
        const float2 b = *reinterpret_cast<const float2*>(vec + n0 + nt * 8 + 2 * t);
        acc[nt][0] *= b.x; acc[nt][1] *= b.y;
        acc[nt][2] *= b.x; acc[nt][3] *= b.y;
    }
}

// ---- blocks of a pair on the tensor cores (TF32) --------------------------------
// Warp (I = row tile, J = column quarter) of the CL x CL tiling owns block (I, J).
// fr(i, k): row-centred operand, fc(j, k): column-centred operand, k = channel.
// fe(i, j, v0, v1) receives every element of the blocks below the diagonal (the
// contraction), above it (zeros) and of the FAST diagonal blocks (masked to j <= i,
// or j < i when STRICT); diagonal blocks that are not fast are left untouched.
template <bool STRICT, class FR, class FC, class FE>
__device__ __forceinline__ void pair_blocks_tf32(const float* s_M, const float* s_ibeta, const int* s_fastw, FR fr,
                                                 FC fc, FE fe) {
    const int r0 = Tile64<CL>::r0(), n0 = Tile64<CL>::n0();
    const int I = r0 / BT, J = n0 / BT;
    if (I == J && !block_is_fast(s_fastw, I)) return;   // left to the direct evaluation
    float acc[NT64][4];
    acc_zero<NT64>(acc);
    if (J <= I) {
        const int m = pair_scale_index(I, J);
        auto fb = [&](int k, int n) { return fc(n, k); };
        if (J < I && m < 0) {
            warp_mma<NT64>(acc, r0, n0, 0, DP, fr, fb);
        } else {
            // beta product between the blocks, or 1 / beta_I inside a fast diagonal block
            const float* mv = (J == I) ? s_ibeta + I * DP : s_M + m * DP;
            warp_mma<NT64>(acc, r0, n0, 0, DP, [&](int i, int k) { return fr(i, k) * mv[k]; }, fb);
        }
    }
    if (I == J) {
        warp_epi<NT64>(acc, r0, n0, [&](int i, int j, float v0, float v1) {
            fe(i, j, (STRICT ? j < i : j <= i) ? v0 : 0.f, (STRICT ? j + 1 < i : j + 1 <= i) ? v1 : 0.f);
        });
    } else {
        warp_epi<NT64>(acc, r0, n0, fe);
    }
}

// BF16 copy of the pair scale table for the BF16 contractions.
template <class FG>
__device__ __forceinline__ void pair_block_scales_bf16(bf16* s_Mb, FG fg) {
    static_assert(NBLK == 4, "pair scale table is written for four blocks");
    for (int idx = threadIdx.x; idx < 3 * DP; idx += NTHREADS) {
        const int m = idx >> 7, c = idx & (DP - 1);
        const float e0 = fg(BT - 1, c), e1 = fg(2 * BT - 1, c), e2 = fg(3 * BT - 1, c);
        s_Mb[idx] = __float2bfloat16_rn(__expf(m == 0 ? e1 - e0 : (m == 1 ? e2 - e1 : e2 - e0)));
    }
}

// Pair blocks, BF16 operands in shared panels of pitch LDB: R row-centred, C column-centred,
// s_ibeta_b the BF16 copy of 1 / beta.  fe as for pair_blocks_tf32.
template <bool STRICT, class FE>
__device__ __forceinline__ void pair_blocks_bf16(const bf16* s_Mb, const bf16* s_ibeta_b, const int* s_fastw,
                                                 const bf16* R, const bf16* C, FE fe) {
    const int r0 = Tile64<CL>::r0(), n0 = Tile64<CL>::n0();
    const int I = r0 / BT, J = n0 / BT;
    if (I == J && !block_is_fast(s_fastw, I)) return;
    float acc[NT64][4];
    acc_zero<NT64>(acc);
    if (J <= I) {
        const int m = pair_scale_index(I, J);
        if (J < I && m < 0)
            warp_mma_bf16<NT64, false, true>(acc, R, LDB, C, LDB, r0, n0, 0, DP);
        else
            warp_mma_bf16_kscale<NT64, true>(acc, R, LDB, C, LDB, r0, n0, 0, DP,
                                             (J == I) ? s_ibeta_b + I * DP : s_Mb + m * DP);
    }
    if (I == J) {
        warp_epi<NT64>(acc, r0, n0, [&](int i, int j, float v0, float v1) {
            fe(i, j, (STRICT ? j < i : j <= i) ? v0 : 0.f, (STRICT ? j + 1 < i : j + 1 <= i) ? v1 : 0.f);
        });
    } else {
        warp_epi<NT64>(acc, r0, n0, fe);
    }
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Sum over the 16 lanes of a half-warp of 16 per-lane values at once: lane l of
// the half-warp ends with the total of v[l].  15 shuffles instead of 64.
__device__ __forceinline__ float transpose_sum16(float (&v)[BT]) {
    static_assert(BT == 16, "written for 16 lanes");
    const int l = threadIdx.x & 15;
    const bool b3 = l & 8, b2 = l & 4, b1 = l & 2, b0 = l & 1;
    float w8[8], w4[4], w2[2];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float send = b3 ? v[k] : v[k + 8];
        const float keep = b3 ? v[k + 8] : v[k];
        w8[k] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float send = b2 ? w8[k] : w8[k + 4];
        const float keep = b2 ? w8[k + 4] : w8[k];
        w4[k] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const float send = b1 ? w4[k] : w4[k + 2];
        const float keep = b1 ? w4[k + 2] : w4[k];
        w2[k] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
    }
    const float send = b0 ? w2[0] : w2[1];
    const float keep = b0 ? w2[1] : w2[0];
    return keep + __shfl_xor_sync(0xffffffffu, send, 1);
}

// Token row of pass pp for the half-warp lr = tid / 16 when a row-wise loop also walks the
// diagonal blocks of a pair: the work of row i grows with its position in its block, so the
// second pass mirrors the position (15 - ii) -- every warp then carries the same total work
// and the rows of a warp stay an adjacent pair of one block.
__device__ __forceinline__ int balanced_row(int lr, int pp) {
    static_assert(ROW_PASSES == 2 && ROWS_PER_PASS == 2 * BT, "written for two passes of two blocks");
    return pp == 0 ? lr : ROWS_PER_PASS + ((lr & BT) | (BT - 1 - (lr & (BT - 1))));
}

// ---- diagonal blocks of a pair, row-wise mapping -----------------------------
// The calling half-warp owns token row i and each lane eight channels of it:
// a[n][8] are NA row operands sharing one exponent, x[8] the row prefix (G or E).
// fb8(j, b) / fg8(j, G) fetch the same eight channels of column-side row j.
// For every j of the row's own block with j <= i (j < i when STRICT):
//   val[n] = sum_c a[n][c] b[j][c] exp(x[c] - G[j][c])
// and lane (j mod BT) of the half-warp receives val in out[n]; other entries of the
// block row are returned as zero.  All 32 lanes of the warp must call together
// (the two rows of a warp lie in the same block).
template <int NA, bool STRICT, class FB8, class FG8>
__device__ __forceinline__ void pair_diag_row(int i, const float (&a)[NA][8], const float (&x)[8], FB8 fb8, FG8 fg8,
                                              float (&out)[NA]) {
    constexpr float LOG2E = 1.4426950408889634f;
    const int i0 = i & ~(BT - 1), ii = i & (BT - 1);
    const int jmax = (ii | 1) - (STRICT ? 1 : 0);  // uniform over the warp's two rows (2w, 2w+1)
    float xs[8], part[NA][BT];
#pragma unroll
    for (int e = 0; e < 8; ++e) xs[e] = x[e] * LOG2E;
#pragma unroll
    for (int jj = 0; jj < BT; ++jj) {
#pragma unroll
        for (int n = 0; n < NA; ++n) part[n][jj] = 0.f;
        if (jj <= jmax) {  // warp-uniform
            float b[8], G[8], s[NA];
            fb8(i0 + jj, b);
            fg8(i0 + jj, G);
#pragma unroll
            for (int n = 0; n < NA; ++n) s[n] = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                // exp(x - G) as 2^((x - G) log2 e); the exponent is <= 0 for every live pair
                const float w = b[e] * ex2_approx(fmaf(-G[e], LOG2E, xs[e]));
#pragma unroll
                for (int n = 0; n < NA; ++n) s[n] = fmaf(a[n][e], w, s[n]);
            }
            const bool live = STRICT ? (jj < ii) : (jj <= ii);
#pragma unroll
            for (int n = 0; n < NA; ++n) part[n][jj] = live ? s[n] : 0.f;
        }
    }
#pragma unroll
    for (int n = 0; n < NA; ++n) out[n] = transpose_sum16(part[n]);
}

// ---- diagonal blocks of a causal / anti-causal sum, one thread per (channel, block) ----
// Thread (c = tid mod DP, I = tid / DP) walks the BT x BT block I of P with the
// retention exp(x_i - G_j) built as a running product of alpha_k = exp(g_k), so
// only BT exponentials are taken per thread.
//   XE: x is the exclusive prefix (the term j == i does not exist then).
template <class FG>
__device__ __forceinline__ void block_alphas(float (&al)[BT], FG fG) {
    static_assert(NTHREADS == NBLK * DP, "one thread per (channel, block)");
    const int c = threadIdx.x & (DP - 1), i0 = (threadIdx.x >> 7) * BT;
    float prev = i0 ? fG(i0 - 1, c) : 0.f;
#pragma unroll
    for (int k = 0; k < BT; ++k) {
        const float g = fG(i0 + k, c);
        al[k] = __expf(g - prev);
        prev = g;
    }
}

// One sweep over the thread's BT x BT diagonal block of P serving both directions:
//   CAUSAL: oc(i, c, sum_{j<=i} P[i][j] b[j] rho_ij)      ANTI: oa(j, c, sum_{i>=j} P[i][j] a[i] rho_ij)
// with rho_ij = exp(x_i - G_j) built by a running product of the alphas (al).
//   XE: x is the exclusive prefix (j < i only);  STRICT: the term j == i is skipped.
//   fP16(i, i0, row): the BT entries P[i][i0 .. i0+BT) (the same address for every thread of a warp);
//   fb(j, c) / fa(i, c): column-side / row-side operand themselves (not centred).
//   reset_rows: bit i set when token row i is a reset token.  Only the exclusive prefix needs it (XE): the
//   reset belongs to row i itself, which the running product over rows j+1 .. i-1 does not contain.
template <bool XE, bool STRICT, bool CAUSAL, bool ANTI, class FP16, class FB, class FA, class FOC, class FOA>
__device__ __forceinline__ void diag_sweep(const float (&al)[BT], FP16 fP16, FB fb, FA fa, FOC oc, FOA oa,
                                           unsigned long long reset_rows = 0ull) {
    const int c = threadIdx.x & (DP - 1), i0 = (threadIdx.x >> 7) * BT;
    float bv[BT], accA[BT];
#pragma unroll
    for (int k = 0; k < BT; ++k) {
        bv[k] = CAUSAL ? fb(i0 + k, c) : 0.f;
        accA[k] = 0.f;
    }
#pragma unroll
    for (int ii = 0; ii < BT; ++ii) {
        float prow[BT];
        fP16(i0 + ii, i0, prow);
        const float av = ANTI ? fa(i0 + ii, c) : 0.f;
        float accC = 0.f, rho = (XE && ((reset_rows >> (i0 + ii)) & 1ull)) ? 0.f : 1.f;
#pragma unroll
        for (int jj = XE ? ii - 1 : ii; jj >= 0; --jj) {
            if (!(STRICT && jj == ii)) {
                const float pr = prow[jj] * rho;
                if (CAUSAL) accC = fmaf(pr, bv[jj], accC);
                if (ANTI) accA[jj] = fmaf(pr, av, accA[jj]);
            }
            rho *= al[jj];
        }
        if (CAUSAL) oc(i0 + ii, c, accC);
    }
    if (ANTI) {
#pragma unroll
        for (int jj = 0; jj < BT; ++jj) oa(i0 + jj, c, accA[jj]);
    }
}

// Row segment loaders for diag_sweep.
__device__ __forceinline__ void prow16_f32(const float* M, int ld, int i, int i0, float (&row)[BT]) {
    const float4* q = reinterpret_cast<const float4*>(M + i * ld + i0);
#pragma unroll
    for (int k = 0; k < BT / 4; ++k) {
        const float4 v = q[k];
        row[4 * k] = v.x; row[4 * k + 1] = v.y; row[4 * k + 2] = v.z; row[4 * k + 3] = v.w;
    }
}
__device__ __forceinline__ void prow16_bf16(const bf16* M, int ld, int i, int i0, float (&row)[BT]) {
    const uint4* q = reinterpret_cast<const uint4*>(M + i * ld + i0);
#pragma unroll
    for (int k = 0; k < BT / 8; ++k) {
        const uint4 raw = q[k];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            row[8 * k + 2 * e] = f.x;
            row[8 * k + 2 * e + 1] = f.y;
        }
    }
}

}  // namespace sd
