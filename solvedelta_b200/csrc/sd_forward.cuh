// Chunk-parallel forward kernels: one CTA per (stream, chunk).
//
// Pipeline: k_prep_fwd -> scan(C) -> k_primal_exterior_fwd -> scan(S) -> k_output_fwd_tc.
#pragma once
#include "sd_bf16.cuh"
#include "sd_common.cuh"
#include "sd_decay.cuh"

namespace sd {

struct FwdParams {
    Geometry g;
    Operand u, h, q, k, v, er, wr, ld, gam;
    // forward scratch
    float *Upd, *Qc, *Ubar, *Wd, *Ud, *Dt;
    bf16 *Xg;        // chi exp(G): operand of the output contraction, kept for backward (R2 of the dS scan)
    bf16 *Aqd;       // pair matrix of the output contraction, kept for backward
    // BF16 panels of the per-token pass of k_primal_exterior_fwd that the reverse pass contracts with; kept so
    // that it does not evaluate the sources a second time: -e exp(G), chi rowG, -e rowG, d col, d exp(GL-G),
    // and (only for chunks with a block on the direct path) chi and -e themselves
    bf16 *Ag, *Xr, *Er, *Dcol, *DtB, *Chi, *Ee;
    // kept for backward
    float *Lam, *Gp, *Delta, *Dprim, *CtCk;
    float *Npair, *Aed;  // pair matrices N = Lm / gamma and Aed, [CL][CL]
    bf16 *Zt, *SCk;  // only BF16 contractions read these
    void* y;
    // predictor-only entry (null otherwise): BF16 [B,T,H,r] outputs frame action d - k^ and update Delta;
    // k_primal_exterior_fwd then stops after its primal half
    void *action, *update;
};

// Per-token frame covector phi, dual address e and query chi for the eight
// channels a lane owns.  All 16 lanes of a row must call together.
struct Sources {
    float phi[8], b[8], e[8], chi[8];
    float s, n2, den, sb, sq;
};

__device__ __forceinline__ void sources_fwd(const float (&uh)[8], const float (&kh)[8], const float (&qh)[8],
                                            const float (&dl)[8], const float (&se)[8], Sources& o) {
    float n2 = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) n2 = fmaf(dl[e], dl[e], n2);
    n2 = row_sum16(n2);
    const float s = RHO * rsqrtf(RHO * RHO + n2);
    float pu = 0.f, ub = 0.f, uq = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        o.phi[e] = s * dl[e];
        o.b[e] = se[e] * kh[e];
        pu = fmaf(o.phi[e], uh[e], pu);
        ub = fmaf(uh[e], o.b[e], ub);
        uq = fmaf(uh[e], qh[e], uq);
    }
    const float den = 1.f + row_sum16(pu);
    const float sb = row_sum16(ub) / den, sq = row_sum16(uq) / den;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        o.e[e] = o.b[e] - o.phi[e] * sb;
        o.chi[e] = qh[e] - o.phi[e] * sq;
    }
    o.s = s;
    o.n2 = n2;
    o.den = den;
    o.sb = sb;
    o.sq = sq;
}

// Eight channels of one normalised BF16 row, in registers (UNIT: taken as they are).
template <bool FAST, bool UNIT = false, class CH>
__device__ __forceinline__ float load8_norm(const Operand& op, const CH& ch, int i, int c0, int width,
                                            float (&x)[8]) {
    load8_bf16<FAST>(row_bf16(op, ch, i), c0, width, op.vec, ch.ok(i), x);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = fmaf(x[e], x[e], ss);
    ss = row_sum16(ss);
    const float rs = UNIT ? 1.f : rsqrtf(ss + 1e-24f);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] *= rs;
    return rs;
}

__device__ __forceinline__ void load8_panel(const float* panel, int i, int c0, float (&x)[8]) {
    float4 a = *reinterpret_cast<const float4*>(panel + i * DP + c0);
    float4 b = *reinterpret_cast<const float4*>(panel + i * DP + c0 + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void store8_panel(float* panel, int i, int c0, const float (&x)[8]) {
    *reinterpret_cast<float4*>(panel + i * DP + c0) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(panel + i * DP + c0 + 4) = make_float4(x[4], x[5], x[6], x[7]);
}
__device__ __forceinline__ void load8_smem(const float* sm, int i, int c0, float (&x)[8]) {
    float4 a = *reinterpret_cast<const float4*>(sm + i * LDP + c0);
    float4 b = *reinterpret_cast<const float4*>(sm + i * LDP + c0 + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void store8_smem(float* sm, int i, int c0, const float (&x)[8]) {
    *reinterpret_cast<float4*>(sm + i * LDP + c0) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(sm + i * LDP + c0 + 4) = make_float4(x[4], x[5], x[6], x[7]);
}

// ---------------------------------------------------------------------------
// Predictor preparation: pair matrix Lm, and the two solved panels
//   Upd = (I+Lm)^-1 (gamma h),  W = (I+Lm)^-1 (gamma U~)   (stored negated as Qc)
// so that the C scan is  Delta = Upd + Qc Ct.
// Two FP32 panel slots only, so that two CTAs share an SM: slot A holds the prefix G, then the
// row-centred u^ exp(E - Gprev), then gamma U~ / W; slot B holds u^, then the column-centred
// u^ exp(Gend - G), then gamma h / Upd.  What later phases still need of G lives in two small
// tables (the prefix just before and at the end of every block).
constexpr size_t PREP_FWD_SMEM =
    2 * SLOT_BYTES + MAT_BYTES + (CL + 3 * DP + NBLK * DP + 16 + 2 * NBLK * DP) * sizeof(float);
static_assert(2 * (PREP_FWD_SMEM + 1024) <= 228 * 1024, "two CTAs of the predictor preparation per SM");

template <bool FAST, bool MASKED, bool PRED = false>
__global__ void __launch_bounds__(NTHREADS, 2) k_prep_fwd(FwdParams p) {
    int ph = 0;
    SD_PHASE(p.g, ph);
    extern __shared__ __align__(16) float smem[];
    float* s_A = smem;
    float* s_B = s_A + SLOT_FLOATS;
    float* s_lm = s_B + SLOT_FLOATS;
    float* s_gam = s_lm + MAT_FLOATS;
    float* s_M = s_gam + CL;
    float* s_ibeta = s_M + 3 * DP;
    int* s_fastw = reinterpret_cast<int*>(s_ibeta + NBLK * DP);
    float* s_gp = reinterpret_cast<float*>(s_fastw + 16);   // [NBLK][DP] prefix just before the block
    float* s_ge = s_gp + NBLK * DP;                         // [NBLK][DP] prefix at the end of the block
    const ChunkT<MASKED> ch = chunk_of<MASKED>(p.g, blockIdx.x);
    const int r = p.g.r;

    load_norm_panel<FAST, PRED>(p.u, ch, r, s_B, nullptr);
    load_f32_panel<FAST>(p.ld, ch, r, s_A);
    load_gamma(p.gam, ch, s_gam);
    prefetch_rows(p.h, ch, 2, r * 2);   // read after the pair phase
    const bool any_reset = ch.reset_rows() != 0ull;
    if (any_reset) {   // block-uniform: a reset token forgets RESET_NATS more (each thread patches what it loaded)
        const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
#pragma unroll
        for (int pp = 0; pp < ROW_PASSES; ++pp) {
            const int i = lr + ROWS_PER_PASS * pp;
            if (ch.rst(i)) {
#pragma unroll
                for (int e = 0; e < 8; ++e) s_A[i * LDP + c0 + e] -= RESET_NATS;
            }
        }
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    chunk_cumsum(s_A);
    __syncthreads();
    SD_PHASE(p.g, ph);
    auto fG = [&](int i, int c) { return s_A[i * LDP + c]; };
    pair_block_scales(s_M, fG);
    block_decay_tables(nullptr, s_ibeta, s_fastw, fG);
    {
        const int J = threadIdx.x >> 7, c = threadIdx.x & (DP - 1);
        s_gp[threadIdx.x] = J ? fG(BT * J - 1, c) : 0.f;
        s_ge[threadIdx.x] = fG(BT * J + BT - 1, c);
    }
    float* gG = panel_ptr(p.Gp, ch.gi);
    for (int idx = threadIdx.x; idx < CL * (DP / 4); idx += NTHREADS) {
        const int i = idx >> 5, c4 = (idx & 31) << 2;
        *reinterpret_cast<float4*>(gG + i * DP + c4) = *reinterpret_cast<const float4*>(s_A + i * LDP + c4);
    }
    __syncthreads();
    // Lm = gamma stril(N), N[i][j] = sum_c u^_ic u^_jc exp(E_ic - G_jc); N itself is kept for backward.
    // Diagonal blocks that are not fast: direct evaluation, while u^ and G are still in the slots.
    float* gN = mat_ptr(p.Npair, ch.gi);
    {
        const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
#pragma unroll 1
        for (int pp = 0; pp < ROW_PASSES; ++pp) {
            const int i = balanced_row(lr, pp);
            if (block_is_fast(s_fastw, i / BT)) continue;   // that diagonal block runs on the tensor cores
            float a[1][8], x[8], out[1];
            load8_smem(s_B, i, c0, a[0]);
            if (i > 0) {
                load8_smem(s_A, i - 1, c0, x);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = 0.f;
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] -= ch.eoff(i);
            pair_diag_row<1, true>(i, a, x, [&](int j, float (&b)[8]) { load8_smem(s_B, j, c0, b); },
                                   [&](int j, float (&G)[8]) { load8_smem(s_A, j, c0, G); }, out);
            const int j = (i & ~(BT - 1)) + (threadIdx.x & 15);
            s_lm[i * LDA + j] = s_gam[i] * out[0];
            gN[i * CL + j] = out[0];
        }
    }
    {   // centred operands in place: every thread first reads what it needs of both slots, then all write
        constexpr int PER = CL * DP / NTHREADS;
        float ut[PER], un[PER];
        const int c = threadIdx.x & (DP - 1), ib = threadIdx.x >> 7;
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = ib + (NTHREADS / DP) * k, I = i / BT;
            const float G = s_A[i * LDP + c];
            float E = i ? s_A[(i - 1) * LDP + c] : 0.f;
            if (any_reset) E -= ch.eoff(i);   // block-uniform branch
            const float uh = s_B[i * LDP + c];
            ut[k] = uh * __expf(E - s_gp[I * DP + c]);
            un[k] = uh * __expf(s_ge[I * DP + c] - G);
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = ib + (NTHREADS / DP) * k;
            s_A[i * LDP + c] = ut[k];
            s_B[i * LDP + c] = un[k];
        }
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    pair_blocks_tf32<true>(s_M, s_ibeta, s_fastw, [&](int i, int k) { return s_A[i * LDP + k]; },
                           [&](int j, int k) { return s_B[j * LDP + k]; },
                           [&](int i, int j, float v0, float v1) {
                               float gm = s_gam[i];
                               *reinterpret_cast<float2*>(s_lm + i * LDA + j) = make_float2(gm * v0, gm * v1);
                               *reinterpret_cast<float2*>(gN + i * CL + j) = make_float2(v0, v1);
                           });
    {   // Ubar = u^ exp(GL - G) = (column-centred u^) exp(GL - Gend), before slot B is reused
        float* gUbar = panel_ptr(p.Ubar, ch.gi);
        const float* GL = s_ge + (NBLK - 1) * DP;
        for (int idx = threadIdx.x; idx < CL * (DP / 4); idx += NTHREADS) {
            const int i = idx >> 5, c4 = (idx & 31) << 2, I = i / BT;
            const float4 un = *reinterpret_cast<const float4*>(s_B + i * LDP + c4);
            const float4 ge = *reinterpret_cast<const float4*>(s_ge + I * DP + c4);
            const float4 gl = *reinterpret_cast<const float4*>(GL + c4);
            *reinterpret_cast<float4*>(gUbar + i * DP + c4) =
                make_float4(un.x * __expf(gl.x - ge.x), un.y * __expf(gl.y - ge.y), un.z * __expf(gl.z - ge.z),
                            un.w * __expf(gl.w - ge.w));
        }
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    {   // right-hand sides: A = gamma u^ exp(E) (from the row-centred panel), B = gamma h
        const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
#pragma unroll
        for (int pp = 0; pp < ROW_PASSES; ++pp) {
            const int i = lr + ROWS_PER_PASS * pp, I = i / BT;
            const float gm = s_gam[i];
            float h[8], ut[8], gp[8];
            load8_bf16<FAST>(row_bf16(p.h, ch, i), c0, r, p.h.vec, ch.ok(i), h);
            load8_smem(s_A, i, c0, ut);
            load8_panel(s_gp, I, c0, gp);   // the tables have pitch DP
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                h[e] *= gm;
                ut[e] *= gm * __expf(gp[e]);
            }
            store8_smem(s_B, i, c0, h);
            store8_smem(s_A, i, c0, ut);
        }
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    trisolve_blocked<false, false>(s_lm, 1.f, PanelF32{s_B, s_A});
    SD_PHASE(p.g, ph);
    float* gUpd = panel_ptr(p.Upd, ch.gi);
    float* gQc = panel_ptr(p.Qc, ch.gi);
    for (int idx = threadIdx.x; idx < CL * (DP / 4); idx += NTHREADS) {
        int i = idx >> 5, c4 = (idx & 31) << 2;
        float4 up = *reinterpret_cast<const float4*>(s_B + i * LDP + c4);
        float4 w = *reinterpret_cast<const float4*>(s_A + i * LDP + c4);
        *reinterpret_cast<float4*>(gUpd + i * DP + c4) = up;
        // contraction operands of the state scan leave here already rounded to TF32
        *reinterpret_cast<float4*>(gQc + i * DP + c4) =
            make_float4(round_tf32(-w.x), round_tf32(-w.y), round_tf32(-w.z), round_tf32(-w.w));
    }
    if (threadIdx.x < DP) p.Lam[ch.gi * DP + threadIdx.x] = __expf(s_ge[(NBLK - 1) * DP + threadIdx.x]);
    SD_PHASE(p.g, ph);
}

// ---------------------------------------------------------------------------
// Primal address and exterior preparation in one CTA per chunk task.
// First half: d = k^ + C_t^T k^ for every token of the chunk,
//   d_i = k^_i + exp(G_i) (K^ Ct^T)_i + sum_{j<=i} (k^_i . Delta_j) u^_j exp(G_i - G_j),
// the decay-weighted sum in block-centred form (Horner over blocks, direct diagonal).
// Second half, on d and the prefix panel still in shared memory: sources (e, chi, z), the pair matrices
//   Aqd[i][j] = sum_c chi_ic d_jc exp(G_ic - G_jc) (j <= i),  Aed likewise with -e (j < i)
// in block-centred form, and the solved panels Wd = (I-Aed)^-1 ag, Ud = (I-Aed)^-1 Z
// for the S scan (ag = -e exp(G), referenced to the chunk start like the scan itself).
constexpr size_t PRIMAL_EXT_FWD_SMEM = 6 * SLOT_BYTES + MAT_BYTES + (NBLK * DP + 3 * DP + NBLK * DP + 16) * sizeof(float);
static_assert(PRIMAL_EXT_FWD_SMEM <= 227 * 1024, "fits the shared memory of one CTA");


__device__ __forceinline__ void async_panel_f32(float* sm, const float* g) {
    for (int idx = threadIdx.x; idx < CL * (DP / 4); idx += NTHREADS) {
        int i = idx >> 5, c4 = (idx & 31) << 2;
        cp16(sm + i * LDP + c4, g + i * DP + c4);
    }
}
__device__ __forceinline__ void async_state_cols_f32(float* sm, const float* st, int half) {
    for (int idx = threadIdx.x; idx < DP * (CL / 4); idx += NTHREADS) {
        int rrow = idx >> 4, c4 = (idx & 15) << 2;
        cp16(sm + rrow * LDH + c4, st + rrow * DP + half * CL + c4);
    }
}

template <bool FAST, bool MASKED, bool PRED = false>
__global__ void __launch_bounds__(NTHREADS, 1) k_primal_exterior_fwd(FwdParams p) {
    int ph = 0;
    SD_PHASE(p.g, ph);
    extern __shared__ __align__(16) float smem[];
    float* s_kh = smem;
    float* s_un = s_kh + SLOT_FLOATS;
    float* s_G = s_un + SLOT_FLOATS;
    float* s_dl = s_G + SLOT_FLOATS;
    float* s_st0 = s_dl + SLOT_FLOATS;
    float* s_st1 = s_st0 + SLOT_FLOATS;
    float* s_aqk = s_st1 + SLOT_FLOATS;   // Aqk, later Aed
    float* s_beta = s_aqk + MAT_FLOATS;
    float* s_M = s_beta + NBLK * DP;
    float* s_ibeta = s_M + 3 * DP;
    int* s_fastw = reinterpret_cast<int*>(s_ibeta + NBLK * DP);
    const int V = p.g.V;
    const ChunkT<MASKED> ch = chunk_of<MASKED>(p.g, blockIdx.x);
    const int r = p.g.r;
    const float* ct = state_ptr(p.CtCk, ch.gi);

    // everything that is already FP32 in HBM streams in while the BF16 operands are normalised
    async_panel_f32(s_G, panel_ptr(p.Gp, ch.gi));
    async_panel_f32(s_dl, panel_ptr(p.Delta, ch.gi));
    cp_commit();
    async_state_cols_f32(s_st0, ct, 0);
    cp_commit();
    async_state_cols_f32(s_st1, ct, 1);
    cp_commit();
    load_norm_panel<FAST, PRED>(p.k, ch, r, s_kh, nullptr);
    load_norm_panel<FAST, PRED>(p.u, ch, r, s_un, nullptr);
    if (!PRED) {   // rows the per-token pass of the exterior half reads from HBM much later: pull them into L2 now
        prefetch_rows(p.q, ch, 2, r * 2);
        prefetch_rows(p.er, ch, 2, r * 2);
        prefetch_rows(p.wr, ch, 2, V * 2);
        prefetch_rows(p.v, ch, 2, V * 2);
    }
    cp_wait<2>();
    __syncthreads();
    SD_PHASE(p.g, ph);
    auto fG = [&](int i, int c) { return s_G[i * LDP + c]; };
    block_decay_tables(s_beta, s_ibeta, s_fastw, fG);
    pair_block_scales(s_M, fG);
    {
        float acc[NT64][4];
        acc_zero<NT64>(acc);
        const int r0 = Tile64<CL>::r0(), n0 = Tile64<CL>::n0();
        if (n0 <= r0)
            warp_mma<NT64>(acc, r0, n0, 0, DP, [&](int i, int k) { return s_kh[i * LDP + k]; },
                        [&](int k, int n) { return s_dl[n * LDP + k]; });
        warp_epi<NT64>(acc, r0, n0, [&](int i, int j, float v0, float v1) {
            s_aqk[i * LDA + j] = (j <= i) ? v0 : 0.f;
            s_aqk[i * LDA + j + 1] = (j + 1 <= i) ? v1 : 0.f;
        });
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    // diagonal blocks directly (Delta is dead: its slot takes the result), then centre u^ on its block end
    if (!block_is_fast(s_fastw, threadIdx.x >> 7)) {
        float al[BT];
        block_alphas(al, fG);
        auto none = [](int, int) { return 0.f; };
        auto sink = [](int, int, float) {};
        diag_sweep<false, false, true, false>(
            al, [&](int i, int i0, float (&row)[BT]) { prow16_f32(s_aqk, LDA, i, i0, row); },
            [&](int j, int c) { return s_un[j * LDP + c]; }, none,
            [&](int i, int c, float v) { s_dl[i * LDP + c] = v; }, sink);
    }
    {
        const int c = threadIdx.x & (DP - 1), i0 = (threadIdx.x >> 7) * BT;
        const float Gend = s_G[(i0 + BT - 1) * LDP + c];
#pragma unroll
        for (int k = 0; k < BT; ++k) s_un[(i0 + k) * LDP + c] *= __expf(Gend - s_G[(i0 + k) * LDP + c]);
    }
    cp_wait<0>();
    __syncthreads();
    SD_PHASE(p.g, ph);
    float acc[NT128][4];
    acc_zero<NT128>(acc);
    const int r0 = Tile64<DP>::r0(), n0 = Tile64<DP>::n0();
    warp_mma<NT128>(acc, r0, n0, 0, CL, [&](int i, int k) { return s_kh[i * LDP + k]; },
                [&](int k, int n) { return s_st0[n * LDH + k]; });
    warp_mma<NT128>(acc, r0, n0, 0, CL, [&](int i, int k) { return s_kh[i * LDP + CL + k]; },
                [&](int k, int n) { return s_st1[n * LDH + k]; });
    // a fast diagonal block is one more Horner step; the sum is then referenced to the block end
    const bool fast = block_is_fast(s_fastw, r0 / BT);
    for (int J = 0; J * BT < r0 + (fast ? BT : 0); ++J) {
        scale_acc<NT128>(acc, s_beta + J * DP, n0);
        warp_mma<NT128>(acc, r0, n0, J * BT, J * BT + BT, [&](int i, int k) { return s_aqk[i * LDA + k]; },
                    [&](int k, int n) { return s_un[k * LDP + n]; });
    }
    SD_PHASE(p.g, ph);
    __syncthreads();   // every warp has read k^ as an operand: d takes its place for the exterior half below
    float* gd = panel_ptr(p.Dprim, ch.gi);
    const int ref = fast ? r0 + BT - 1 : r0 - 1;   // row whose prefix the accumulated sum is referenced to
    warp_epi<NT128>(acc, r0, n0, [&](int i, int j, float v0, float v1) {
        float2 kh = *reinterpret_cast<const float2*>(s_kh + i * LDP + j);
        float2 G = *reinterpret_cast<const float2*>(s_G + i * LDP + j);
        float2 Gp = make_float2(0.f, 0.f), dg = make_float2(0.f, 0.f);
        if (ref >= 0) Gp = *reinterpret_cast<const float2*>(s_G + ref * LDP + j);
        if (!fast) dg = *reinterpret_cast<const float2*>(s_dl + i * LDP + j);
        const float2 act = make_float2(__expf(G.x - Gp.x) * v0 + dg.x, __expf(G.y - Gp.y) * v1 + dg.y);
        const float2 d = make_float2(kh.x + act.x, kh.y + act.y);
        *reinterpret_cast<float2*>(gd + i * DP + j) = d;
        *reinterpret_cast<float2*>(s_kh + i * LDP + j) = PRED ? act : d;
    });
    __syncthreads();
    SD_PHASE(p.g, ph);
    if (PRED) {   // the predictor-only entry returns the frame action and the update, and stops here
        const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
        const float* gDelta = panel_ptr(p.Delta, ch.gi);
#pragma unroll
        for (int pp = 0; pp < ROW_PASSES; ++pp) {
            const int i = lr + ROWS_PER_PASS * pp;
            float a[8], dl[8];
            load8_smem(s_kh, i, c0, a);
            load8_panel(gDelta, i, c0, dl);
            store8_bf16<FAST>(p.action, p.g, ch, i, c0, r, a);
            store8_bf16<FAST>(p.update, p.g, ch, i, c0, r, dl);
        }
        return;
    }
    // ---- exterior half: the slots of the primal half take the panels of the exterior preparation ----
    float* s_xr = s_un;     // chi rowG   (block-centred row operand)
    float* s_er = s_dl;     // -e rowG
    float* s_d = s_kh;      // d itself for the diagonal rows, then the column operand d col
    float* s_ag = s_st0;    // -e exp(G)  -> Wd
    float* s_z = s_st1;     // z          -> Ud
    float* s_aed = s_aqk;
    bf16* gAqd = bmat_ptr(p.Aqd, ch.gi);
    float* gAed = mat_ptr(p.Aed, ch.gi);
    // with no block left to the direct evaluation nobody needs d itself: each row is centred as it is read
    const bool all_fast = block_is_fast(s_fastw, 0) && block_is_fast(s_fastw, 1) && block_is_fast(s_fastw, 2) &&
                          block_is_fast(s_fastw, 3);
    {
        const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8, l16 = threadIdx.x & 15;
        const float* gDelta = panel_ptr(p.Delta, ch.gi);
        float* gDt = panel_ptr(p.Dt, ch.gi);
        bf16* gXg = bpanel_ptr(p.Xg, ch.gi);
        float GL[8];
        load8_smem(s_G, CL - 1, c0, GL);
#pragma unroll 1
        for (int pp = 0; pp < ROW_PASSES; ++pp) {
            const int i = balanced_row(lr, pp), i0 = i & ~(BT - 1);
            float uh[8], kh[8], qh[8], dl[8], d[8], er[8], wr[8], v[8], G[8], Gp[8], se[8];
            load8_norm<FAST>(p.k, ch, i, c0, r, kh);
            load8_norm<FAST>(p.q, ch, i, c0, r, qh);
            if (all_fast) {
                // u^ and Delta of this row are still in shared memory (u^ centred on its block end, undone here;
                // the factor is at most exp(60) on a fast block); this thread overwrites exactly these elements below
                float Gi[8], Ge[8];
                load8_smem(s_un, i, c0, uh);
                load8_smem(s_G, i, c0, Gi);
                load8_smem(s_G, i0 + BT - 1, c0, Ge);
#pragma unroll
                for (int e = 0; e < 8; ++e) uh[e] *= __expf(Gi[e] - Ge[e]);
                load8_smem(s_dl, i, c0, dl);
            } else {
                load8_norm<FAST>(p.u, ch, i, c0, r, uh);
                load8_panel(gDelta, i, c0, dl);
            }
            load8_bf16<FAST>(row_bf16(p.er, ch, i), c0, r, p.er.vec, ch.ok(i), er);
            load8_bf16<FAST>(row_bf16(p.wr, ch, i), c0, V, p.wr.vec, ch.ok(i), wr);
            load8_bf16<FAST>(row_bf16(p.v, ch, i), c0, V, p.v.vec, ch.ok(i), v);
            load8_smem(s_d, i, c0, d);
            load8_smem(s_G, i, c0, G);
            load8_smem(s_G, i0 ? i0 - 1 : 0, c0, Gp);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                se[e] = sigmoidf_(er[e]);
                if (i0 == 0) Gp[e] = 0.f;
            }
            Sources src;
            sources_fwd(uh, kh, qh, dl, se, src);
            float xg[8], ag[8], xr[8], ern[8], z[8], dt[8];
            float a[2][8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float ep = __expf(G[e]), rw = __expf(G[e] - Gp[e]);
                xg[e] = src.chi[e] * ep;
                ag[e] = -src.e[e] * ep;
                xr[e] = src.chi[e] * rw;
                ern[e] = -src.e[e] * rw;
                dt[e] = d[e] * __expf(GL[e] - G[e]);
                z[e] = sigmoidf_(wr[e]) * v[e];
                a[0][e] = src.chi[e];
                a[1][e] = -src.e[e];
            }
            store8_smem(s_xr, i, c0, xr);
            store8_smem(s_er, i, c0, ern);
            store8_smem(s_ag, i, c0, ag);
            store8_smem(s_z, i, c0, z);
            store8_panel(gDt, i, c0, dt);
            store8_bpanel(gXg, i, c0, xg);
            store8_bpanel(bpanel_ptr(p.Ag, ch.gi), i, c0, ag);
            store8_bpanel(bpanel_ptr(p.Xr, ch.gi), i, c0, xr);
            store8_bpanel(bpanel_ptr(p.Er, ch.gi), i, c0, ern);
            store8_bpanel(bpanel_ptr(p.DtB, ch.gi), i, c0, dt);
            if (all_fast) {
                float Ge[8], dc[8];
                load8_smem(s_G, i0 + BT - 1, c0, Ge);
#pragma unroll
                for (int e = 0; e < 8; ++e) dc[e] = d[e] * __expf(Ge[e] - G[e]);
                store8_smem(s_d, i, c0, dc);
                store8_bpanel(bpanel_ptr(p.Dcol, ch.gi), i, c0, dc);
            } else {
                store8_bpanel(bpanel_ptr(p.Chi, ch.gi), i, c0, a[0]);
                store8_bpanel(bpanel_ptr(p.Ee, ch.gi), i, c0, a[1]);
            }
            // diagonal blocks that are not fast: exp(G_i - G_j) directly; both pairs share the exponentials
            if (!block_is_fast(s_fastw, i / BT)) {
                float out[2];
                pair_diag_row<2, false>(i, a, G, [&](int j, float (&b)[8]) { load8_smem(s_d, j, c0, b); },
                                        [&](int j, float (&Gj)[8]) { load8_smem(s_G, j, c0, Gj); }, out);
                gAqd[i * CL + i0 + l16] = __float2bfloat16_rn(out[0]);
                s_aed[i * LDA + i0 + l16] = (i0 + l16 < i) ? out[1] : 0.f;
                gAed[i * CL + i0 + l16] = (i0 + l16 < i) ? out[1] : 0.f;
            }
        }
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    // the diagonal rows are done with d itself: centre it on the end of its block, d_j exp(Gend_J - G_j)
    if (!all_fast) {
        for (int idx = threadIdx.x; idx < CL * (DP / 4); idx += NTHREADS) {
            const int j = idx >> 5, c4 = (idx & 31) << 2;
            float4 d = *reinterpret_cast<const float4*>(s_d + j * LDP + c4);
            const float4 G = *reinterpret_cast<const float4*>(s_G + j * LDP + c4);
            const float4 Ge = *reinterpret_cast<const float4*>(s_G + (j | (BT - 1)) * LDP + c4);
            d.x *= __expf(Ge.x - G.x); d.y *= __expf(Ge.y - G.y);
            d.z *= __expf(Ge.z - G.z); d.w *= __expf(Ge.w - G.w);
            *reinterpret_cast<float4*>(s_d + j * LDP + c4) = d;
            bf16* gDc = bpanel_ptr(p.Dcol, ch.gi) + j * DP + c4;
            *reinterpret_cast<__nv_bfloat162*>(gDc) = __floats2bfloat162_rn(d.x, d.y);
            *reinterpret_cast<__nv_bfloat162*>(gDc + 2) = __floats2bfloat162_rn(d.z, d.w);
        }
        __syncthreads();
    }
    {
        auto fc = [&](int j, int k) { return s_d[j * LDP + k]; };
        pair_blocks_tf32<false>(s_M, s_ibeta, s_fastw, [&](int i, int k) { return s_xr[i * LDP + k]; }, fc,
                                [&](int i, int j, float v0, float v1) {
                                    *reinterpret_cast<__nv_bfloat162*>(gAqd + i * CL + j) =
                                        __floats2bfloat162_rn(v0, v1);
                                });
        pair_blocks_tf32<true>(s_M, s_ibeta, s_fastw, [&](int i, int k) { return s_er[i * LDP + k]; }, fc,
                               [&](int i, int j, float v0, float v1) {
                                   *reinterpret_cast<float2*>(s_aed + i * LDA + j) = make_float2(v0, v1);
                                   *reinterpret_cast<float2*>(gAed + i * CL + j) = make_float2(v0, v1);
                               });
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    trisolve_blocked<false, false>(s_aed, -1.f, PanelF32{s_ag, s_z});
    SD_PHASE(p.g, ph);
    s2g_panel_tf32(panel_ptr(p.Wd, ch.gi), s_ag);   // a contraction operand of the state scan
    s2g_panel(panel_ptr(p.Ud, ch.gi), s_z);
    SD_PHASE(p.g, ph);
}

// The output rows y = Xg S_c + tril(Aqd) Z~ are k_output_fwd_tc (sd_output_tc.cuh).

}  // namespace sd
