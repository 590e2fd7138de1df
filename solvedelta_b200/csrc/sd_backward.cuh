// Chunk-parallel backward kernels: one CTA per (stream, chunk).
//
// Pipeline: k_exterior_prep_bwd -> scan(dS, reverse) -> k_exterior_pair_bwd
//           (contractions + per-token source reverse) -> k_primal_bwd (also prepares the dC scan)
//           -> scan(dC, reverse) -> k_predictor_close_bwd (contractions + gate closure).
// Forward locals are recomputed from the raw inputs and the panels the forward
// pass kept (G, Delta, d, Z~, the chunk-entry states and lam).  Gradients
// tolerate BF16 operands, so every contraction here is BF16 x BF16 -> FP32 and
// every panel that only feeds a contraction or a gradient row is BF16 in HBM.
#pragma once
#include "sd_bf16.cuh"
#include "sd_common.cuh"
#include "sd_decay.cuh"
#include "sd_forward.cuh"

namespace sd {

struct BwdParams {
    Geometry g;
    Operand u, h, q, k, v, er, wr, ld, gam, dy;
    // kept by forward (FP32)
    const float *Lam, *Gp, *Delta, *Dprim, *CtCk;
    const float *Npair, *Aed;   // pair matrices N and Aed of the forward pass, [CL][CL]
    const bf16 *Zt, *SCk, *CtCkB, *Aqd;
    const bf16 *Ag, *Xg;           // -e exp(G), chi exp(G): R and R2 of the dS scan
    const bf16 *Xr, *Er, *Dcol;    // block-centred chi rowG, -e rowG, d col (operands of the centred contractions)
    const bf16 *DtB;               // d exp(GL - G)
    const bf16 *Chi, *Ee;          // chi, -e themselves (diagonal blocks on the direct path; only written for those chunks)
    // backward scratch: BF16 contraction operands / scanned panels
    bf16 *Pp, *Qp, *Dyf, *dR, *dSeCk;
    bf16 *DG, *Dd, *Tu, *Khat;
    bf16 *Ppp, *Qpp, *Rneg, *dRr, *dCeCk;
    // partial cotangents (BF16: they are final up to gradient tolerance) and FP32 reductions
    bf16 *duPart, *dkPart, *dGPart, *dDelta, *Xext;
    float *SdS;
    // outputs
    void *du, *dh, *dq, *dk, *dv, *der, *dwr;
    float *dld, *dgam;
};

__device__ __forceinline__ void norm_vjp8(const float (&dxh)[8], const float (&xh)[8], float rstd,
                                          float (&dx)[8]) {
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) dot = fmaf(dxh[e], xh[e], dot);
    dot = row_sum16(dot);
#pragma unroll
    for (int e = 0; e < 8; ++e) dx[e] = (dxh[e] - dot * xh[e]) * rstd;
}

// shared BF16 panel -> dense BF16 global panel
__device__ __forceinline__ void s2g_bpanel(bf16* g, const bf16* sm) {
    for (int idx = threadIdx.x; idx < CL * (DP / 8); idx += NTHREADS) {
        int i = idx >> 4, c8 = (idx & 15) << 3;
        *reinterpret_cast<uint4*>(g + i * DP + c8) = *reinterpret_cast<const uint4*>(sm + i * LDB + c8);
    }
}
// whole BF16 global state [DP][DP] -> shared [DP][LDB], asynchronously
__device__ __forceinline__ void async_bstate(bf16* sm, const bf16* g) {
    for (int idx = threadIdx.x; idx < DP * (DP / 8); idx += NTHREADS) {
        int i = idx >> 4, c8 = (idx & 15) << 3;
        cp16(sm + i * LDB + c8, g + i * DP + c8);
    }
}
__device__ __forceinline__ bf16* bstate_ptr(bf16* base, long long gi) { return base + gi * (long long)(DP * DP); }
__device__ __forceinline__ const bf16* bstate_ptr(const bf16* base, long long gi) {
    return base + gi * (long long)(DP * DP);
}

// Mr[j][i] = scale(i) * M[i][j] for a dense FP32 [CL][CL] matrix in global memory
// (a strictly lower M arrives as the "rows of the transposed system" the solves expect).
template <class FS>
__device__ __forceinline__ void g2s_mat_transposed(float* Mr, const float* M, FS scale) {
    for (int idx = threadIdx.x; idx < CL * (CL / 4); idx += NTHREADS) {
        const int j4 = (idx >> 6) << 2, i = idx & (CL - 1);   // consecutive threads: consecutive i (conflict-free stores)
        const float4 v = *reinterpret_cast<const float4*>(M + i * CL + j4);
        const float sc = scale(i);
        Mr[(j4 + 0) * LDA + i] = sc * v.x;
        Mr[(j4 + 1) * LDA + i] = sc * v.y;
        Mr[(j4 + 2) * LDA + i] = sc * v.z;
        Mr[(j4 + 3) * LDA + i] = sc * v.w;
    }
}

template <int NTW>
__device__ __forceinline__ void epi_store_bsm(float (&acc)[NTW][4], int r0, int n0, bf16* spanel) {
    warp_epi<NTW>(acc, r0, n0, [&](int i, int j, float v0, float v1) {
        *reinterpret_cast<__nv_bfloat162*>(spanel + i * LDB + j) = __floats2bfloat162_rn(v0, v1);
    });
}

// ---------------------------------------------------------------------------
// With Aqd, Aed and Dt = d exp(GL - G) of the forward pass solve the transposed system for
//   P' = (I-Aed)^-T (Aqd^T dy),  Q' = (I-Aed)^-T Dt
// so that the reverse S scan is dR = P' + Q' dS.  Also leaves dy as a dense panel for the scan and the
// next kernel.  (The source panels chi, e and their centred forms come from the forward pass.)
constexpr size_t EXT_PREP_BWD_SMEM = 2 * BSLOT_BYTES + BMAT_BYTES + MAT_BYTES;

// 61 KB of shared memory and few registers: two CTAs share an SM
template <bool FAST, bool MASKED>
__global__ void __launch_bounds__(NTHREADS, 2) k_exterior_prep_bwd(BwdParams p) {
    int ph = 0;
    SD_PHASE(p.g, ph);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* b_dy = reinterpret_cast<bf16*>(smem_raw);
    bf16* b_dt = b_dy + BSLOT_ELEMS;
    bf16* b_aqd = b_dt + BSLOT_ELEMS;
    float* f_aedT = reinterpret_cast<float*>(b_aqd + BMAT_ELEMS);
    const ChunkT<MASKED> ch = chunk_of<MASKED>(p.g, blockIdx.x);
    const int V = p.g.V;
    async_bmat(b_aqd, bmat_ptr(p.Aqd, ch.gi));
    async_bpanel(b_dt, bpanel_ptr(p.DtB, ch.gi));
    cp_commit();
    {
        const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
        bf16* gDyf = bpanel_ptr(p.Dyf, ch.gi);
#pragma unroll
        for (int pp = 0; pp < ROW_PASSES; ++pp) {
            const int i = lr + ROWS_PER_PASS * pp;
            float dy[8];
            load8_bf16<FAST>(row_bf16(p.dy, ch, i), c0, V, p.dy.vec, ch.ok(i), dy);
            store8_bsm(b_dy, i, c0, dy);
            store8_bpanel(gDyf, i, c0, dy);
        }
    }
    g2s_mat_transposed(f_aedT, mat_ptr(p.Aed, ch.gi), [](int) { return 1.f; });
    cp_wait<0>();
    __syncthreads();
    SD_PHASE(p.g, ph);
    {
        float acc[NT128][4];
        acc_zero<NT128>(acc);
        const int r0 = Tile64<DP>::r0(), n0 = Tile64<DP>::n0();
        warp_mma_bf16<NT128, true, false>(acc, b_aqd, LDM, b_dy, LDB, r0, n0, r0, CL);
        __syncthreads();
        SD_PHASE(p.g, ph);
        warp_epi<NT128>(acc, r0, n0, [&](int i, int j, float v0, float v1) {
            *reinterpret_cast<__nv_bfloat162*>(b_dy + i * LDB + j) = __floats2bfloat162_rn(v0, v1);
        });
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    trisolve_blocked<true, false>(f_aedT, -1.f, PanelBF16{b_dy, b_dt});
    SD_PHASE(p.g, ph);
    s2g_bpanel(bpanel_ptr(p.Pp, ch.gi), b_dy);
    s2g_bpanel(bpanel_ptr(p.Qp, ch.gi), b_dt);
    SD_PHASE(p.g, ph);
}

// ---------------------------------------------------------------------------
// Per-token reverse of the sources and of the gate factors of the exterior.
// Writes the final gradients of q, values, erase_raw, write_raw and the
// partial cotangents the predictor reverse still has to complete.
// d chi, -d e, the decay part of d d (all final), dDt and dR are read from the
// shared BF16 panels the contractions of the same CTA just produced.
template <bool FAST, class CH>
__device__ __forceinline__ void sources_bwd_rows(const BwdParams& p, const CH& ch, const bf16* sA1,
                                                 const bf16* sA2, const bf16* sPY, const bf16* sdDt,
                                                 const bf16* sdR) {
    const int r = p.g.r, V = p.g.V;
    const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
    const float* gDelta = panel_ptr(p.Delta, ch.gi);
    const float* gd = panel_ptr(p.Dprim, ch.gi);
    const float* gG = panel_ptr(p.Gp, ch.gi);
    float GL[8];
    load8_panel(gG, CL - 1, c0, GL);
#pragma unroll 1
    for (int pp = 0; pp < ROW_PASSES; ++pp) {
        const int i = lr + ROWS_PER_PASS * pp;
        // the part that does not involve the sources first, stored at once (keeps the live set small)
        float dd[8], xext[8];
        {
            float G[8], d[8], py[8], ddt[8], dg_[8];
            load8_panel(gG, i, c0, G);
            load8_panel(gd, i, c0, d);
            load8_bsm(sPY, i, c0, py);
            load8_bsm(sdDt, i, c0, ddt);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float ep = __expf(G[e]), et = __expf(GL[e] - G[e]);
                dd[e] = py[e] + et * ddt[e];
                xext[e] = ddt[e] * d[e] * et;
                dg_[e] = dd[e] * ep;
            }
            store8_bpanel(bpanel_ptr(p.DG, ch.gi), i, c0, dg_);
            store8_bpanel(bpanel_ptr(p.Dd, ch.gi), i, c0, dd);
            store8_bpanel(bpanel_ptr(p.Xext, ch.gi), i, c0, xext);
        }
        float uh[8], kh[8], qh[8], dl[8], se[8];
        load8_norm<FAST>(p.u, ch, i, c0, r, uh);
        load8_norm<FAST>(p.k, ch, i, c0, r, kh);
        const float rstd_q = load8_norm<FAST>(p.q, ch, i, c0, r, qh);
        load8_panel(gDelta, i, c0, dl);
        load8_bf16<FAST>(row_bf16(p.er, ch, i), c0, r, p.er.vec, ch.ok(i), se);
#pragma unroll
        for (int e = 0; e < 8; ++e) se[e] = sigmoidf_(se[e]);
        Sources src;
        sources_fwd(uh, kh, qh, dl, se, src);
        float dchi[8], de[8], dG[8];
        load8_bsm(sA1, i, c0, dchi);
        load8_bsm(sA2, i, c0, de);
        float dsb = 0.f, dsq = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            de[e] = -de[e];
            // d(-d py + dd (d - k^)) with dd - py = exp(GL - G) dDt: the d terms collapse into xext
            dG[e] = src.chi[e] * dchi[e] + src.e[e] * de[e] + xext[e] - dd[e] * kh[e];
            dsb = fmaf(-de[e], src.phi[e], dsb);
            dsq = fmaf(-dchi[e], src.phi[e], dsq);
        }
        store8_bpanel(bpanel_ptr(p.dGPart, ch.gi), i, c0, dG);
        dsb = row_sum16(dsb);
        dsq = row_sum16(dsq);
        const float inv_den = 1.f / src.den;
        const float dden = -(dsb * src.sb + dsq * src.sq) * inv_den;
        float db[8], dqh[8], dphi[8], duh[8];
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            db[e] = de[e] + dsb * inv_den * uh[e];
            dqh[e] = dchi[e] + dsq * inv_den * uh[e];
            dphi[e] = -de[e] * src.sb - dchi[e] * src.sq + dden * uh[e];
            duh[e] = dsb * inv_den * src.b[e] + dsq * inv_den * qh[e] + dden * src.phi[e];
            dot = fmaf(dphi[e], dl[e], dot);
        }
        dot = row_sum16(dot);
        const float coef = dot * src.s / (RHO * RHO + src.n2);
        float ddl[8], dkp[8], der[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            ddl[e] = src.s * dphi[e] - coef * dl[e];
            dkp[e] = se[e] * db[e] + dd[e];
            der[e] = db[e] * kh[e] * se[e] * (1.f - se[e]);
        }
        float dq[8];
        norm_vjp8(dqh, qh, rstd_q, dq);
        store8_bf16<FAST>(p.dq, p.g, ch, i, c0, r, dq);
        store8_bf16<FAST>(p.der, p.g, ch, i, c0, r, der);
        store8_bpanel(bpanel_ptr(p.duPart, ch.gi), i, c0, duh);
        store8_bpanel(bpanel_ptr(p.dkPart, ch.gi), i, c0, dkp);
        store8_bpanel(bpanel_ptr(p.dDelta, ch.gi), i, c0, ddl);
    }
    // value side: dv = sigmoid(write) dR, d write_raw = dR v sigmoid'(write)
#pragma unroll
    for (int pp = 0; pp < ROW_PASSES; ++pp) {
        const int i = lr + ROWS_PER_PASS * pp;
        float wr[8], v[8], dr[8], dv[8], dwr[8];
        load8_bf16<FAST>(row_bf16(p.wr, ch, i), c0, V, p.wr.vec, ch.ok(i), wr);
        load8_bf16<FAST>(row_bf16(p.v, ch, i), c0, V, p.v.vec, ch.ok(i), v);
        load8_bsm(sdR, i, c0, dr);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float sw = sigmoidf_(wr[e]);
            dv[e] = sw * dr[e];
            dwr[e] = dr[e] * v[e] * sw * (1.f - sw);
        }
        store8_bf16<FAST>(p.dv, p.g, ch, i, c0, V, dv);
        store8_bf16<FAST>(p.dwr, p.g, ch, i, c0, V, dwr);
    }
}

// ---------------------------------------------------------------------------
// Contractions of the exterior reverse step.  With dAqd = tril(dy Z~^T), dAed = stril(dR Z~^T):
//   d chi_i = exp(G_i) (dy S^T)_i + sum_{j<=i} dAqd_ij d_j exp(G_i - G_j)
//   -d e_i  = exp(G_i) (dR S^T)_i + sum_{j<i}  dAed_ij d_j exp(G_i - G_j)
//   ddp_j   = sum_{i>=j} (dAqd_ij chi_i - dAed_ij e_i) exp(G_i - G_j)     (decay part of d d)
//   dDt = Z~ dS_end^T ,  SdS[c] = sum_v S[c][v] dS_end[c][v]
// The decay-weighted sums are block-centred: Horner accumulation over the blocks
// off the diagonal on the tensor cores (the state term enters as the block before
// the first), diagonal blocks directly.  Every operand streams in with cp.async.
// The four results stay in shared memory (over operands that are no longer
// needed) and the per-token reverse of the sources runs on them in the same CTA.
constexpr size_t EXT_PAIR_BWD_SMEM =
    6 * BSLOT_BYTES + 2 * BSTATE_BYTES + 2 * BMAT_BYTES + (NBLK * DP + 16) * sizeof(float);

// acc rows (i = r0+g, r0+g+8) x columns scaled by exp(x_i - ref) with x, ref rows of the prefix panel
template <int NTW, class FX>
__device__ __forceinline__ void epi_scale_store_bsm(float (&acc)[NTW][4], int r0, int n0, bf16* spanel, FX fx) {
    warp_epi<NTW>(acc, r0, n0, [&](int i, int j, float v0, float v1) {
        const float2 f = fx(i, j);
        *reinterpret_cast<__nv_bfloat162*>(spanel + i * LDB + j) = __floats2bfloat162_rn(f.x * v0, f.y * v1);
    });
}

template <bool FAST, bool MASKED>
__global__ void __launch_bounds__(NTHREADS, 1) k_exterior_pair_bwd(BwdParams p) {
    int ph = 0;
    SD_PHASE(p.g, ph);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* b_dy = reinterpret_cast<bf16*>(smem_raw);   // dy      -> d chi
    bf16* b_zt = b_dy + BSLOT_ELEMS;
    bf16* b_dr = b_zt + BSLOT_ELEMS;
    bf16* b_dc = b_dr + BSLOT_ELEMS;                   // d col   -> -d e
    bf16* b_xr = b_dc + BSLOT_ELEMS;                   // chi row -> ddp
    bf16* b_er = b_xr + BSLOT_ELEMS;                   // -e row  -> dDt
    bf16* b_S = b_er + BSLOT_ELEMS;
    bf16* b_dS = b_S + DP * LDB;
    bf16* b_daqd = b_dS + DP * LDB;
    bf16* b_daed = b_daqd + BMAT_ELEMS;
    float* s_beta = reinterpret_cast<float*>(b_daed + BMAT_ELEMS);
    int* s_fastw = reinterpret_cast<int*>(s_beta + NBLK * DP);
    const ChunkT<MASKED> ch = chunk_of<MASKED>(p.g, blockIdx.x);
    const float* gG = panel_ptr(p.Gp, ch.gi);
    auto fG = [&](int i, int c) { return gG[i * DP + c]; };

    async_bpanel(b_dy, bpanel_ptr(p.Dyf, ch.gi));
    async_bpanel(b_dr, bpanel_ptr(p.dR, ch.gi));
    async_bpanel(b_zt, bpanel_ptr(p.Zt, ch.gi));
    cp_commit();
    async_bpanel(b_dc, bpanel_ptr(p.Dcol, ch.gi));
    async_bstate(b_S, bstate_ptr(p.SCk, ch.gi));
    cp_commit();
    async_bpanel(b_xr, bpanel_ptr(p.Xr, ch.gi));
    async_bpanel(b_er, bpanel_ptr(p.Er, ch.gi));
    cp_commit();
    async_bstate(b_dS, bstate_ptr(p.dSeCk, ch.gi));
    cp_commit();
    // what the diagonal sweeps and the per-token reverse read from HBM much later
    prefetch_region(panel_ptr(p.Dprim, ch.gi), CL * DP * 4);
    prefetch_region(panel_ptr(p.Delta, ch.gi), CL * DP * 4);
    prefetch_region(bpanel_ptr(p.Chi, ch.gi), CL * DP * 2);
    prefetch_region(bpanel_ptr(p.Ee, ch.gi), CL * DP * 2);
    prefetch_rows(p.u, ch, 2, p.g.r * 2);
    prefetch_rows(p.k, ch, 2, p.g.r * 2);
    prefetch_rows(p.q, ch, 2, p.g.r * 2);
    prefetch_rows(p.er, ch, 2, p.g.r * 2);
    prefetch_rows(p.wr, ch, 2, p.g.V * 2);
    prefetch_rows(p.v, ch, 2, p.g.V * 2);
    block_decay_tables(s_beta, nullptr, s_fastw, fG);
    cp_wait<3>();
    __syncthreads();
    SD_PHASE(p.g, ph);
    {
        float a1[NT64][4], a2[NT64][4];
        acc_zero<NT64>(a1);
        acc_zero<NT64>(a2);
        const int r0 = Tile64<CL>::r0(), n0 = Tile64<CL>::n0();
        if (n0 <= r0) {
            warp_mma_bf16<NT64, false, true>(a1, b_dy, LDB, b_zt, LDB, r0, n0, 0, DP);
            warp_mma_bf16<NT64, false, true>(a2, b_dr, LDB, b_zt, LDB, r0, n0, 0, DP);
        }
        warp_epi<NT64>(a1, r0, n0, [&](int i, int j, float v0, float v1) {
            *reinterpret_cast<__nv_bfloat162*>(b_daqd + i * LDM + j) =
                __floats2bfloat162_rn((j <= i) ? v0 : 0.f, (j + 1 <= i) ? v1 : 0.f);
        });
        warp_epi<NT64>(a2, r0, n0, [&](int i, int j, float v0, float v1) {
            *reinterpret_cast<__nv_bfloat162*>(b_daed + i * LDM + j) =
                __floats2bfloat162_rn((j < i) ? v0 : 0.f, (j + 1 < i) ? v1 : 0.f);
        });
    }
    cp_wait<2>();
    __syncthreads();
    SD_PHASE(p.g, ph);
    const int r0 = Tile64<DP>::r0(), n0 = Tile64<DP>::n0();
    const int I = r0 / BT;
    // a fast diagonal block is one more Horner step, and the sum is then referenced to the other end of the block
    const bool fast = block_is_fast(s_fastw, I);
    // exp(G_i - G_ref) for the accumulator element pair (i, j), (i, j + 1); ref < 0: the chunk start
    auto row_factor = [&](int i, int j) {
        const int ref = fast ? r0 + BT - 1 : r0 - 1;
        const float2 G = *reinterpret_cast<const float2*>(gG + i * DP + j);
        float2 Gp = make_float2(0.f, 0.f);
        if (ref >= 0) Gp = *reinterpret_cast<const float2*>(gG + ref * DP + j);
        return make_float2(__expf(G.x - Gp.x), __expf(G.y - Gp.y));
    };
    // exp(G_ref - G_j) for rows of block J = I of the anti-causal result
    auto col_factor = [&](int i, int j) {
        const int ref = fast ? r0 - 1 : r0 + BT - 1;
        const float2 G = *reinterpret_cast<const float2*>(gG + i * DP + j);
        float2 Ge = make_float2(0.f, 0.f);
        if (ref >= 0) Ge = *reinterpret_cast<const float2*>(gG + ref * DP + j);
        return make_float2(__expf(Ge.x - G.x), __expf(Ge.y - G.y));
    };
    {
        float a1[NT128][4], a2[NT128][4];
        acc_zero<NT128>(a1);
        acc_zero<NT128>(a2);
        warp_mma_bf16<NT128, false, true>(a1, b_dy, LDB, b_S, LDB, r0, n0, 0, DP);
        warp_mma_bf16<NT128, false, true>(a2, b_dr, LDB, b_S, LDB, r0, n0, 0, DP);
        for (int J = 0; J < I + (fast ? 1 : 0); ++J) {
            scale_acc<NT128>(a1, s_beta + J * DP, n0);
            scale_acc<NT128>(a2, s_beta + J * DP, n0);
            warp_mma_bf16<NT128, false, false>(a1, b_daqd, LDM, b_dc, LDB, r0, n0, J * BT, J * BT + BT);
            warp_mma_bf16<NT128, false, false>(a2, b_daed, LDM, b_dc, LDB, r0, n0, J * BT, J * BT + BT);
        }
        cp_wait<1>();
        __syncthreads();  // nobody reads dy / d col any more: d chi and -d e take their place
        SD_PHASE(p.g, ph);
        epi_scale_store_bsm<NT128>(a1, r0, n0, b_dy, row_factor);
        epi_scale_store_bsm<NT128>(a2, r0, n0, b_dc, row_factor);
    }
    {
        float acc[NT128][4];
        acc_zero<NT128>(acc);
        bool first = true;
        for (int K = NBLK - 1; K >= I + (fast ? 0 : 1); --K) {
            if (!first) scale_acc<NT128>(acc, s_beta + K * DP, n0);
            first = false;
            warp_mma_bf16<NT128, true, false>(acc, b_daqd, LDM, b_xr, LDB, r0, n0, K * BT, K * BT + BT);
            warp_mma_bf16<NT128, true, false>(acc, b_daed, LDM, b_er, LDB, r0, n0, K * BT, K * BT + BT);
        }
        cp_wait<0>();
        __syncthreads();  // chi row is free: the decay part of d d takes its place
        SD_PHASE(p.g, ph);
        epi_scale_store_bsm<NT128>(acc, r0, n0, b_xr, col_factor);
    }
    {
        float acc[NT128][4];
        acc_zero<NT128>(acc);
        warp_mma_bf16<NT128, false, true>(acc, b_zt, LDB, b_dS, LDB, r0, n0, 0, DP);
        epi_store_bsm<NT128>(acc, r0, n0, b_er);  // -e row was last read before the barrier above
    }
    {
        const int c = threadIdx.x >> 2, qt = threadIdx.x & 3;  // four lanes per state row
        float acc = 0.f;
#pragma unroll
        for (int v8 = 0; v8 < DP / 4; v8 += 8) {
            float a[8], b[8];
            load8_bsm(b_S, c, qt * (DP / 4) + v8, a);
            load8_bsm(b_dS, c, qt * (DP / 4) + v8, b);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc = fmaf(a[e], b[e], acc);
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        if (qt == 0) p.SdS[ch.gi * DP + c] = acc;
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    if (!block_is_fast(s_fastw, threadIdx.x >> 7)) {
        // diagonal blocks that are not fast, one thread per (channel, block): d, chi, -e themselves from HBM (L2)
        const float* gd = panel_ptr(p.Dprim, ch.gi);
        const bf16* gChi = bpanel_ptr(p.Chi, ch.gi);
        const bf16* gEe = bpanel_ptr(p.Ee, ch.gi);
        float al[BT];
        block_alphas(al, fG);
        auto add_to = [](bf16* panel) {
            return [panel](int i, int c, float v) {
                bf16* q = panel + i * LDB + c;
                *q = __float2bfloat16_rn(__bfloat162float(*q) + v);
            };
        };
        auto fd = [&](int j, int c) { return gd[j * DP + c]; };
        diag_sweep<false, false, true, true>(
            al, [&](int i, int i0, float (&row)[BT]) { prow16_bf16(b_daqd, LDM, i, i0, row); }, fd,
            [&](int i, int c) { return __bfloat162float(gChi[i * DP + c]); }, add_to(b_dy), add_to(b_xr));
        diag_sweep<false, true, true, true>(
            al, [&](int i, int i0, float (&row)[BT]) { prow16_bf16(b_daed, LDM, i, i0, row); }, fd,
            [&](int i, int c) { return __bfloat162float(gEe[i * DP + c]); }, add_to(b_dc), add_to(b_xr));
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    sources_bwd_rows<FAST>(p, ch, b_dy, b_dc, b_xr, b_er, b_dr);
    SD_PHASE(p.g, ph);
}

// ---------------------------------------------------------------------------
// Predictor-only reverse pass (the sub-owner entry, causallsso/ops/residual_frame/predictor.py:129-282):
// the cotangents of the frame action d - k^ and of the update Delta come from the caller instead of
// from the exterior kernels.  This kernel writes the panels that k_primal_bwd and
// k_predictor_close_bwd otherwise receive from k_exterior_pair_bwd:
//   Dd = d_action, DG = d_action exp(G), dDelta = d_update, dGPart = d_action (d - k^)  (d(d_i)/dG_i),
// and zeros for what only the exterior contributes (dkPart: d - k^ has no direct k^ term; duPart, Xext, SdS).
template <bool MASKED>
__global__ void __launch_bounds__(NTHREADS) k_predictor_seed_bwd(BwdParams p, Operand dact, Operand dupd, Operand act) {
    const ChunkT<MASKED> ch = chunk_of<MASKED>(p.g, blockIdx.x);
    const int r = p.g.r;
    const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
    const float* gG = panel_ptr(p.Gp, ch.gi);
    const float zero[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int pp = 0; pp < ROW_PASSES; ++pp) {
        const int i = lr + ROWS_PER_PASS * pp;
        float dd[8], a[8], dup[8], G[8], dg[8], dgp[8];
        load8_bf16<false>(row_bf16(dact, ch, i), c0, r, dact.vec, ch.ok(i) && dact.ptr != nullptr, dd);
        load8_bf16<false>(row_bf16(dupd, ch, i), c0, r, dupd.vec, ch.ok(i) && dupd.ptr != nullptr, dup);
        load8_bf16<false>(row_bf16(act, ch, i), c0, r, act.vec, ch.ok(i), a);
        load8_panel(gG, i, c0, G);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            dg[e] = dd[e] * __expf(G[e]);
            dgp[e] = dd[e] * a[e];
        }
        store8_bpanel(bpanel_ptr(p.DG, ch.gi), i, c0, dg);
        store8_bpanel(bpanel_ptr(p.Dd, ch.gi), i, c0, dd);
        store8_bpanel(bpanel_ptr(p.dDelta, ch.gi), i, c0, dup);
        store8_bpanel(bpanel_ptr(p.dGPart, ch.gi), i, c0, dgp);
        store8_bpanel(bpanel_ptr(p.dkPart, ch.gi), i, c0, zero);
        store8_bpanel(bpanel_ptr(p.duPart, ch.gi), i, c0, zero);
        store8_bpanel(bpanel_ptr(p.Xext, ch.gi), i, c0, zero);
    }
    if (threadIdx.x < DP) p.SdS[ch.gi * DP + threadIdx.x] = 0.f;
}

// ---------------------------------------------------------------------------
// Reverse of the primal address d = k^ + C_t^T k^, and preparation of the dC
// scan.  With dd the cotangent of d, DG = dd exp(G), Aqk = tril(K^ Delta^T):
//   dAqk_ij = sum_c dd_ic u^_jc exp(G_ic - G_jc)   (j <= i)
//   dk^ = dkPart + DG Ct + dAqk Delta                                   -> final dkeys
//   dDelta_loc = dDelta_src + dAqk^T K^
//   t_u[j] = sum_{i>=j} Aqk_ij dd_i exp(G_i - G_j)                      (-> d u^, d log decay)
//   P'' = (I+Lm)^-T dDelta_loc,  Q'' = (I+Lm)^-T Ubar,  Rneg = -gamma U~.
// dAqk and t_u are block-centred (tensor cores off the diagonal blocks, direct
// evaluation on them); Lm = gamma N comes from the pair matrix the forward pass kept.
constexpr size_t PRIMAL_BWD_SMEM = 7 * BSLOT_BYTES + BSTATE_BYTES + 2 * BMAT_BYTES + MAT_BYTES +
                                   (3 * CL + 4 * CL + NBLK * DP + 16) * sizeof(float) +
                                   (3 + NBLK) * DP * sizeof(bf16);

template <bool FAST, bool MASKED, bool PRED = false>
__global__ void __launch_bounds__(NTHREADS, 1) k_primal_bwd(BwdParams p) {
    int ph = 0;
    SD_PHASE(p.g, ph);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* b_uc = reinterpret_cast<bf16*>(smem_raw);   // u^ col
    bf16* b_ur = b_uc + BSLOT_ELEMS;   // u^ itself (diagonal blocks), then t_u off the diagonal blocks
    bf16* b_ub = b_ur + BSLOT_ELEMS;   // Ubar, then Q''
    bf16* b_kh = b_ub + BSLOT_ELEMS;
    bf16* b_dl = b_kh + BSLOT_ELEMS;   // Delta, then dDelta_loc / P''
    bf16* b_dg = b_dl + BSLOT_ELEMS;   // dd exp(G)
    bf16* b_ddr = b_dg + BSLOT_ELEMS;  // dd rowG
    bf16* b_Ct = b_ddr + BSLOT_ELEMS;  // arrives after the pair phase; until then its place holds
    float* s_G = reinterpret_cast<float*>(b_Ct);   // the FP32 chunk prefix [CL][LDP] for the diagonal blocks
    static_assert(size_t(CL) * LDP * 4 <= BSTATE_BYTES, "the prefix panel fits in the state slot");
    bf16* b_aqk = b_Ct + DP * LDB;
    bf16* b_daqk = b_aqk + BMAT_ELEMS;
    float* f_lmT = reinterpret_cast<float*>(b_daqk + BMAT_ELEMS);
    float* s_rk = f_lmT + MAT_FLOATS;   // 1/|k| per row
    float* s_ru = s_rk + CL;            // 1/|u| per row
    float* s_gam = s_ru + CL;
    float* s_dot = s_gam + CL;          // [CL][4] partial dots of the norm VJP
    float* s_beta = s_dot + 4 * CL;
    int* s_fastw = reinterpret_cast<int*>(s_beta + NBLK * DP);
    bf16* s_Mb = reinterpret_cast<bf16*>(s_fastw + 16);
    bf16* s_ibeta_b = s_Mb + 3 * DP;
    const ChunkT<MASKED> ch = chunk_of<MASKED>(p.g, blockIdx.x);
    const int r = p.g.r;
    const float* gG = panel_ptr(p.Gp, ch.gi);
    const bf16* gDd = bpanel_ptr(p.Dd, ch.gi);
    auto fG = [&](int i, int c) { return gG[i * DP + c]; };

    async_bpanel(b_dg, bpanel_ptr(p.DG, ch.gi));
    async_panel_f32(s_G, gG);
    cp_commit();
    // read much later: the partial cotangents of the exterior and the pair matrix of the forward pass
    prefetch_region(bpanel_ptr(p.dkPart, ch.gi), CL * DP * 2);
    prefetch_region(bpanel_ptr(p.dDelta, ch.gi), CL * DP * 2);
    prefetch_region(mat_ptr(p.Npair, ch.gi), CL * CL * 4);
    load_gamma(p.gam, ch, s_gam);
    block_decay_tables(s_beta, nullptr, s_fastw, fG);
    {   // BF16 copy of 1 / beta for the fast diagonal pair blocks (0 where the block is not fast)
        const int J = threadIdx.x >> 7, c = threadIdx.x & (DP - 1);
        const float d = fG(BT * J + BT - 1, c) - (J ? fG(BT * J - 1, c) : 0.f);
        s_ibeta_b[threadIdx.x] = __float2bfloat16_rn(d >= -FAST_BLOCK_NATS ? __expf(-d) : 0.f);
    }
    pair_block_scales_bf16(s_Mb, fG);
    {
        const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
        const float* gDelta = panel_ptr(p.Delta, ch.gi);
        bf16* gKhat = bpanel_ptr(p.Khat, ch.gi);
        bf16* gR = bpanel_ptr(p.Rneg, ch.gi);
        float GL[8];
        load8_panel(gG, CL - 1, c0, GL);
#pragma unroll 1
        for (int pp = 0; pp < ROW_PASSES; ++pp) {
            const int i = lr + ROWS_PER_PASS * pp, i0 = i & ~(BT - 1);
            float uh[8], kh[8], G[8], E[8], Gp[8], Ge[8], dl[8], dd[8];
            const float ru = load8_norm<FAST, PRED>(p.u, ch, i, c0, r, uh);
            const float rk = load8_norm<FAST, PRED>(p.k, ch, i, c0, r, kh);
            load8_panel(gG, i, c0, G);
            load8_panel(gG, i > 0 ? i - 1 : 0, c0, E);  // E = G of the previous row (0 for the first)
            load8_panel(gG, i0 ? i0 - 1 : 0, c0, Gp);
            load8_panel(gG, i0 + BT - 1, c0, Ge);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                E[e] = (i > 0 ? E[e] : 0.f) - ch.eoff(i);
                Gp[e] = i0 ? Gp[e] : 0.f;
            }
            load8_panel(gDelta, i, c0, dl);
            load8_bpanel(gDd, i, c0, dd);
            const float gm = ch.ok(i) ? *row_f32(p.gam, ch, i) : 0.f;
            float uc[8], ub[8], rn[8], ddr[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                uc[e] = uh[e] * __expf(Ge[e] - G[e]);
                ub[e] = uh[e] * __expf(GL[e] - G[e]);
                rn[e] = -gm * uh[e] * __expf(E[e]);
                ddr[e] = dd[e] * __expf(G[e] - Gp[e]);
            }
            store8_bsm(b_uc, i, c0, uc);
            store8_bsm(b_ur, i, c0, uh);
            store8_bsm(b_ub, i, c0, ub);
            store8_bsm(b_kh, i, c0, kh);
            store8_bsm(b_dl, i, c0, dl);
            store8_bsm(b_ddr, i, c0, ddr);
            store8_bpanel(gKhat, i, c0, kh);
            store8_bpanel(gR, i, c0, rn);
            if ((threadIdx.x & 15) == 0) {
                s_rk[i] = rk;
                s_ru[i] = ru;
            }
        }
    }
    cp_wait<0>();
    __syncthreads();
    SD_PHASE(p.g, ph);
    // Lm^T = (gamma N)^T from the pair matrix the forward pass kept (read by the solve at the end)
    g2s_mat_transposed(f_lmT, mat_ptr(p.Npair, ch.gi), [&](int i) { return s_gam[i]; });
    {
        const int r0 = Tile64<CL>::r0(), n0 = Tile64<CL>::n0();
        float a1[NT64][4];
        acc_zero<NT64>(a1);
        if (n0 <= r0) warp_mma_bf16<NT64, false, true>(a1, b_kh, LDB, b_dl, LDB, r0, n0, 0, DP);
        warp_epi<NT64>(a1, r0, n0, [&](int i, int j, float v0, float v1) {
            *reinterpret_cast<__nv_bfloat162*>(b_aqk + i * LDM + j) =
                __floats2bfloat162_rn((j <= i) ? v0 : 0.f, (j + 1 <= i) ? v1 : 0.f);
        });
        pair_blocks_bf16<false>(s_Mb, s_ibeta_b, s_fastw, b_ddr, b_uc, [&](int i, int j, float v0, float v1) {
            *reinterpret_cast<__nv_bfloat162*>(b_daqk + i * LDM + j) = __floats2bfloat162_rn(v0, v1);
        });
    }
    {   // diagonal blocks of dAqk that are not fast
        const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8, l16 = threadIdx.x & 15;
        auto fu8 = [&](int j, float (&b)[8]) { load8_bsm(b_ur, j, c0, b); };
        auto fg8 = [&](int j, float (&Gj)[8]) { load8_smem(s_G, j, c0, Gj); };
#pragma unroll 1
        for (int pp = 0; pp < ROW_PASSES; ++pp) {
            const int i = balanced_row(lr, pp), i0 = i & ~(BT - 1);
            if (block_is_fast(s_fastw, i / BT)) continue;
            float a[1][8], G[8], out[1];
            load8_smem(s_G, i, c0, G);
            load8_bpanel(gDd, i, c0, a[0]);
            pair_diag_row<1, false>(i, a, G, fu8, fg8, out);
            b_daqk[i * LDM + i0 + l16] = __float2bfloat16_rn(out[0]);
        }
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    async_bstate(b_Ct, bstate_ptr(p.CtCkB, ch.gi));   // the prefix panel is dead: the state takes its place
    cp_commit();
    const int r0 = Tile64<DP>::r0(), n0 = Tile64<DP>::n0();
    float accd[NT128][4];  // dAqk^T K^  (added to dDelta_src below)
    acc_zero<NT128>(accd);
    warp_mma_bf16<NT128, true, false>(accd, b_daqk, LDM, b_kh, LDB, r0, n0, r0, CL);
    const bool fast = block_is_fast(s_fastw, r0 / BT);
    {   // t_u: Horner from the chunk end (a fast diagonal block is its last step), then exp(G_ref - G_j)
        float acc[NT128][4];
        acc_zero<NT128>(acc);
        bool first = true;
        for (int K = NBLK - 1; K * BT >= r0 + (fast ? 0 : BT); --K) {
            if (!first) scale_acc<NT128>(acc, s_beta + K * DP, n0);
            first = false;
            warp_mma_bf16<NT128, true, false>(acc, b_aqk, LDM, b_ddr, LDB, r0, n0, K * BT, K * BT + BT);
        }
        const int ref = fast ? r0 - 1 : r0 + BT - 1;
        epi_scale_store_bsm<NT128>(acc, r0, n0, b_ur, [&](int i, int j) {
            const float2 G = *reinterpret_cast<const float2*>(gG + i * DP + j);
            float2 Ge = make_float2(0.f, 0.f);
            if (ref >= 0) Ge = *reinterpret_cast<const float2*>(gG + ref * DP + j);
            return make_float2(__expf(Ge.x - G.x), __expf(Ge.y - G.y));
        });
    }
    cp_wait<0>();
    __syncthreads();
    {
        // dk^ and its norm VJP, in accumulator layout
        float acc[NT128][4];
        acc_zero<NT128>(acc);
        warp_mma_bf16<NT128, false, false>(acc, b_dg, LDB, b_Ct, LDB, r0, n0, 0, DP);
        warp_mma_bf16<NT128, false, false>(acc, b_daqk, LDM, b_dl, LDB, r0, n0, 0, r0 + 16);
        const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
        const int ia = r0 + g, ib = ia + 8;
        const bf16* gkp = bpanel_ptr(p.dkPart, ch.gi);
        const __nv_bfloat16* ka = row_bf16(p.k, ch, ia);
        const __nv_bfloat16* kb = row_bf16(p.k, ch, ib);
        const float rka = s_rk[ia], rkb = s_rk[ib];
        float kha[NT128][2], khb[NT128][2];
        float dota = 0.f, dotb = 0.f;
#pragma unroll
        for (int nt = 0; nt < NT128; ++nt) {
            const int j = n0 + nt * 8 + 2 * t;
            float2 pa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gkp + ia * DP + j));
            float2 pb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gkp + ib * DP + j));
            acc[nt][0] += pa.x; acc[nt][1] += pa.y;
            acc[nt][2] += pb.x; acc[nt][3] += pb.y;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                kha[nt][e] = (ch.ok(ia) && j + e < r) ? __bfloat162float(ka[j + e]) * rka : 0.f;
                khb[nt][e] = (ch.ok(ib) && j + e < r) ? __bfloat162float(kb[j + e]) * rkb : 0.f;
            }
            dota = fmaf(acc[nt][0], kha[nt][0], fmaf(acc[nt][1], kha[nt][1], dota));
            dotb = fmaf(acc[nt][2], khb[nt][0], fmaf(acc[nt][3], khb[nt][1], dotb));
        }
        dota += __shfl_xor_sync(0xffffffffu, dota, 1);
        dota += __shfl_xor_sync(0xffffffffu, dota, 2);
        dotb += __shfl_xor_sync(0xffffffffu, dotb, 1);
        dotb += __shfl_xor_sync(0xffffffffu, dotb, 2);
        const int nq = threadIdx.x >> 7;  // column quarter of this warp
        if (t == 0) {
            s_dot[ia * 4 + nq] = dota;
            s_dot[ib * 4 + nq] = dotb;
        }
        __syncthreads();
    SD_PHASE(p.g, ph);
        dota = (s_dot[ia * 4] + s_dot[ia * 4 + 1]) + (s_dot[ia * 4 + 2] + s_dot[ia * 4 + 3]);
        dotb = (s_dot[ib * 4] + s_dot[ib * 4 + 1]) + (s_dot[ib * 4 + 2] + s_dot[ib * 4 + 3]);
        __nv_bfloat16* dk = reinterpret_cast<__nv_bfloat16*>(p.dk);
        __nv_bfloat16* rowa = dk + (((long long)ch.b * p.g.T + ch.t0 + ia) * p.g.H + ch.hh) * (long long)r;
        __nv_bfloat16* rowb = dk + (((long long)ch.b * p.g.T + ch.t0 + ib) * p.g.H + ch.hh) * (long long)r;
#pragma unroll
        for (int nt = 0; nt < NT128; ++nt) {
            const int j = n0 + nt * 8 + 2 * t;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                if (j + e < r) {
                    // rows that came in as unit vectors get the gradient of the row itself (no projection)
                    const float va = PRED ? acc[nt][e] : (acc[nt][e] - dota * kha[nt][e]) * rka;
                    const float vb = PRED ? acc[nt][2 + e] : (acc[nt][2 + e] - dotb * khb[nt][e]) * rkb;
                    if (ia < ch.nvalid) rowa[j + e] = __float2bfloat16_rn(ch.ok(ia) ? va : 0.f);
                    if (ib < ch.nvalid) rowb[j + e] = __float2bfloat16_rn(ch.ok(ib) ? vb : 0.f);
                }
            }
        }
    }
    // every contraction that reads b_dl (Delta) is done: reuse it for dDelta_loc
    __syncthreads();
    SD_PHASE(p.g, ph);
    {   // diagonal blocks of t_u that are not fast, one thread per (channel, block); the finished panel goes to HBM
        bf16* gTu = bpanel_ptr(p.Tu, ch.gi);
        if (block_is_fast(s_fastw, threadIdx.x >> 7)) {
            const int c = threadIdx.x & (DP - 1), j0 = (threadIdx.x >> 7) * BT;
#pragma unroll
            for (int k = 0; k < BT; ++k) gTu[(j0 + k) * DP + c] = b_ur[(j0 + k) * LDB + c];
        } else {
            float al[BT];
            block_alphas(al, fG);
            auto none = [](int, int) { return 0.f; };
            auto sink = [](int, int, float) {};
            diag_sweep<false, false, false, true>(
                al, [&](int i, int i0, float (&row)[BT]) { prow16_bf16(b_aqk, LDM, i, i0, row); }, none,
                [&](int i, int c) { return __bfloat162float(gDd[i * DP + c]); }, sink,
                [&](int j, int c, float v) {
                    gTu[j * DP + c] = __float2bfloat16_rn(__bfloat162float(b_ur[j * LDB + c]) + v);
                });
        }
    }
    {
        const bf16* gdd = bpanel_ptr(p.dDelta, ch.gi);
        warp_epi<NT128>(accd, r0, n0, [&](int i, int j, float v0, float v1) {
            float2 src = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gdd + i * DP + j));
            *reinterpret_cast<__nv_bfloat162*>(b_dl + i * LDB + j) = __floats2bfloat162_rn(src.x + v0, src.y + v1);
        });
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    trisolve_blocked<true, false>(f_lmT, 1.f, PanelBF16{b_dl, b_ub});
    SD_PHASE(p.g, ph);
    s2g_bpanel(bpanel_ptr(p.Ppp, ch.gi), b_dl);
    s2g_bpanel(bpanel_ptr(p.Qpp, ch.gi), b_ub);
    SD_PHASE(p.g, ph);
}

// ---------------------------------------------------------------------------
// Last kernel of the reverse pass: the contractions that need the scanned
// dRr / dC, then the gate closure, in one CTA.
//   dUbar = Delta dC_end ,  dUt = -gamma (dRr Ct^T) ,
//   dgamma = rowsum(dRr * (h - U~ Ct - stril(N) Delta)) ,
//   t_i[i] = sum_{j<i} dN_ij u^_j exp(E_i - G_j) ,  t_j[j] = sum_{i>j} dN_ij u^_i exp(E_i - G_j)
//   with dN = -gamma stril(dRr Delta^T),   CdC[c] = sum_a Ct[c][a] dCt_end[c][a];
// then d u^, dG, dE are assembled per token and
//   d log_decay = -dE + reverse_cumsum(dG), with dG[last] += dGL.
// t_i and t_j are block-centred (tensor cores off the diagonal blocks, direct
// evaluation on them); N comes from the forward pass.  Writes the final gradients of u, h, gamma and
// log_decay.  The four contraction results and the three FP32 closure panels
// overlay operands that are dead by then.
constexpr size_t PRED_CLOSE_BWD_SMEM = 5 * BSLOT_BYTES + 2 * BMAT_BYTES + 3 * size_t(CL) * LDP * 4 +
                                       (2 * CL + 4 * CL + DP + NBLK * DP + 16) * sizeof(float) +
                                       6 * DP * sizeof(bf16);
static_assert(3 * size_t(CL) * LDP * 4 >= 2 * BSTATE_BYTES, "closure panels overlay both BF16 states");

template <bool FAST, bool MASKED, bool PRED = false>
__global__ void __launch_bounds__(NTHREADS, 1) k_predictor_close_bwd(BwdParams p) {
    int ph = 0;
    SD_PHASE(p.g, ph);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* b_ur = reinterpret_cast<bf16*>(smem_raw);   // u^ rowE -> dUbar
    bf16* b_uc = b_ur + BSLOT_ELEMS;                   // u^ col  -> dUt
    bf16* b_dl = b_uc + BSLOT_ELEMS;                   // Delta   -> t_i
    bf16* b_dr = b_dl + BSLOT_ELEMS;                   // dRr (kept)
    bf16* b_tj = b_dr + BSLOT_ELEMS;                   // t_j
    bf16* b_N = b_tj + BSLOT_ELEMS;
    bf16* b_dN = b_N + BMAT_ELEMS;
    unsigned char* region = reinterpret_cast<unsigned char*>(b_dN + BMAT_ELEMS);
    bf16* b_Ct = reinterpret_cast<bf16*>(region);      // Ct, dC  -> dG, dE, X (FP32)
    bf16* b_dC = b_Ct + DP * LDB;
    float* s_dG = reinterpret_cast<float*>(region);
    float* s_dE = s_dG + CL * LDP;
    float* s_X = s_dE + CL * LDP;
    float* s_gam = s_X + CL * LDP;
    float* s_ru = s_gam + CL;    // 1/|u| per row
    float* s_dot = s_ru + CL;    // [CL][4]
    float* s_cdc = s_dot + 4 * CL;  // [DP]
    float* s_beta = s_cdc + DP;
    int* s_fastw = reinterpret_cast<int*>(s_beta + NBLK * DP);
    bf16* s_Mb = reinterpret_cast<bf16*>(s_fastw + 16);
    bf16* s_pref = s_Mb + 3 * DP;   // exp(Gprev_I) for I = 1..3: U~ = (u^ rowE) .* pref along channels
    const ChunkT<MASKED> ch = chunk_of<MASKED>(p.g, blockIdx.x);
    const int r = p.g.r;
    const float* gG = panel_ptr(p.Gp, ch.gi);
    auto fG = [&](int i, int c) { return gG[i * DP + c]; };

    async_bpanel(b_dr, bpanel_ptr(p.dRr, ch.gi));
    async_bstate(b_dC, bstate_ptr(p.dCeCk, ch.gi));
    async_bstate(b_Ct, bstate_ptr(p.CtCkB, ch.gi));
    cp_commit();
    load_gamma(p.gam, ch, s_gam);
    block_decay_tables(s_beta, nullptr, s_fastw, fG);
    for (int idx = threadIdx.x; idx < 3 * DP; idx += NTHREADS) {
        const int m = idx >> 7, c = idx & (DP - 1);
        s_pref[idx] = __float2bfloat16_rn(__expf(gG[((m + 1) * BT - 1) * DP + c]));
    }
    {
        const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
        const float* gDelta = panel_ptr(p.Delta, ch.gi);
#pragma unroll 1
        for (int pp = 0; pp < ROW_PASSES; ++pp) {
            const int i = lr + ROWS_PER_PASS * pp, i0 = i & ~(BT - 1);
            float uh[8], G[8], E[8], Gp[8], Ge[8], dl[8];
            const float ru = load8_norm<FAST, PRED>(p.u, ch, i, c0, r, uh);
            load8_panel(gG, i, c0, G);
            load8_panel(gG, i > 0 ? i - 1 : 0, c0, E);  // E = G of the previous row (0 for the first)
            load8_panel(gG, i0 ? i0 - 1 : 0, c0, Gp);
            load8_panel(gG, i0 + BT - 1, c0, Ge);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                E[e] = (i > 0 ? E[e] : 0.f) - ch.eoff(i);
                Gp[e] = i0 ? Gp[e] : 0.f;
            }
            load8_panel(gDelta, i, c0, dl);
            float uc[8], ur[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                uc[e] = uh[e] * __expf(Ge[e] - G[e]);
                ur[e] = uh[e] * __expf(E[e] - Gp[e]);
            }
            store8_bsm(b_uc, i, c0, uc);
            store8_bsm(b_ur, i, c0, ur);
            store8_bsm(b_dl, i, c0, dl);
            if ((threadIdx.x & 15) == 0) s_ru[i] = ru;
        }
    }
    cp_wait<0>();
    __syncthreads();
    SD_PHASE(p.g, ph);
    {
        const int r0 = Tile64<CL>::r0(), n0 = Tile64<CL>::n0();
        float a2[NT64][4];
        acc_zero<NT64>(a2);
        if (n0 <= r0) warp_mma_bf16<NT64, false, true>(a2, b_dr, LDB, b_dl, LDB, r0, n0, 0, DP);
        warp_epi<NT64>(a2, r0, n0, [&](int i, int j, float v0, float v1) {
            float gm = -s_gam[i];
            *reinterpret_cast<__nv_bfloat162*>(b_dN + i * LDM + j) =
                __floats2bfloat162_rn((j < i) ? gm * v0 : 0.f, (j + 1 < i) ? gm * v1 : 0.f);
        });
    }
    {   // N of the forward pass -> BF16 operand
        const float* gN = mat_ptr(p.Npair, ch.gi);
        for (int idx = threadIdx.x; idx < CL * (CL / 4); idx += NTHREADS) {
            const int i = idx >> 4, j4 = (idx & 15) << 2;
            const float4 v = *reinterpret_cast<const float4*>(gN + i * CL + j4);
            *reinterpret_cast<__nv_bfloat162*>(b_N + i * LDM + j4) = __floats2bfloat162_rn(v.x, v.y);
            *reinterpret_cast<__nv_bfloat162*>(b_N + i * LDM + j4 + 2) = __floats2bfloat162_rn(v.z, v.w);
        }
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    const int r0 = Tile64<DP>::r0(), n0 = Tile64<DP>::n0();
    const int I = r0 / BT;
    const bool fast = block_is_fast(s_fastw, I);
    {   // residual rows and dgamma_i = sum_a dRr[i][a] (h[i][a] - (U~ Ct)[i][a] - (N Delta)[i][a])
        float acc[NT128][4];
        acc_zero<NT128>(acc);
        if (I == 0)
            warp_mma_bf16<NT128, false, false>(acc, b_ur, LDB, b_Ct, LDB, r0, n0, 0, DP);
        else
            warp_mma_bf16_kscale<NT128, false>(acc, b_ur, LDB, b_Ct, LDB, r0, n0, 0, DP, s_pref + (I - 1) * DP);
        warp_mma_bf16<NT128, false, false>(acc, b_N, LDM, b_dl, LDB, r0, n0, 0, r0 + 16);
        const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
        const int ia = r0 + g, ib = ia + 8;
        const __nv_bfloat16* ha = row_bf16(p.h, ch, ia);
        const __nv_bfloat16* hb = row_bf16(p.h, ch, ib);
        float suma = 0.f, sumb = 0.f;
#pragma unroll
        for (int nt = 0; nt < NT128; ++nt) {
            const int j = n0 + nt * 8 + 2 * t;
            __nv_bfloat162 da = *reinterpret_cast<const __nv_bfloat162*>(b_dr + ia * LDB + j);
            __nv_bfloat162 db = *reinterpret_cast<const __nv_bfloat162*>(b_dr + ib * LDB + j);
            float2 fa = __bfloat1622float2(da), fb = __bfloat1622float2(db);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float h_a = (ch.ok(ia) && j + e < r) ? __bfloat162float(ha[j + e]) : 0.f;
                float h_b = (ch.ok(ib) && j + e < r) ? __bfloat162float(hb[j + e]) : 0.f;
                suma = fmaf(e ? fa.y : fa.x, h_a - acc[nt][e], suma);
                sumb = fmaf(e ? fb.y : fb.x, h_b - acc[nt][2 + e], sumb);
            }
        }
        suma += __shfl_xor_sync(0xffffffffu, suma, 1);
        suma += __shfl_xor_sync(0xffffffffu, suma, 2);
        sumb += __shfl_xor_sync(0xffffffffu, sumb, 1);
        sumb += __shfl_xor_sync(0xffffffffu, sumb, 2);
        const int nq = threadIdx.x >> 7;  // column quarter of this warp
        if (t == 0) {
            s_dot[ia * 4 + nq] = suma;
            s_dot[ib * 4 + nq] = sumb;
        }
    }
    {   // CdC
        const int c = threadIdx.x >> 2, qt = threadIdx.x & 3;  // four lanes per state row
        float acc = 0.f;
#pragma unroll
        for (int v8 = 0; v8 < DP / 4; v8 += 8) {
            float a[8], b[8];
            load8_bsm(b_Ct, c, qt * (DP / 4) + v8, a);
            load8_bsm(b_dC, c, qt * (DP / 4) + v8, b);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc = fmaf(a[e], b[e], acc);
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        if (qt == 0) s_cdc[c] = acc;
    }
    {
        float aub[NT128][4], aut[NT128][4], ati[NT128][4], atj[NT128][4];
        acc_zero<NT128>(aub);
        acc_zero<NT128>(aut);
        acc_zero<NT128>(ati);
        acc_zero<NT128>(atj);
        // dUbar[j][c] = sum_a Delta[j][a] dCt[c][a] ; dUt[i][c] = -gamma_i sum_a dRr[i][a] Ct[c][a]
        warp_mma_bf16<NT128, false, true>(aub, b_dl, LDB, b_dC, LDB, r0, n0, 0, DP);
        warp_mma_bf16<NT128, false, true>(aut, b_dr, LDB, b_Ct, LDB, r0, n0, 0, DP);
        // t_i: Horner from the chunk start, t_j: from the chunk end; a fast diagonal block is the last step
        for (int J = 0; J < I + (fast ? 1 : 0); ++J) {
            if (J > 0) scale_acc<NT128>(ati, s_beta + J * DP, n0);
            warp_mma_bf16<NT128, false, false>(ati, b_dN, LDM, b_uc, LDB, r0, n0, J * BT, J * BT + BT);
        }
        bool first = true;
        for (int K = NBLK - 1; K >= I + (fast ? 0 : 1); --K) {
            if (!first) scale_acc<NT128>(atj, s_beta + K * DP, n0);
            first = false;
            warp_mma_bf16<NT128, true, false>(atj, b_dN, LDM, b_ur, LDB, r0, n0, K * BT, K * BT + BT);
        }
        __syncthreads();  // every contraction has read its operands: overlay the results
        SD_PHASE(p.g, ph);
        epi_store_bsm<NT128>(aub, r0, n0, b_ur);
        warp_epi<NT128>(aut, r0, n0, [&](int i, int j, float v0, float v1) {
            float gm = -s_gam[i];
            *reinterpret_cast<__nv_bfloat162*>(b_uc + i * LDB + j) = __floats2bfloat162_rn(gm * v0, gm * v1);
        });
        epi_scale_store_bsm<NT128>(ati, r0, n0, b_dl, [&](int i, int j) {   // exp(E_i - G_ref)
            const int ref = fast ? r0 + BT - 1 : r0 - 1;
            float2 E = make_float2(0.f, 0.f), Gp = make_float2(0.f, 0.f);
            if (i > 0) E = *reinterpret_cast<const float2*>(gG + (i - 1) * DP + j);
            E.x -= ch.eoff(i);
            E.y -= ch.eoff(i);
            if (ref >= 0) Gp = *reinterpret_cast<const float2*>(gG + ref * DP + j);
            return make_float2(__expf(E.x - Gp.x), __expf(E.y - Gp.y));
        });
        epi_scale_store_bsm<NT128>(atj, r0, n0, b_tj, [&](int i, int j) {   // exp(G_ref - G_j)
            const int ref = fast ? r0 - 1 : r0 + BT - 1;
            const float2 G = *reinterpret_cast<const float2*>(gG + i * DP + j);
            float2 Ge = make_float2(0.f, 0.f);
            if (ref >= 0) Ge = *reinterpret_cast<const float2*>(gG + ref * DP + j);
            return make_float2(__expf(Ge.x - G.x), __expf(Ge.y - G.y));
        });
    }
    if (threadIdx.x < CL && threadIdx.x < ch.nvalid) {
        const int i = threadIdx.x;
        p.dgam[((long long)ch.b * p.g.T + ch.t0 + i) * p.g.H + ch.hh] =
            ch.ok(i) ? (s_dot[i * 4] + s_dot[i * 4 + 1]) + (s_dot[i * 4 + 2] + s_dot[i * 4 + 3]) : 0.f;
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    if (!block_is_fast(s_fastw, threadIdx.x >> 7)) {
        // diagonal blocks of t_i and t_j that are not fast, one thread per (channel, block)
        float al[BT];
        block_alphas(al, fG);
        auto fu = [&](int j, int c) {
            return (ch.ok(j) && c < r) ? __bfloat162float(row_bf16(p.u, ch, j)[c]) * s_ru[j] : 0.f;
        };
        auto add_to = [](bf16* panel) {
            return [panel](int i, int c, float v) {
                bf16* q = panel + i * LDB + c;
                *q = __float2bfloat16_rn(__bfloat162float(*q) + v);
            };
        };
        diag_sweep<true, true, true, true>(
            al, [&](int i, int i0, float (&row)[BT]) { prow16_bf16(b_dN, LDM, i, i0, row); }, fu, fu,
            add_to(b_dl), add_to(b_tj), ch.reset_rows());
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    {
        const int lr = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 8;
        float GL[8];
        load8_panel(gG, CL - 1, c0, GL);
#pragma unroll 1
        for (int pp = 0; pp < ROW_PASSES; ++pp) {
            const int i = lr + ROWS_PER_PASS * pp;
            float uh[8], G[8], E[8];
            const float rstd_u = load8_norm<FAST, PRED>(p.u, ch, i, c0, r, uh);
            load8_panel(gG, i, c0, G);
            load8_panel(gG, i > 0 ? i - 1 : 0, c0, E);  // E = G of the previous row (0 for the first)
#pragma unroll
            for (int e = 0; e < 8; ++e) E[e] = (i > 0 ? E[e] : 0.f) - ch.eoff(i);
            float dup[8], tpre[8], dub[8], dut[8], ti[8], tj[8], dgp[8], xext[8], drr[8];
            load8_bpanel(bpanel_ptr(p.duPart, ch.gi), i, c0, dup);
            load8_bpanel(bpanel_ptr(p.Tu, ch.gi), i, c0, tpre);
            load8_bpanel(bpanel_ptr(p.dGPart, ch.gi), i, c0, dgp);
            load8_bpanel(bpanel_ptr(p.Xext, ch.gi), i, c0, xext);
            load8_bsm(b_ur, i, c0, dub);
            load8_bsm(b_uc, i, c0, dut);
            load8_bsm(b_dl, i, c0, ti);
            load8_bsm(b_tj, i, c0, tj);
            load8_bsm(b_dr, i, c0, drr);
            float duh[8], dE[8], dG[8], X[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float eE = __expf(E[e]), et = __expf(GL[e] - G[e]);
                const float tu = tpre[e], t_i = ti[e], t_j = tj[e];
                duh[e] = dup[e] + tu + dub[e] * et + dut[e] * eE + t_i + t_j;
                dE[e] = dut[e] * (uh[e] * eE) + uh[e] * t_i;
                X[e] = xext[e] + dub[e] * (uh[e] * et);
                dG[e] = dgp[e] - uh[e] * tu - X[e] - uh[e] * t_j + dE[e];
            }
            store8_smem(s_dG, i, c0, dG);
            store8_smem(s_dE, i, c0, dE);
            store8_smem(s_X, i, c0, X);
            float du[8], dh[8];
            if (PRED) {   // the source rows came in as unit vectors
#pragma unroll
                for (int e = 0; e < 8; ++e) du[e] = duh[e];
            } else {
                norm_vjp8(duh, uh, rstd_u, du);
            }
            const float gm = s_gam[i];
#pragma unroll
            for (int e = 0; e < 8; ++e) dh[e] = gm * drr[e];
            store8_bf16<FAST>(p.du, p.g, ch, i, c0, r, du);
            store8_bf16<FAST>(p.dh, p.g, ch, i, c0, r, dh);
        }
    }
    __syncthreads();
    SD_PHASE(p.g, ph);
    {
        // d log_decay[i] = (suffix sum of dG from row i) + end-of-chunk terms - dE[i], per channel.  Four
        // threads per channel, 16 rows each: segment totals first, then the short suffix walk.
        float* s_tot = reinterpret_cast<float*>(b_N);          // [4][DP] totals of dG, then [4][DP] totals of X
        static_assert(2 * BMAT_BYTES >= 8 * DP * sizeof(float), "segment totals overlay the two pair matrices");
        const int c = threadIdx.x & (DP - 1), seg = threadIdx.x >> 7, i0 = seg * 16;
        float tg = 0.f, tx = 0.f;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            tg += s_dG[(i0 + k) * LDP + c];
            tx += s_X[(i0 + k) * LDP + c];
        }
        s_tot[seg * DP + c] = tg;
        s_tot[(4 + seg) * DP + c] = tx;
        __syncthreads();
        if (c < r) {
            float run = __expf(gG[(CL - 1) * DP + c]) * (p.SdS[ch.gi * DP + c] + s_cdc[c]) +
                        ((s_tot[4 * DP + c] + s_tot[5 * DP + c]) + (s_tot[6 * DP + c] + s_tot[7 * DP + c]));
            for (int s2 = seg + 1; s2 < 4; ++s2) run += s_tot[s2 * DP + c];
            // a masked token has no gradient; nor does the decay of a reset token, which multiplies the zero state
            const unsigned keep = (unsigned)((ch.valid_rows() & ~ch.reset_rows()) >> i0) & 0xffffu;
            float* out = p.dld + (((long long)ch.b * p.g.T + ch.t0 + i0) * p.g.H + ch.hh) * (long long)r + c;
            const long long row_stride = (long long)p.g.H * r;
#pragma unroll
            for (int k = 15; k >= 0; --k) {
                run += s_dG[(i0 + k) * LDP + c];
                if (i0 + k < ch.nvalid) out[k * row_stride] = ((keep >> k) & 1u) ? run - s_dE[(i0 + k) * LDP + c] : 0.f;
            }
        }
    }
    SD_PHASE(p.g, ph);
}

}  // namespace sd
