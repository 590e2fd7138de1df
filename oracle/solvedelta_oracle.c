/*
 * TEST INFRASTRUCTURE -- not part of the shipped product.
 *
 * FP64 CPU restatement of the SolveDelta token recurrence (forward and full
 * vector-Jacobian product).  It is the checker for the CUDA path: only the
 * test-suite, the smoke entry and the benchmark's CPU-baseline leg may call
 * it.  The product library never links or loads this file.
 *
 * Algorithm followed: causallsso/reference.py:82-229 (token loop):
 *   - L2 normalisation of u, q, keys            reference.py:147-149
 *   - reset / valid handling                     reference.py:157-164,216-226
 *   - residual h - C u against the OLD C         reference.py:166-169
 *   - C <- C * diag(exp(log_decay)) + (gamma r) u^T   reference.py:170-173
 *   - radial frame covector phi, denominator     reference.py:175-185
 *   - primal d = k + C_new^T k                   reference.py:191-193
 *   - dual e and query chi (rank-one residual)   reference.py:194-201
 *   - S' = D S ; S = S' + d (z - S'^T e)^T ; o = S^T chi   reference.py:203-215
 * The reverse sweep is the hand-derived adjoint of exactly these statements;
 * it is pinned against torch.autograd through the reference on committed
 * golden vectors (tests/golden).
 *
 * Layouts (all double, contiguous):
 *   u,h,q,k,g(log_decay),erase : [B,T,H,r]     v,write : [B,T,H,V]
 *   gamma : [B,T,H]     C : [B,H,r,r] (prediction = C u)     S : [B,H,r,V]
 *   valid, reset : [B,T] bytes (may be NULL)
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <stdint.h>

#define SDO_RADIUS 0.625
#define SDO_SEG 32

typedef struct {
    int B, T, H, r, V;
} sdo_shape;

static void normalize(const double *x, int n, double *y, double *inv_norm) {
    double s = 0.0;
    for (int i = 0; i < n; ++i) s += x[i] * x[i];
    double nrm = sqrt(s);
    if (nrm < 1e-12) nrm = 1e-12; /* F.normalize eps */
    double inv = 1.0 / nrm;
    for (int i = 0; i < n; ++i) y[i] = x[i] * inv;
    *inv_norm = inv;
}

/* Per-token scratch of forward quantities needed again by the adjoint. */
typedef struct {
    double *uh, *qh, *kh;      /* normalised vectors [r] */
    double iu, iq, ik;         /* 1/norm */
    double *res, *delta, *phi; /* [r] */
    double uu, dd2, fs, den, sb, sq;
    double *b, *d, *e, *chi;   /* [r] */
    double *z, *w;             /* [V] */
} tok_tmp;

static double *dalloc(size_t n) {
    double *p = (double *)calloc(n ? n : 1, sizeof(double));
    return p;
}

static void tok_alloc(tok_tmp *t, int r, int V) {
    t->uh = dalloc(r); t->qh = dalloc(r); t->kh = dalloc(r);
    t->res = dalloc(r); t->delta = dalloc(r); t->phi = dalloc(r);
    t->b = dalloc(r); t->d = dalloc(r); t->e = dalloc(r); t->chi = dalloc(r);
    t->z = dalloc(V); t->w = dalloc(V);
}
static void tok_free(tok_tmp *t) {
    free(t->uh); free(t->qh); free(t->kh); free(t->res); free(t->delta);
    free(t->phi); free(t->b); free(t->d); free(t->e); free(t->chi);
    free(t->z); free(t->w);
}

/*
 * One token of one (batch, head) stream.  Cin/Sin are the states before the
 * token (already reset if requested); Cout/Sout receive the states after it.
 * `o` receives the output row.  Fills `t` with the intermediates.
 */
static void token_forward(int r, int V, const double *u, const double *h,
                          const double *q, const double *k, const double *v,
                          const double *g, const double *erase,
                          const double *write, double gamma, const double *Cin,
                          const double *Sin, double *Cout, double *Sout,
                          double *o, tok_tmp *t) {
    normalize(u, r, t->uh, &t->iu);
    normalize(q, r, t->qh, &t->iq);
    normalize(k, r, t->kh, &t->ik);
    /* residual against the old predictor, then right-decay + rank-one write */
    for (int a = 0; a < r; ++a) {
        double p = 0.0;
        const double *Ca = Cin + (size_t)a * r;
        for (int c = 0; c < r; ++c) p += Ca[c] * t->uh[c];
        t->res[a] = h[a] - p;
        t->delta[a] = gamma * t->res[a];
    }
    for (int a = 0; a < r; ++a) {
        const double *Ca = Cin + (size_t)a * r;
        double *Na = Cout + (size_t)a * r;
        for (int c = 0; c < r; ++c)
            Na[c] = Ca[c] * exp(g[c]) + t->delta[a] * t->uh[c];
    }
    double uu = 0.0, dd2 = 0.0;
    for (int c = 0; c < r; ++c) {
        uu += t->uh[c] * t->uh[c];
        dd2 += t->delta[c] * t->delta[c];
    }
    t->uu = uu; t->dd2 = dd2;
    t->fs = SDO_RADIUS / sqrt(SDO_RADIUS * SDO_RADIUS + uu * dd2);
    double den = 1.0, ub = 0.0, uq = 0.0;
    for (int c = 0; c < r; ++c) {
        t->phi[c] = t->fs * t->delta[c];
        den += t->phi[c] * t->uh[c];
        t->b[c] = erase[c] * t->kh[c];
        ub += t->uh[c] * t->b[c];
        uq += t->uh[c] * t->qh[c];
    }
    t->den = den; t->sb = ub / den; t->sq = uq / den;
    for (int c = 0; c < r; ++c) {
        double acc = t->kh[c];
        for (int a = 0; a < r; ++a) acc += Cout[(size_t)a * r + c] * t->kh[a];
        t->d[c] = acc;
        t->e[c] = t->b[c] - t->phi[c] * t->sb;
        t->chi[c] = t->qh[c] - t->phi[c] * t->sq;
    }
    /* memory: decay rows, erase/read along e, write along d, read along chi */
    for (int j = 0; j < V; ++j) {
        double pred = 0.0;
        for (int c = 0; c < r; ++c)
            pred += exp(g[c]) * Sin[(size_t)c * V + j] * t->e[c];
        t->z[j] = write[j] * v[j];
        t->w[j] = t->z[j] - pred;
    }
    for (int c = 0; c < r; ++c) {
        double a = exp(g[c]);
        for (int j = 0; j < V; ++j)
            Sout[(size_t)c * V + j] = a * Sin[(size_t)c * V + j] + t->d[c] * t->w[j];
    }
    for (int j = 0; j < V; ++j) {
        double acc = 0.0;
        for (int c = 0; c < r; ++c) acc += Sout[(size_t)c * V + j] * t->chi[c];
        o[j] = acc;
    }
}

static inline size_t row4(const sdo_shape *s, int b, int t, int h, int n) {
    return (((size_t)b * s->T + t) * s->H + h) * (size_t)n;
}

int sdo_forward(int B, int T, int H, int r, int V, const double *u,
                const double *h, const double *q, const double *k,
                const double *v, const double *g, const double *erase,
                const double *write, const double *gamma, const double *C0,
                const double *S0, const uint8_t *valid, const uint8_t *reset,
                double *y, double *CT, double *ST) {
    sdo_shape s = {B, T, H, r, V};
    int streams = B * H;
    int failed = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int sidx = 0; sidx < streams; ++sidx) {
        int b = sidx / H, hh = sidx % H;
        size_t nC = (size_t)r * r, nS = (size_t)r * V;
        double *Ca = dalloc(nC), *Cb = dalloc(nC), *Sa = dalloc(nS), *Sb = dalloc(nS);
        tok_tmp tmp; tok_alloc(&tmp, r, V);
        if (!Ca || !Cb || !Sa || !Sb) { failed = 1; }
        else {
            if (C0) memcpy(Ca, C0 + (size_t)sidx * nC, nC * sizeof(double));
            if (S0) memcpy(Sa, S0 + (size_t)sidx * nS, nS * sizeof(double));
            for (int t = 0; t < T; ++t) {
                int ok = valid ? valid[(size_t)b * T + t] != 0 : 1;
                int rs = (reset ? reset[(size_t)b * T + t] != 0 : 0) && ok;
                double *o = y + row4(&s, b, t, hh, V);
                if (!ok) { memset(o, 0, V * sizeof(double)); continue; }
                if (rs) { memset(Ca, 0, nC * sizeof(double)); memset(Sa, 0, nS * sizeof(double)); }
                size_t ir = row4(&s, b, t, hh, r), iv = row4(&s, b, t, hh, V);
                token_forward(r, V, u + ir, h + ir, q + ir, k + ir, v + iv, g + ir,
                              erase + ir, write + iv,
                              gamma[((size_t)b * T + t) * H + hh], Ca, Sa, Cb, Sb, o, &tmp);
                double *x = Ca; Ca = Cb; Cb = x; x = Sa; Sa = Sb; Sb = x;
            }
            if (CT) memcpy(CT + (size_t)sidx * nC, Ca, nC * sizeof(double));
            if (ST) memcpy(ST + (size_t)sidx * nS, Sa, nS * sizeof(double));
        }
        tok_free(&tmp); free(Ca); free(Cb); free(Sa); free(Sb);
    }
    return failed ? -1 : 0;
}

static void normalize_vjp(const double *xh, double inv, const double *dxh, int n,
                          double *dx) {
    /* x_hat = x / |x|  =>  dx = (dxh - (dxh . xh) xh) / |x| */
    double dot = 0.0;
    for (int i = 0; i < n; ++i) dot += dxh[i] * xh[i];
    for (int i = 0; i < n; ++i) dx[i] = (dxh[i] - dot * xh[i]) * inv;
}

/*
 * Adjoint of token_forward.  dC/dS enter holding the cotangent of the states
 * AFTER the token and leave holding the cotangent of the states BEFORE it.
 */
static void token_backward(int r, int V, const double *v, const double *g,
                           const double *erase, const double *write, double gamma,
                           const double *Cin, const double *Sin, const double *Cout,
                           const double *Sout, const tok_tmp *t, const double *dout,
                           double *dC, double *dS, double *du, double *dh, double *dq,
                           double *dk, double *dv, double *dg, double *derase,
                           double *dwrite, double *dgamma, double *wk) {
    double *dchi = wk, *dd = dchi + r, *de = dd + r, *duh = de + r, *dqh = duh + r,
           *dkh = dqh + r, *dphi = dkh + r, *db = dphi + r, *ddelta = db + r,
           *dres = ddelta + r, *dalpha = dres + r, *dw = dalpha + r; /* dw: [V] */
    for (int c = 0; c < r; ++c) { duh[c] = 0; dalpha[c] = 0; }
    /* o = Sout^T chi */
    for (int c = 0; c < r; ++c) {
        double acc = 0.0;
        for (int j = 0; j < V; ++j) {
            acc += Sout[(size_t)c * V + j] * dout[j];
            dS[(size_t)c * V + j] += t->chi[c] * dout[j];
        }
        dchi[c] = acc;
    }
    /* Sout = S' + d w^T */
    for (int j = 0; j < V; ++j) dw[j] = 0.0;
    for (int c = 0; c < r; ++c) {
        double acc = 0.0;
        for (int j = 0; j < V; ++j) {
            acc += dS[(size_t)c * V + j] * t->w[j];
            dw[j] += dS[(size_t)c * V + j] * t->d[c];
        }
        dd[c] = acc;
    }
    /* w = z - S'^T e ; S' = alpha S  (dS currently = dS') */
    for (int c = 0; c < r; ++c) {
        double a = exp(g[c]);
        double acc_e = 0.0, acc_a = 0.0;
        for (int j = 0; j < V; ++j) {
            double sp = a * Sin[(size_t)c * V + j];
            acc_e += sp * (-dw[j]);
            double dsp = dS[(size_t)c * V + j] + t->e[c] * (-dw[j]);
            acc_a += dsp * Sin[(size_t)c * V + j];
            dS[(size_t)c * V + j] = a * dsp;
        }
        de[c] = acc_e;
        dalpha[c] += acc_a;
    }
    for (int j = 0; j < V; ++j) { dwrite[j] = dw[j] * v[j]; dv[j] = dw[j] * write[j]; }
    /* chi = qh - phi sq ; e = b - phi sb */
    double dsq = 0.0, dsb = 0.0, dden = 0.0;
    for (int c = 0; c < r; ++c) {
        dqh[c] = dchi[c];
        db[c] = de[c];
        dphi[c] = -t->sq * dchi[c] - t->sb * de[c];
        dsq -= t->phi[c] * dchi[c];
        dsb -= t->phi[c] * de[c];
    }
    for (int c = 0; c < r; ++c) {
        duh[c] += (dsq / t->den) * t->qh[c] + (dsb / t->den) * t->b[c];
        dqh[c] += (dsq / t->den) * t->uh[c];
        db[c] += (dsb / t->den) * t->uh[c];
    }
    dden = -(dsq * t->sq + dsb * t->sb) / t->den;
    /* d = kh + Cout^T kh */
    for (int a = 0; a < r; ++a) {
        double acc = dd[a];
        for (int c = 0; c < r; ++c) {
            acc += Cout[(size_t)a * r + c] * dd[c];
            dC[(size_t)a * r + c] += t->kh[a] * dd[c];
        }
        dkh[a] = acc;
    }
    /* b = erase * kh */
    for (int c = 0; c < r; ++c) {
        derase[c] = db[c] * t->kh[c];
        dkh[c] += db[c] * erase[c];
    }
    /* den = 1 + phi . uh ; phi = fs delta ; fs = R / sqrt(R^2 + uu dd2) */
    double dfs = 0.0;
    for (int c = 0; c < r; ++c) {
        dphi[c] += dden * t->uh[c];
        duh[c] += dden * t->phi[c];
    }
    for (int c = 0; c < r; ++c) {
        ddelta[c] = t->fs * dphi[c];
        dfs += dphi[c] * t->delta[c];
    }
    double n2 = SDO_RADIUS * SDO_RADIUS + t->uu * t->dd2;
    double dn2 = -0.5 * dfs * t->fs / n2;
    double duu = dn2 * t->dd2, ddd2 = dn2 * t->uu;
    for (int c = 0; c < r; ++c) {
        ddelta[c] += 2.0 * ddd2 * t->delta[c];
        duh[c] += 2.0 * duu * t->uh[c];
    }
    /* Cout = Cin * alpha + delta uh^T  (dC currently = dCout) */
    for (int a = 0; a < r; ++a) {
        double acc = 0.0;
        for (int c = 0; c < r; ++c) {
            double dc = dC[(size_t)a * r + c];
            acc += dc * t->uh[c];
            duh[c] += dc * t->delta[a];
            dalpha[c] += dc * Cin[(size_t)a * r + c];
            dC[(size_t)a * r + c] = dc * exp(g[c]);
        }
        ddelta[a] += acc;
    }
    /* delta = gamma res ; res = h - Cin uh */
    double dgm = 0.0;
    for (int a = 0; a < r; ++a) {
        dgm += ddelta[a] * t->res[a];
        dres[a] = gamma * ddelta[a];
        dh[a] = dres[a];
    }
    *dgamma = dgm;
    for (int a = 0; a < r; ++a) {
        for (int c = 0; c < r; ++c) {
            dC[(size_t)a * r + c] -= dres[a] * t->uh[c];
            duh[c] -= Cin[(size_t)a * r + c] * dres[a];
        }
    }
    for (int c = 0; c < r; ++c) dg[c] = dalpha[c] * exp(g[c]);
    normalize_vjp(t->uh, t->iu, duh, r, du);
    normalize_vjp(t->qh, t->iq, dqh, r, dq);
    normalize_vjp(t->kh, t->ik, dkh, r, dk);
}

/*
 * Full VJP.  dy may not be NULL; dCT/dST may be NULL (treated as zero).
 * Gradients of erase/write are with respect to the post-sigmoid gates, as
 * in the reference's signature.  dC0/dS0 may be NULL.
 */
int sdo_backward(int B, int T, int H, int r, int V, const double *u,
                 const double *h, const double *q, const double *k,
                 const double *v, const double *g, const double *erase,
                 const double *write, const double *gamma, const double *C0,
                 const double *S0, const uint8_t *valid, const uint8_t *reset,
                 const double *dy, const double *dCT, const double *dST,
                 double *du, double *dh, double *dq, double *dk, double *dv,
                 double *dg, double *derase, double *dwrite, double *dgamma,
                 double *dC0, double *dS0) {
    sdo_shape s = {B, T, H, r, V};
    int streams = B * H;
    int nseg = (T + SDO_SEG - 1) / SDO_SEG;
    int failed = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int sidx = 0; sidx < streams; ++sidx) {
        int b = sidx / H, hh = sidx % H;
        size_t nC = (size_t)r * r, nS = (size_t)r * V;
        /* checkpoints at segment starts, and per-token states inside a segment */
        double *ckC = dalloc(nC * (nseg + 1)), *ckS = dalloc(nS * (nseg + 1));
        double *sgC = dalloc(nC * (SDO_SEG + 1)), *sgS = dalloc(nS * (SDO_SEG + 1));
        double *dC = dalloc(nC), *dS = dalloc(nS);
        double *wk = dalloc((size_t)12 * r + V), *otmp = dalloc(V);
        tok_tmp tmp; tok_alloc(&tmp, r, V);
        if (!ckC || !ckS || !sgC || !sgS || !dC || !dS || !wk) { failed = 1; }
        else {
            if (C0) memcpy(ckC, C0 + (size_t)sidx * nC, nC * sizeof(double));
            if (S0) memcpy(ckS, S0 + (size_t)sidx * nS, nS * sizeof(double));
            /* forward pass storing one checkpoint per segment */
            {
                double *Ca = dalloc(nC), *Cb = dalloc(nC), *Sa = dalloc(nS), *Sb = dalloc(nS);
                memcpy(Ca, ckC, nC * sizeof(double)); memcpy(Sa, ckS, nS * sizeof(double));
                for (int t = 0; t < T; ++t) {
                    if (t % SDO_SEG == 0) {
                        memcpy(ckC + nC * (t / SDO_SEG), Ca, nC * sizeof(double));
                        memcpy(ckS + nS * (t / SDO_SEG), Sa, nS * sizeof(double));
                    }
                    int ok = valid ? valid[(size_t)b * T + t] != 0 : 1;
                    int rs = (reset ? reset[(size_t)b * T + t] != 0 : 0) && ok;
                    if (!ok) continue;
                    if (rs) { memset(Ca, 0, nC * sizeof(double)); memset(Sa, 0, nS * sizeof(double)); }
                    size_t ir = row4(&s, b, t, hh, r), iv = row4(&s, b, t, hh, V);
                    token_forward(r, V, u + ir, h + ir, q + ir, k + ir, v + iv, g + ir,
                                  erase + ir, write + iv,
                                  gamma[((size_t)b * T + t) * H + hh], Ca, Sa, Cb, Sb, otmp, &tmp);
                    double *x = Ca; Ca = Cb; Cb = x; x = Sa; Sa = Sb; Sb = x;
                }
                free(Ca); free(Cb); free(Sa); free(Sb);
            }
            if (dCT) memcpy(dC, dCT + (size_t)sidx * nC, nC * sizeof(double));
            if (dST) memcpy(dS, dST + (size_t)sidx * nS, nS * sizeof(double));
            for (int seg = nseg - 1; seg >= 0; --seg) {
                int t0 = seg * SDO_SEG, t1 = t0 + SDO_SEG; if (t1 > T) t1 = T;
                /* recompute the segment, keeping the state before every token
                   (after the reset, if any) and after it */
                memcpy(sgC, ckC + nC * seg, nC * sizeof(double));
                memcpy(sgS, ckS + nS * seg, nS * sizeof(double));
                for (int t = t0; t < t1; ++t) {
                    double *Cin = sgC + nC * (t - t0), *Sin = sgS + nS * (t - t0);
                    double *Cout = Cin + nC, *Sout = Sin + nS;
                    int ok = valid ? valid[(size_t)b * T + t] != 0 : 1;
                    int rs = (reset ? reset[(size_t)b * T + t] != 0 : 0) && ok;
                    if (!ok) { memcpy(Cout, Cin, nC * sizeof(double)); memcpy(Sout, Sin, nS * sizeof(double)); continue; }
                    if (rs) { memset(Cin, 0, nC * sizeof(double)); memset(Sin, 0, nS * sizeof(double)); }
                    size_t ir = row4(&s, b, t, hh, r), iv = row4(&s, b, t, hh, V);
                    token_forward(r, V, u + ir, h + ir, q + ir, k + ir, v + iv, g + ir,
                                  erase + ir, write + iv,
                                  gamma[((size_t)b * T + t) * H + hh], Cin, Sin, Cout, Sout, otmp, &tmp);
                }
                for (int t = t1 - 1; t >= t0; --t) {
                    double *Cin = sgC + nC * (t - t0), *Sin = sgS + nS * (t - t0);
                    double *Cout = Cin + nC, *Sout = Sin + nS;
                    int ok = valid ? valid[(size_t)b * T + t] != 0 : 1;
                    int rs = (reset ? reset[(size_t)b * T + t] != 0 : 0) && ok;
                    size_t ir = row4(&s, b, t, hh, r), iv = row4(&s, b, t, hh, V);
                    size_t ig = ((size_t)b * T + t) * H + hh;
                    if (!ok) {
                        memset(du + ir, 0, r * sizeof(double)); memset(dh + ir, 0, r * sizeof(double));
                        memset(dq + ir, 0, r * sizeof(double)); memset(dk + ir, 0, r * sizeof(double));
                        memset(dg + ir, 0, r * sizeof(double)); memset(derase + ir, 0, r * sizeof(double));
                        memset(dv + iv, 0, V * sizeof(double)); memset(dwrite + iv, 0, V * sizeof(double));
                        dgamma[ig] = 0.0;
                        continue;
                    }
                    /* intermediates of this token (Cin/Sin already hold the reset state) */
                    token_forward(r, V, u + ir, h + ir, q + ir, k + ir, v + iv, g + ir,
                                  erase + ir, write + iv, gamma[ig], Cin, Sin, Cout, Sout, otmp, &tmp);
                    token_backward(r, V, v + iv, g + ir, erase + ir, write + iv, gamma[ig],
                                   Cin, Sin, Cout, Sout, &tmp, dy + iv, dC, dS, du + ir,
                                   dh + ir, dq + ir, dk + ir, dv + iv, dg + ir, derase + ir,
                                   dwrite + iv, dgamma + ig, wk);
                    if (rs) { memset(dC, 0, nC * sizeof(double)); memset(dS, 0, nS * sizeof(double)); }
                }
            }
            if (dC0) memcpy(dC0 + (size_t)sidx * nC, dC, nC * sizeof(double));
            if (dS0) memcpy(dS0 + (size_t)sidx * nS, dS, nS * sizeof(double));
        }
        tok_free(&tmp);
        free(ckC); free(ckS); free(sgC); free(sgS); free(dC); free(dS); free(wk); free(otmp);
    }
    return failed ? -1 : 0;
}

int sdo_version(void) { return 1; }
