"""Chunk-form model of the CUDA pipeline, in PyTorch on the CPU (test helper).

It restates, stage by stage, what the CUDA kernels compute (same panels, same
names, same order), so that a failing GPU parity test can be narrowed to one
kernel by comparing workspace panels, and so that the chunk algebra itself is
checked against the token-by-token FP64 checker without a GPU.

Per (batch, head) stream and per chunk of L tokens (rows = tokens):
  g = log decay, G = inclusive cumsum of g inside the chunk, E = G - g,
  GL = last row of G, lam = exp(GL).
Forward stages: prep -> scan(C) -> mid -> scan(S) -> out.
Backward stages: ext_prep -> scan(dS) -> ext_main -> scan(dC) -> pred_main.
All four scans share one recurrence:
  X = P + Q @ St ; checkpoint St ; St = lam * St + R^T X (+ R2^T X2).
The predictor state is carried transposed, Ct[c, a] = C[a, c].

Decay-weighted intra-chunk terms never form a reciprocal-retention factor
exp(-G) (it overflows under strong forgetting).  A chunk is cut into blocks
of BT = 16 tokens.  With Gprev / Gend the prefix at the start / end of a
block, every factor used is bounded by one:
  rowG_i = exp(G_i - Gprev_I), rowE_i = exp(E_i - Gprev_I)   (row side)
  col_j  = exp(Gend_J - G_j)                                  (column side)
  beta_J = exp(Gend_J - Gprev_J)                              (whole block)
Off-diagonal block pairs (I > J) are contractions of row- and column-centred
panels with the product of the betas strictly between them; the diagonal
blocks evaluate exp(x_i - G_j) <= 1 directly.  `pair`, `csum` and `asum`
below are the three forms the kernels use (same block order, same Horner
accumulation over blocks).
"""
from __future__ import annotations

import torch

RHO = 5.0 / 8.0
BT = 16  # tokens per decay block


def _round_operand(x, mode):
    if mode is None:
        return x
    if mode == "bf16":
        return x.to(torch.bfloat16).to(x.dtype)
    if mode == "tf32":
        # round-to-nearest on a 10-bit mantissa, emulated in fp32
        xf = x.to(torch.float32)
        bits = xf.view(torch.int32)
        bits = (bits + 0x1000) & ~0x1FFF
        return bits.view(torch.float32).to(x.dtype)
    raise ValueError(mode)


class Model:
    def __init__(self, chunk=64, dtype=torch.float64, mma=None):
        self.L = chunk
        self.dtype = dtype
        self.mma = mma  # None | "tf32" | "bf16": operand rounding of every contraction

    def mm(self, a, b):
        return _round_operand(a, self.mma) @ _round_operand(b, self.mma)

    # ---- layout helpers -------------------------------------------------
    def _chunks(self, x, T, NC):
        """[B,T,H,D] -> [B*H, NC, L, D] with neutral (zero) padding."""
        B, _, H, D = x.shape
        pad = NC * self.L - T
        if pad:
            x = torch.cat([x, x.new_zeros(B, pad, H, D)], dim=1)
        return x.permute(0, 2, 1, 3).reshape(B * H, NC, self.L, D)

    def _unchunks(self, x, B, T, H):
        S, NC, L, D = x.shape
        return x.reshape(B, H, NC * L, D).permute(0, 2, 1, 3)[:, :T]

    @staticmethod
    def _norm(x):
        ss = (x * x).sum(-1, keepdim=True)
        rstd = torch.rsqrt(ss + 1e-24)
        return x * rstd, rstd

    @staticmethod
    def _solve_unit_lower(M, rhs, transpose=False):
        """Solve (I + M) X = rhs (or its transpose), M strictly lower."""
        L = M.shape[-1]
        eye = torch.eye(L, dtype=M.dtype)
        A = eye + M
        if transpose:
            return torch.linalg.solve_triangular(A.transpose(-1, -2), rhs, upper=True, unitriangular=True)
        return torch.linalg.solve_triangular(A, rhs, upper=False, unitriangular=True)

    def _scan(self, P, Q, R, lam, St0, R2=None, X2=None, reverse=False):
        """X = P + Q St ; ckpt St ; St = lam St + R^T X (+ R2^T X2)."""
        S_, NC = P.shape[0], P.shape[1]
        St = St0.clone()
        Xs = [None] * NC
        cks = [None] * NC
        order = range(NC - 1, -1, -1) if reverse else range(NC)
        for c in order:
            X = P[:, c] + self.mm(Q[:, c], St)
            Xs[c] = X
            cks[c] = St
            St = lam[:, c].unsqueeze(-1) * St + self.mm(R[:, c].transpose(-1, -2), X)
            if R2 is not None:
                St = St + self.mm(R2[:, c].transpose(-1, -2), X2[:, c])
        return torch.stack(Xs, 1), torch.stack(cks, 1), St

    # ---- shared chunk-local quantities ---------------------------------
    def _locals(self, inp):
        """Everything that depends only on the raw inputs of a chunk."""
        B, T, H, r = inp["u"].shape
        L = self.L
        NC = (T + L - 1) // L
        dt = self.dtype
        c = lambda x: self._chunks(x.to(dt), T, NC)
        loc = {"B": B, "T": T, "H": H, "NC": NC}
        loc["uh"], loc["u_rstd"] = self._norm(c(inp["u"]))
        loc["kh"], loc["k_rstd"] = self._norm(c(inp["k"]))
        loc["qh"], loc["q_rstd"] = self._norm(c(inp["q"]))
        loc["h"] = c(inp["h"])
        loc["v"] = c(inp["v"])
        loc["se"] = torch.sigmoid(c(inp["erase_raw"]))
        sw = torch.sigmoid(c(inp["write_raw"]))
        loc["sw"] = sw
        # neutral tail tokens have v = 0, so z = 0 although sigmoid(0) = 0.5
        loc["z"] = sw * loc["v"]
        g = c(inp["g"])
        gam = inp["gamma"].to(dt)
        gam = self._chunks(gam.unsqueeze(-1), T, NC)  # [S,NC,L,1]
        loc["gamma"] = gam
        G = torch.cumsum(g, dim=2)
        loc["G"], loc["E"] = G, G - g
        loc["GL"] = G[:, :, -1:, :]
        loc["lam"] = torch.exp(loc["GL"]).squeeze(2)  # [S,NC,r]
        loc["epos"] = torch.exp(G)
        loc["eE"] = torch.exp(loc["E"])
        loc["etail"] = torch.exp(loc["GL"] - G)
        loc["Ut"] = loc["uh"] * loc["eE"]          # U-tilde
        loc["Ubar"] = loc["uh"] * loc["etail"]
        tri = torch.ones(L, L, dtype=dt)
        loc["stril"] = torch.tril(tri, -1)
        loc["tril"] = torch.tril(tri)
        # block-centred decay factors
        bt = min(BT, L)
        nb = L // bt
        loc["bt"], loc["nb"] = bt, nb
        Gb = G.reshape(G.shape[0], NC, nb, bt, -1)
        gend = Gb[:, :, :, -1:, :]                                    # [S,NC,nb,1,r]
        gprev = torch.cat([torch.zeros_like(gend[:, :, :1]), gend[:, :, :-1]], dim=2)
        flat = lambda x: x.expand(-1, -1, -1, bt, -1).reshape(G.shape)
        loc["rowG"] = torch.exp(G - flat(gprev))
        loc["rowE"] = torch.exp(loc["E"] - flat(gprev))
        loc["col"] = torch.exp(flat(gend) - G)
        loc["beta"] = torch.exp(gend - gprev).squeeze(3)              # [S,NC,nb,r]
        loc["N"] = self.pair(loc, loc["uh"], loc["uh"], xe=True, strict=True)
        loc["Lm"] = gam * loc["N"]
        return loc

    # ---- block-centred decay contractions ---------------------------------
    def _blk(self, loc, x, I):
        bt = loc["bt"]
        return x[:, :, I * bt:(I + 1) * bt]

    def _rho(self, loc, I, xe):
        """exp(x_i - G_j) <= 1 for i, j inside block I (entries above the diagonal are unused)."""
        G = self._blk(loc, loc["G"], I)
        x = self._blk(loc, loc["E"] if xe else loc["G"], I)
        return torch.exp(torch.clamp(x.unsqueeze(3) - G.unsqueeze(2), max=0.0))  # [S,NC,i,j,c]

    def pair(self, loc, a, b, xe, strict):
        """[L,L]: sum_c a[i,c] b[j,c] exp(x[i,c] - G[j,c]) for j <= i (j < i if strict)."""
        nb, bt = loc["nb"], loc["bt"]
        R = a * (loc["rowE"] if xe else loc["rowG"])
        Cc = b * loc["col"]
        out = torch.zeros(a.shape[0], a.shape[1], self.L, self.L, dtype=a.dtype)
        mask = torch.tril(torch.ones(bt, bt, dtype=a.dtype), -1 if strict else 0)
        for I in range(nb):
            for J in range(I):
                M = torch.ones_like(loc["beta"][:, :, 0])
                for K in range(J + 1, I):
                    M = M * loc["beta"][:, :, K]
                blk = self.mm(self._blk(loc, R, I) * M.unsqueeze(2), self._blk(loc, Cc, J).transpose(-1, -2))
                out[:, :, I * bt:(I + 1) * bt, J * bt:(J + 1) * bt] = blk
            rho = self._rho(loc, I, xe)
            diag = torch.einsum("snic,snjc,snijc->snij", self._blk(loc, a, I), self._blk(loc, b, I), rho)
            out[:, :, I * bt:(I + 1) * bt, I * bt:(I + 1) * bt] = diag * mask
        return out

    def csum(self, loc, P, b, xe, strict, state=None):
        """[L,r]: sum_{j<=i} P[i,j] b[j,c] exp(x[i,c] - G[j,c]) (+ exp(x[i,c]) state[i,c]).
        Blocks below the diagonal accumulate Horner-style from the chunk start."""
        nb, bt = loc["nb"], loc["bt"]
        Cc = b * loc["col"]
        rowf = loc["rowE"] if xe else loc["rowG"]
        mask = torch.tril(torch.ones(bt, bt, dtype=P.dtype), -1 if strict else 0)
        outs = []
        for I in range(nb):
            PI = self._blk(loc, P, I)
            acc = self._blk(loc, state, I) if state is not None else None
            for J in range(I):
                if acc is not None:
                    acc = acc * loc["beta"][:, :, J].unsqueeze(2)
                term = self.mm(PI[..., J * bt:(J + 1) * bt], self._blk(loc, Cc, J))
                acc = term if acc is None else acc + term
            rho = self._rho(loc, I, xe)
            diag = torch.einsum("snij,snjc,snijc->snic", PI[..., I * bt:(I + 1) * bt] * mask,
                                self._blk(loc, b, I), rho)
            res = diag if acc is None else self._blk(loc, rowf, I) * acc + diag
            outs.append(res)
        return torch.cat(outs, dim=2)

    def asum(self, loc, P, a, xe, strict):
        """[L,r]: out[j,c] = sum_{i>=j} P[i,j] a[i,c] exp(x[i,c] - G[j,c]); Horner from the chunk end."""
        nb, bt = loc["nb"], loc["bt"]
        R = a * (loc["rowE"] if xe else loc["rowG"])
        mask = torch.tril(torch.ones(bt, bt, dtype=P.dtype), -1 if strict else 0)
        outs = []
        for J in range(nb):
            acc = None
            for I in range(nb - 1, J, -1):
                if acc is not None:
                    acc = acc * loc["beta"][:, :, I].unsqueeze(2)
                PIJ = self._blk(loc, P, I)[..., J * bt:(J + 1) * bt]
                term = self.mm(PIJ.transpose(-1, -2), self._blk(loc, R, I))
                acc = term if acc is None else acc + term
            rho = self._rho(loc, J, xe)
            PJJ = self._blk(loc, P, J)[..., J * bt:(J + 1) * bt] * mask
            diag = torch.einsum("snij,snic,snijc->snjc", PJJ, self._blk(loc, a, J), rho)
            res = diag if acc is None else self._blk(loc, loc["col"], J) * acc + diag
            outs.append(res)
        return torch.cat(outs, dim=2)

    def _sources(self, loc, Delta):
        """Per-token frame covector, dual address e and query chi."""
        uh, kh, qh = loc["uh"], loc["kh"], loc["qh"]
        n2 = (Delta * Delta).sum(-1, keepdim=True)
        s = RHO / torch.sqrt(RHO * RHO + n2)
        phi = s * Delta
        den = 1.0 + (phi * uh).sum(-1, keepdim=True)
        b = loc["se"] * kh
        sb = (uh * b).sum(-1, keepdim=True) / den
        sq = (uh * qh).sum(-1, keepdim=True) / den
        e = b - phi * sb
        chi = qh - phi * sq
        return dict(n2=n2, s=s, phi=phi, den=den, b=b, sb=sb, sq=sq, e=e, chi=chi)

    def _exterior_locals(self, loc, d, src):
        out = {}
        out["Xg"] = src["chi"] * loc["epos"]
        out["ag"] = -src["e"] * loc["epos"]
        out["Dt"] = d * loc["etail"]
        out["Aqd"] = self.pair(loc, src["chi"], d, xe=False, strict=False)
        out["Aed"] = self.pair(loc, -src["e"], d, xe=False, strict=True)
        return out

    # ---- forward --------------------------------------------------------
    def forward(self, inp, C0=None, S0=None):
        """inp: dict u,h,q,k,v [B,T,H,*], g [B,T,H,r], erase_raw, write_raw,
        gamma [B,T,H].  Returns y, C_T, S_T and a dict of saved panels."""
        dt = self.dtype
        loc = self._locals(inp)
        B, T, H, NC = loc["B"], loc["T"], loc["H"], loc["NC"]
        r, V = inp["u"].shape[-1], inp["v"].shape[-1]
        S_ = B * H
        gam = loc["gamma"]
        # prep
        rhs = torch.cat([gam * loc["h"], gam * loc["Ut"]], dim=-1)
        sol = self._solve_unit_lower(loc["Lm"], rhs)
        Upd, W = sol[..., :r], sol[..., r:]
        # scan C (transposed state)
        Ct0 = torch.zeros(S_, r, r, dtype=dt) if C0 is None else C0.to(dt).reshape(S_, r, r).transpose(-1, -2)
        Delta, Ct_ck, Ct_fin = self._scan(Upd, -W, loc["Ubar"], loc["lam"], Ct0)
        # mid
        Aqk = self.mm(loc["kh"], Delta.transpose(-1, -2)) * loc["tril"]
        d = loc["kh"] + self.csum(loc, Aqk, loc["uh"], xe=False, strict=False,
                                  state=self.mm(loc["kh"], Ct_ck.transpose(-1, -2)))
        src = self._sources(loc, Delta)
        ext = self._exterior_locals(loc, d, src)
        rhs = torch.cat([ext["ag"], loc["z"]], dim=-1)
        sol = self._solve_unit_lower(-ext["Aed"], rhs)
        Wd, Ud = sol[..., :r], sol[..., r:]
        # scan S
        St0 = torch.zeros(S_, r, V, dtype=dt) if S0 is None else S0.to(dt).reshape(S_, r, V)
        Zt, S_ck, S_fin = self._scan(Ud, Wd, ext["Dt"], loc["lam"], St0)
        # out
        y = self.mm(ext["Xg"], S_ck) + self.mm(ext["Aqd"], Zt)
        saved = dict(loc=loc, Upd=Upd, W=W, Delta=Delta, Ct_ck=Ct_ck, d=d, Wd=Wd, Ud=Ud,
                     Zt=Zt, S_ck=S_ck, Xg=ext["Xg"], Aqd=ext["Aqd"], Dt=ext["Dt"])
        # the same quantities under the names the CUDA library gives its panels
        saved["panels"] = dict(Lam=loc["lam"], G=loc["G"], Delta=Delta, Dprim=d, Zt=Zt, CtCk=Ct_ck, SCk=S_ck,
                               Upd=Upd, Qc=-W, Ubar=loc["Ubar"], Wd=Wd, Ud=Ud, Dt=ext["Dt"],
                               Xg=ext["Xg"], Aqd=ext["Aqd"], N=loc["N"], Aed=ext["Aed"])
        yo = self._unchunks(y, B, T, H)
        C_T = Ct_fin.transpose(-1, -2).reshape(B, H, r, r)
        S_T = S_fin.reshape(B, H, r, V)
        return yo, C_T, S_T, saved

    # ---- backward -------------------------------------------------------
    def backward(self, inp, saved, dy, dC_T=None, dS_T=None):
        dt = self.dtype
        loc = saved["loc"]
        B, T, H, NC = loc["B"], loc["T"], loc["H"], loc["NC"]
        r, V = inp["u"].shape[-1], inp["v"].shape[-1]
        S_, L = B * H, self.L
        uh, kh, qh = loc["uh"], loc["kh"], loc["qh"]
        gam = loc["gamma"]
        Delta, d, Zt = saved["Delta"], saved["d"], saved["Zt"]
        Ct_ck, S_ck = saved["Ct_ck"], saved["S_ck"]
        dyc = self._chunks(dy.to(dt), T, NC)
        # ext_prep
        src = self._sources(loc, Delta)
        ext = self._exterior_locals(loc, d, src)
        rhs = torch.cat([self.mm(ext["Aqd"].transpose(-1, -2), dyc), ext["Dt"]], dim=-1)
        sol = self._solve_unit_lower(-ext["Aed"], rhs, transpose=True)
        Pp, Qp = sol[..., :V], sol[..., V:]
        # scan dS (reverse)
        dS_end = torch.zeros(S_, r, V, dtype=dt) if dS_T is None else dS_T.to(dt).reshape(S_, r, V)
        dR, dSe, dS0 = self._scan(Pp, Qp, ext["ag"], loc["lam"], dS_end, R2=ext["Xg"], X2=dyc, reverse=True)
        # ext_main
        dAqd = self.mm(dyc, Zt.transpose(-1, -2)) * loc["tril"]
        dAed = self.mm(dR, Zt.transpose(-1, -2)) * loc["stril"]
        dXg = self.mm(dyc, S_ck.transpose(-1, -2))
        dag = self.mm(dR, S_ck.transpose(-1, -2))
        dDt = self.mm(Zt, dSe.transpose(-1, -2))
        dchi = self.csum(loc, dAqd, d, xe=False, strict=False, state=dXg)
        de = -self.csum(loc, dAed, d, xe=False, strict=True, state=dag)
        ddp = self.asum(loc, dAqd, src["chi"], xe=False, strict=False) + \
            self.asum(loc, dAed, -src["e"], xe=False, strict=True)
        dd = ddp + dDt * loc["etail"]
        dG = src["chi"] * dchi + src["e"] * de - d * ddp
        dGL = loc["lam"] * (S_ck * dSe).sum(-1) + (dDt * ext["Dt"]).sum(2)  # [S,NC,r]
        # sources backward
        phi, den, sb, sq, b = src["phi"], src["den"], src["sb"], src["sq"], src["b"]
        db = de.clone()
        dqh = dchi.clone()
        dphi = -de * sb - dchi * sq
        dsb = -(de * phi).sum(-1, keepdim=True)
        dsq = -(dchi * phi).sum(-1, keepdim=True)
        db = db + (dsb / den) * uh
        dqh = dqh + (dsq / den) * uh
        dden = -(dsb * sb + dsq * sq) / den
        duh = (dsb / den) * b + (dsq / den) * qh + dden * phi
        dphi = dphi + dden * uh
        s = src["s"]
        dDelta = s * dphi - (dphi * Delta).sum(-1, keepdim=True) * s / (RHO * RHO + src["n2"]) * Delta
        se, sw = loc["se"], loc["sw"]
        dkh = se * db
        duPart, dkPart, dDeltaSrc = duh.clone(), dkh + dd, dDelta.clone()
        dGPart = dG + dd * (d - kh)
        Xext = dDt * ext["Dt"]
        dG = dG - Xext
        d_erase_raw = db * kh * se * (1 - se)
        dv = sw * dR
        d_write_raw = dR * loc["v"] * sw * (1 - sw)
        # predictor part 1
        dact = dd
        dkh = dkh + dd
        DG = dact * loc["epos"]
        dkh = dkh + self.mm(DG, Ct_ck)
        dAqk = self.pair(loc, dact, uh, xe=False, strict=False)
        Aqk = self.mm(kh, Delta.transpose(-1, -2)) * loc["tril"]
        t_u = self.asum(loc, Aqk, dact, xe=False, strict=False)
        duh = duh + t_u
        dG = dG + dact * (d - kh) - uh * t_u
        dkh = dkh + self.mm(dAqk, Delta)
        dDelta = dDelta + self.mm(dAqk.transpose(-1, -2), kh)
        rhs = torch.cat([dDelta, loc["Ubar"]], dim=-1)
        sol = self._solve_unit_lower(loc["Lm"], rhs, transpose=True)
        Ppp, Qpp = sol[..., :r], sol[..., r:]
        # scan dC (reverse, transposed state)
        dCt_end = torch.zeros(S_, r, r, dtype=dt) if dC_T is None else dC_T.to(dt).reshape(S_, r, r).transpose(-1, -2)
        dRr, dCe, dCt0 = self._scan(Ppp, Qpp, -gam * loc["Ut"], loc["lam"], dCt_end, R2=DG, X2=kh, reverse=True)
        # pred_main
        dUbar = self.mm(Delta, dCe.transpose(-1, -2))
        duh = duh + dUbar * loc["etail"]
        dG = dG - dUbar * loc["Ubar"]
        dGL = dGL + (dUbar * loc["Ubar"]).sum(2) + loc["lam"] * (Ct_ck * dCe).sum(-1)
        dLm = -self.mm(dRr, Delta.transpose(-1, -2)) * loc["stril"]
        dh = gam * dRr
        Rh = loc["h"] - self.mm(loc["Ut"], Ct_ck)
        res = Rh - self.mm(loc["N"], Delta)
        dgamma = (dRr * res).sum(-1)
        dUt = -self.mm(gam * dRr, Ct_ck.transpose(-1, -2))
        duh = duh + dUt * loc["eE"]
        dE = dUt * loc["Ut"]
        dN = gam * dLm
        t_i = self.csum(loc, dN, uh, xe=True, strict=True)
        t_j = self.asum(loc, dN, uh, xe=True, strict=True)
        duh = duh + t_i + t_j
        dE = dE + uh * t_i
        dG = dG - uh * t_j
        # gate closure
        dG = dG + dE
        dG[:, :, -1, :] = dG[:, :, -1, :] + dGL
        dg = -dE + torch.flip(torch.cumsum(torch.flip(dG, [2]), 2), [2])

        def norm_vjp(dxh, xh, rstd):
            return (dxh - (dxh * xh).sum(-1, keepdim=True) * xh) * rstd

        un = lambda x: self._unchunks(x, B, T, H)
        grads = dict(
            u=un(norm_vjp(duh, uh, loc["u_rstd"])),
            h=un(dh),
            q=un(norm_vjp(dqh, qh, loc["q_rstd"])),
            k=un(norm_vjp(dkh, kh, loc["k_rstd"])),
            v=un(dv),
            g=un(dg),
            erase_raw=un(d_erase_raw),
            write_raw=un(d_write_raw),
            gamma=un(dgamma.unsqueeze(-1)).squeeze(-1),
            C0=dCt0.transpose(-1, -2).reshape(B, H, r, r),
            S0=dS0.reshape(B, H, r, V),
        )
        panels = dict(Pp=Pp, Qp=Qp, Ag=ext["ag"], Xg=ext["Xg"], Dyf=dyc, dR=dR,
                      dSeCk=dSe, dDt=dDt, Chi=src["chi"], Ee=-src["e"],
                      SdS=(S_ck * dSe).sum(-1), duPart=duPart, dkPart=dkPart, dGPart=dGPart,
                      dDelta=dDeltaSrc, DG=DG, Dd=dact, Xext=Xext, Tu=t_u, Khat=kh, Ppp=Ppp, Qpp=Qpp,
                      Rneg=-gam * loc["Ut"], dRr=dRr, dCeCk=dCe, dUbar=dUbar, dUt=dUt,
                      CdC=(Ct_ck * dCe).sum(-1))
        return grads, panels
