"""FP64 numpy restatement of the SolveDelta mixer around the recurrence
(TEST INFRASTRUCTURE -- never imported by the product package).

Follows the CPU branches of causallsso/model.py: fused input projection and
its ten slices (model.py:39-60,321-367), the token-loop conv4 + SiLU with a
[B,D,3] state (model.py:146-164), the decay gate
-exp(log_rate) * softplus(raw + bias) (model.py:383-390), the geometry rate
sigmoid(raw + bias) (model.py:391-394), the operator through the C checker
(oracle/solvedelta_oracle.c), the sigmoid-gated RMSNorm
(causallsso/ops/norm_gate.py:19-43) and the output projection.  ``backward``
is the hand-written adjoint of exactly these steps; both are pinned against
the upstream module + torch.autograd on committed golden vectors
(tests/golden/mixer_small.npz).
"""
from __future__ import annotations

import numpy as np

from . import solvedelta_oracle as orc


def _sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def _softplus(z):
    return np.where(z > 30, z, np.log1p(np.exp(np.minimum(z, 30))))


def conv4_silu_forward(x, weight, state=None):
    """x [B,T,D], weight [D,4] (tap 3 = current token), state [B,D,3] (oldest first).
    Returns (y, final_state, (ext, pre)).  causallsso/model.py:146-164 without masks."""
    x = np.asarray(x, dtype=np.float64)
    B, T, D = x.shape
    state = np.zeros((B, D, 3)) if state is None else np.asarray(state, dtype=np.float64)
    ext = np.concatenate([state.transpose(0, 2, 1), x], axis=1)  # ext[:, t+3] = x[:, t]
    pre = sum(ext[:, j:j + T] * weight[:, j] for j in range(4))
    return pre * _sigmoid(pre), ext[:, T:T + 3].transpose(0, 2, 1).copy(), (ext, pre)


def conv4_silu_backward(dy, weight, saved, dfinal=None):
    """Returns (dx, dweight, dstate)."""
    ext, pre = saved
    T = pre.shape[1]
    s = _sigmoid(pre)
    dpre = np.asarray(dy, dtype=np.float64) * s * (1 + pre * (1 - s))
    dw = np.stack([(dpre * ext[:, j:j + T]).sum((0, 1)) for j in range(4)], axis=-1)
    dext = np.zeros_like(ext)
    for j in range(4):
        dext[:, j:j + T] += dpre * weight[:, j]
    if dfinal is not None:
        dext[:, T:T + 3] += np.asarray(dfinal, dtype=np.float64).transpose(0, 2, 1)
    return dext[:, 3:], dw, dext[:, :3].transpose(0, 2, 1).copy()


def conv4_silu_masked_forward(x, weight, state=None, valid_mask=None, reset_mask=None):
    """The masked token loop of causallsso/model.py:146-164: a reset (on a valid token) zeroes the
    state first, an invalid token yields zero and leaves the state untouched.  Returns
    (y, final_state, saved)."""
    x = np.asarray(x, dtype=np.float64)
    B, T, D = x.shape
    state = np.zeros((B, D, 3)) if state is None else np.asarray(state, dtype=np.float64).copy()
    valid = np.ones((B, T), bool) if valid_mask is None else np.asarray(valid_mask, bool)
    reset = (np.zeros((B, T), bool) if reset_mask is None else np.asarray(reset_mask, bool)) & valid
    y = np.zeros_like(x)
    windows, pres = [], []
    for t in range(T):
        state = np.where(reset[:, t, None, None], 0.0, state)
        window = np.concatenate([state, x[:, t, :, None]], axis=-1)      # [B,D,4]
        pre = (window * weight[None]).sum(-1)
        y[:, t] = np.where(valid[:, t, None], pre * _sigmoid(pre), 0.0)
        state = np.where(valid[:, t, None, None], window[..., 1:], state)
        windows.append(window)
        pres.append(pre)
    return y, state, (windows, pres, valid, reset)


def conv4_silu_masked_backward(dy, weight, saved, dfinal=None):
    """Adjoint of the masked loop.  Returns (dx, dweight, dstate)."""
    windows, pres, valid, reset = saved
    dy = np.asarray(dy, dtype=np.float64)
    B, T, D = dy.shape
    dstate = np.zeros((B, D, 3)) if dfinal is None else np.asarray(dfinal, dtype=np.float64).copy()
    dx = np.zeros_like(dy)
    dw = np.zeros_like(weight)
    for t in range(T - 1, -1, -1):
        v = valid[:, t, None, None]
        # state_after = valid ? window[..., 1:] : state_before
        dwindow = np.zeros((B, D, 4))
        dwindow[..., 1:] = np.where(v, dstate, 0.0)
        dstate_before = np.where(v, 0.0, dstate)
        s = _sigmoid(pres[t])
        dpre = np.where(valid[:, t, None], dy[:, t], 0.0) * s * (1 + pres[t] * (1 - s))
        dwindow += dpre[..., None] * weight[None]
        dw += (dpre[..., None] * windows[t]).sum(0)
        dx[:, t] = dwindow[..., 3]
        dstate_before = dstate_before + dwindow[..., :3]
        dstate = np.where(reset[:, t, None, None], 0.0, dstate_before)
    return dx, dw, dstate


def kda_gate_forward(raw, log_rate, bias):
    """-exp(log_rate[h]) * softplus(raw + bias[h,c]); raw [...,H,r].  model.py:383-390."""
    H, r = raw.shape[-2:]
    z = np.asarray(raw, dtype=np.float64) + np.asarray(bias, dtype=np.float64).reshape(H, r)
    rate = -np.exp(np.asarray(log_rate, dtype=np.float64)).reshape(H, 1)
    return rate * _softplus(z), (z, rate)


def kda_gate_backward(dout, saved):
    """Returns (draw, dlog_rate [H], dbias [H,r])."""
    z, rate = saved
    H, r = z.shape[-2:]
    dout = np.asarray(dout, dtype=np.float64)
    lead = tuple(range(z.ndim - 2))
    dlog_rate = (dout * rate * _softplus(z)).sum(lead + (z.ndim - 1,))
    draw = dout * rate * _sigmoid(z)
    return draw, dlog_rate, draw.sum(lead)


def norm_gate_forward(x, gate, weight, eps):
    """x * rsqrt(mean(x^2) + eps) * weight * sigmoid(gate).  ops/norm_gate.py:19-43."""
    x = np.asarray(x, dtype=np.float64)
    rstd = 1.0 / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    sg = _sigmoid(np.asarray(gate, dtype=np.float64))
    return x * rstd * weight * sg, (x, rstd, sg)


def norm_gate_backward(dy, weight, saved):
    """Returns (dx, dgate, dweight)."""
    x, rstd, sg = saved
    dy = np.asarray(dy, dtype=np.float64)
    xn = x * rstd
    dweight = (dy * xn * sg).reshape(-1, x.shape[-1]).sum(0)
    dxn = dy * weight * sg
    dgate = dy * xn * weight * sg * (1 - sg)
    dx = (dxn - xn * (dxn * xn).mean(-1, keepdims=True)) * rstd
    return dx, dgate, dweight


class MixerOracle:
    """params: dict with the upstream parameter names (numpy, any float dtype)."""

    def __init__(self, params, *, hidden_size, num_heads, head_k_dim, head_v_dim, use_short_conv=True,
                 norm_eps=1e-6, activation_rounding=None):
        """``activation_rounding``: optional callable applied to every activation a
        reduced-precision implementation stores between two kernels (projection row,
        conv output, gate pre-activations, operator output, normalised output); the
        adjoint treats it as the identity.  None = exact FP64 (the upstream CPU path)."""
        self.rnd = activation_rounding if activation_rounding is not None else (lambda z: z)
        self.p = {k: np.asarray(v, dtype=np.float64) for k, v in params.items()}
        self.hidden, self.H, self.r, self.V = hidden_size, num_heads, head_k_dim, head_v_dim
        self.conv = use_short_conv
        self.eps = norm_eps
        H, r, V = self.H, self.r, self.V
        self.sizes = (H * r, H * r, H * V, H * r, H * r, H * r, H * V, H, V, V)
        self.offsets = np.concatenate([[0], np.cumsum(self.sizes)])

    def _piece(self, row, i):
        return row[..., self.offsets[i]:self.offsets[i + 1]]

    def forward(self, x, conv_state=None, operator_state=None, valid_mask=None, reset_mask=None):
        p, H, r, V = self.p, self.H, self.r, self.V
        x = np.asarray(x, dtype=np.float64)
        B, T, _ = x.shape
        row = x @ p["in_proj.weight"].T
        if "in_proj.bias" in p:
            row = row + p["in_proj.bias"]
        row = self.rnd(row)
        c = {"x": x, "row": row}
        Dc = sum(self.sizes[:3])
        if self.conv:
            if valid_mask is None and reset_mask is None:
                qkv, final_conv, c["conv_saved"] = conv4_silu_forward(row[..., :Dc], p["conv_weight"], conv_state)
            else:
                qkv, final_conv, c["conv_saved"] = conv4_silu_masked_forward(
                    row[..., :Dc], p["conv_weight"], conv_state, valid_mask, reset_mask)
        else:
            pre = row[..., :Dc]
            qkv = pre * _sigmoid(pre)
            c.update(pre=pre)
            final_conv = None
        qkv = self.rnd(qkv)
        q = qkv[..., :H * r].reshape(B, T, H, r)
        k = qkv[..., H * r:2 * H * r].reshape(B, T, H, r)
        v = qkv[..., 2 * H * r:].reshape(B, T, H, V)
        u = self._piece(row, 3).reshape(B, T, H, r)
        h = self._piece(row, 4).reshape(B, T, H, r)
        er = self._piece(row, 5).reshape(B, T, H, r)
        wr = self._piece(row, 6).reshape(B, T, H, V)
        graw = self._piece(row, 7)
        dhid, ghid = self._piece(row, 8), self._piece(row, 9)
        araw = self.rnd((dhid @ p["decay_proj.weight"].T).reshape(B, T, H, r))
        gate = self.rnd((ghid @ p["output_gate_proj.weight"].T + p["output_gate_proj.bias"]).reshape(B, T, H, V))
        log_decay, c["gate_saved"] = kda_gate_forward(araw, p["associative_log_rate"], p["associative_decay_bias"])
        gamma = _sigmoid(graw + p["geometry_write_bias"].reshape(1, 1, H))
        erase, write = _sigmoid(er), _sigmoid(wr)
        o, fin = orc.forward(u, h, q, k, v, log_decay, erase, write, gamma, initial_state=operator_state,
                             valid_mask=valid_mask, reset_mask=reset_mask)
        o = self.rnd(o)
        y, c["norm_saved"] = norm_gate_forward(o, gate, p["output_norm.weight"], self.eps)
        y = self.rnd(y)
        out = y.reshape(B, T, H * V) @ p["output_proj.weight"].T
        if "output_proj.bias" in p:
            out = out + p["output_proj.bias"]
        c.update(q=q, k=k, v=v, u=u, h=h, log_decay=log_decay, gamma=gamma, erase=erase, write=write, y=y,
                 dhid=dhid, ghid=ghid, operator_state=operator_state, B=B, T=T,
                 masks=(valid_mask, reset_mask))
        self.cache = c
        return out, fin, final_conv

    def backward(self, dout, dC_T=None, dS_T=None, dconv_T=None, operator_grads=None):
        """Returns (dx, dict of parameter gradients, d conv_state or None, operator-state grads).
        dC_T/dS_T/dconv_T are cotangents of the final operator and conv states.

        ``operator_grads``: optional dict of gradients with respect to the operator's
        operands (u, h, q, keys, values, log_decay, erase_raw, write_raw, geometry_write,
        C0, S0) to chain through the glue instead of the checker's own operator VJP --
        used to check the glue's adjoint separately from the operator's.  The
        operator gradients actually used are left in ``self.operator_grads``
        (erase / write with respect to the raw logits) and ``self.do``."""
        p, c, H, r, V = self.p, self.cache, self.H, self.r, self.V
        B, T = c["B"], c["T"]
        g = {}
        dout = np.asarray(dout, dtype=np.float64)
        yflat = c["y"].reshape(B, T, H * V)
        g["output_proj.weight"] = np.einsum("bto,bti->oi", dout, yflat)
        if "output_proj.bias" in p:
            g["output_proj.bias"] = dout.sum((0, 1))
        dy = (dout @ p["output_proj.weight"]).reshape(B, T, H, V)
        do, dgate, g["output_norm.weight"] = norm_gate_backward(dy, p["output_norm.weight"], c["norm_saved"])
        self.do = do
        if operator_grads is None:
            og = orc.backward(c["u"], c["h"], c["q"], c["k"], c["v"], c["log_decay"], c["erase"], c["write"],
                              c["gamma"], do, dC_T=dC_T, dS_T=dS_T, initial_state=c["operator_state"],
                              valid_mask=c["masks"][0], reset_mask=c["masks"][1])
            og["erase_raw"] = og["erase"] * c["erase"] * (1 - c["erase"])
            og["write_raw"] = og["write"] * c["write"] * (1 - c["write"])
        else:
            og = {k: np.asarray(v, dtype=np.float64) for k, v in operator_grads.items()}
            og.setdefault("C0", None)
            og.setdefault("S0", None)
        self.operator_grads = og
        drow = np.zeros_like(c["row"])
        put = lambda i, val: drow.__setitem__((Ellipsis, slice(self.offsets[i], self.offsets[i + 1])),
                                              val.reshape(B, T, -1))
        put(3, og["u"])
        put(4, og["h"])
        put(5, og["erase_raw"])
        put(6, og["write_raw"])
        dgraw = og["geometry_write"] * c["gamma"] * (1 - c["gamma"])
        put(7, dgraw)
        g["geometry_write_bias"] = dgraw.sum((0, 1))
        dz, g["associative_log_rate"], dbias = kda_gate_backward(og["log_decay"], c["gate_saved"])
        g["associative_decay_bias"] = dbias.reshape(p["associative_decay_bias"].shape)
        dz2 = dz.reshape(B, T, H * r)
        g["decay_proj.weight"] = np.einsum("bto,bti->oi", dz2, c["dhid"])
        put(8, dz2 @ p["decay_proj.weight"])
        dgate2 = dgate.reshape(B, T, H * V)
        g["output_gate_proj.weight"] = np.einsum("bto,bti->oi", dgate2, c["ghid"])
        g["output_gate_proj.bias"] = dgate2.sum((0, 1))
        put(9, dgate2 @ p["output_gate_proj.weight"])
        dqkv = np.concatenate([og["q"].reshape(B, T, -1), og["keys"].reshape(B, T, -1),
                               og["values"].reshape(B, T, -1)], axis=-1)
        Dc = dqkv.shape[-1]
        dconv_state = None
        if self.conv:
            unmasked = c["masks"][0] is None and c["masks"][1] is None
            conv_vjp = conv4_silu_backward if unmasked else conv4_silu_masked_backward
            drow[..., :Dc], g["conv_weight"], dconv_state = conv_vjp(dqkv, p["conv_weight"], c["conv_saved"], dconv_T)
        else:
            pre = c["pre"]
            s = _sigmoid(pre)
            drow[..., :Dc] = dqkv * s * (1 + pre * (1 - s))
        g["in_proj.weight"] = np.einsum("bto,bti->oi", drow, c["x"])
        if "in_proj.bias" in p:
            g["in_proj.bias"] = drow.sum((0, 1))
        dx = drow @ p["in_proj.weight"]
        return dx, g, dconv_state, (og["C0"], og["S0"])
