"""Helpers shared by the GPU parity tests: seeded inputs, direct C-ABI calls
that keep the workspace alive, and oracle-side conversions."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from solvedelta_b200 import _lib
from solvedelta_b200.ops import _fill_operands, _operand


def make_inputs(B, T, H, r, V, *, seed=0, gamma_mode="token", decay_scale=None, device="cuda",
                with_state=True, gamma_max=0.1):
    """Benchmark-like seeded inputs (BF16 vectors, FP32 gates) generated on the
    CPU so the checker and the GPU see identical bits."""
    gen = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=gen)
    bf = lambda x: x.to(torch.bfloat16)
    u, h = bf(rn(B, T, H, r)), bf(rn(B, T, H, r))
    q = bf(torch.nn.functional.normalize(rn(B, T, H, r), dim=-1))
    k = bf(torch.nn.functional.normalize(rn(B, T, H, 1, r), dim=-1))
    v = bf(rn(B, T, H, 1, V))
    er = bf(0.5 * rn(B, T, H, 1, r))
    wr = bf(0.5 * rn(B, T, H, 1, V))
    if decay_scale is None:
        ld = torch.nn.functional.logsigmoid(rn(B, T, H, r) + 4.0)
    else:
        ld = -decay_scale * torch.rand(B, T, H, r, generator=gen)
    if gamma_mode == "token":
        gam = gamma_max * torch.rand(B, T, H, generator=gen)
    elif gamma_mode == "head":
        gam = gamma_max * torch.rand(H, generator=gen)
    elif gamma_mode == "zero":
        gam = torch.zeros(B, T, H)
    else:
        raise ValueError(gamma_mode)
    C0 = 0.02 * rn(B, H, r, r) if with_state else None
    S0 = 0.02 * rn(B, H, r, V) if with_state else None
    cpu = dict(u=u, h=h, q=q, keys=k, values=v, log_decay=ld, erase_raw=er, write_raw=wr,
               geometry_write=gam, C0=C0, S0=S0)
    dev = {n: (None if t is None else t.to(device)) for n, t in cpu.items()}
    return cpu, dev


def oracle_args(cpu):
    """FP64 operands for the checker from the quantised CPU copies."""
    d = lambda x: x.double().numpy()
    return [d(cpu["u"]), d(cpu["h"]), d(cpu["q"]), d(cpu["keys"]), d(cpu["values"]),
            d(cpu["log_decay"]), d(torch.sigmoid(cpu["erase_raw"].double())),
            d(torch.sigmoid(cpu["write_raw"].double())), d(cpu["geometry_write"])]


def oracle_state(cpu):
    if cpu["C0"] is None:
        return None
    return (cpu["C0"].double().numpy(), cpu["S0"].double().numpy())


def raw_gate_grads(cpu, grads):
    """Chain the checker's gradients of the post-sigmoid gates to the raw logits."""
    se = torch.sigmoid(cpu["erase_raw"].double()).numpy()[:, :, :, 0]
    sw = torch.sigmoid(cpu["write_raw"].double()).numpy()[:, :, :, 0]
    return grads["erase"] * se * (1 - se), grads["write"] * sw * (1 - sw)


def model_inputs(cpu):
    B, T, H, r = cpu["u"].shape
    gam = cpu["geometry_write"]
    if gam.ndim != 3:
        gam = gam.reshape(1, 1, H).expand(B, T, H)
    f = lambda x: x.double()
    return dict(u=f(cpu["u"]), h=f(cpu["h"]), q=f(cpu["q"]), k=f(cpu["keys"][:, :, :, 0]),
                v=f(cpu["values"][:, :, :, 0]), g=f(cpu["log_decay"]),
                erase_raw=f(cpu["erase_raw"][:, :, :, 0]), write_raw=f(cpu["write_raw"][:, :, :, 0]),
                gamma=f(gam))


class RawRun:
    """Calls sd_forward / sd_backward directly and keeps every buffer."""

    def __init__(self, dev, dy=None, dC_T=None, dS_T=None):
        lib = _lib.load()
        u = dev["u"]
        B, T, H, r = u.shape
        V = dev["values"].shape[-1]
        device = u.device
        self.shape = _lib.Shape(B, T, H, r, V)
        gam = dev["geometry_write"]
        if gam.ndim != 3:
            gam = gam.reshape(1, 1, H).expand(B, T, H)
        sq = lambda x: x.squeeze(-2)
        tensors = (u, dev["h"], dev["q"], sq(dev["keys"]), sq(dev["values"]), dev["log_decay"],
                   sq(dev["erase_raw"]), sq(dev["write_raw"]), gam)
        self.keep = tensors
        stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        nb = lambda f: max(int(f(ctypes.byref(self.shape))), 16)
        self.saved = torch.zeros(nb(lib.sd_saved_bytes), dtype=torch.uint8, device=device)
        self.fwd_scratch = torch.zeros(nb(lib.sd_forward_scratch_bytes), dtype=torch.uint8, device=device)
        self.y = torch.empty(B, T, H, V, dtype=torch.bfloat16, device=device)
        self.C_T = torch.empty(B, H, r, r, dtype=torch.float32, device=device)
        self.S_T = torch.empty(B, H, r, V, dtype=torch.float32, device=device)
        fa = _lib.ForwardArgs()
        fa.shape = self.shape
        _fill_operands(fa, tensors)
        fa.C0 = None if dev["C0"] is None else dev["C0"].data_ptr()
        fa.S0 = None if dev["S0"] is None else dev["S0"].data_ptr()
        fa.y, fa.C_T, fa.S_T = self.y.data_ptr(), self.C_T.data_ptr(), self.S_T.data_ptr()
        fa.saved, fa.saved_bytes = self.saved.data_ptr(), self.saved.numel()
        fa.scratch, fa.scratch_bytes = self.fwd_scratch.data_ptr(), self.fwd_scratch.numel()
        _lib.check(lib.sd_forward(ctypes.byref(fa), stream))
        torch.cuda.synchronize()
        self.grads = None
        if dy is None:
            return
        self.bwd_scratch = torch.zeros(nb(lib.sd_backward_scratch_bytes), dtype=torch.uint8, device=device)
        bf = dict(dtype=torch.bfloat16, device=device)
        g = dict(u=torch.empty(B, T, H, r, **bf), h=torch.empty(B, T, H, r, **bf),
                 q=torch.empty(B, T, H, r, **bf), keys=torch.empty(B, T, H, r, **bf),
                 values=torch.empty(B, T, H, V, **bf), erase_raw=torch.empty(B, T, H, r, **bf),
                 write_raw=torch.empty(B, T, H, V, **bf),
                 log_decay=torch.empty(B, T, H, r, dtype=torch.float32, device=device),
                 geometry_write=torch.empty(B, T, H, dtype=torch.float32, device=device),
                 C0=torch.empty(B, H, r, r, dtype=torch.float32, device=device),
                 S0=torch.empty(B, H, r, V, dtype=torch.float32, device=device))
        ba = _lib.BackwardArgs()
        ba.shape = self.shape
        _fill_operands(ba, tensors)
        ba.dy = _operand(dy)
        ba.dC_T = None if dC_T is None else dC_T.data_ptr()
        ba.dS_T = None if dS_T is None else dS_T.data_ptr()
        ba.saved, ba.saved_bytes = self.saved.data_ptr(), self.saved.numel()
        ba.scratch, ba.scratch_bytes = self.bwd_scratch.data_ptr(), self.bwd_scratch.numel()
        ba.du, ba.dh, ba.dq = g["u"].data_ptr(), g["h"].data_ptr(), g["q"].data_ptr()
        ba.dkeys, ba.dvalues = g["keys"].data_ptr(), g["values"].data_ptr()
        ba.derase_raw, ba.dwrite_raw = g["erase_raw"].data_ptr(), g["write_raw"].data_ptr()
        ba.dlog_decay, ba.dgamma = g["log_decay"].data_ptr(), g["geometry_write"].data_ptr()
        ba.dC0, ba.dS0 = g["C0"].data_ptr(), g["S0"].data_ptr()
        _lib.check(lib.sd_backward(ctypes.byref(ba), stream))
        torch.cuda.synchronize()
        self.grads = g

    def panel(self, which, name):
        """Fetch an intermediate panel as a CPU float tensor [chunks, rows, cols] and its dtype tag."""
        lib = _lib.load()
        off, nbytes = ctypes.c_size_t(), ctypes.c_size_t()
        _lib.check(lib.sd_panel_info(ctypes.byref(self.shape), which, name.encode(),
                                     ctypes.byref(off), ctypes.byref(nbytes)))
        kind = lib.sd_panel_kind(ctypes.byref(self.shape), which, name.encode())
        buf = (self.saved, self.fwd_scratch, getattr(self, "bwd_scratch", None))[which]
        raw = buf[off.value: off.value + nbytes.value]
        flat = (raw.view(torch.bfloat16) if kind >= 4 else raw.view(torch.float32)).float().cpu()
        L = lib.sd_chunk_tokens()
        chunks = self.shape.B * self.shape.H * ((self.shape.T + L - 1) // L)
        dims = {0: (L, 128), 1: (L, L), 2: (128, 128), 3: (1, 128), 4: (L, 128), 5: (L, L), 6: (128, 128)}[kind]
        return flat.view(chunks, *dims), ("bf16" if kind >= 4 else "f32")
