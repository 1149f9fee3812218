"""Muon on the hidden matrices + AdamW on word tables, norms and vectors, one shared learning rate.

The comparison optimizer of the reference's race runs (`OPT=muon`, `_MuonCombo`, fastloop.py:63-82, which wraps
`torch.optim.Muon(adjust_lr_fn="match_rms_adamw")` and a fused AdamW).  Here the Muon half is written out: Nesterov
momentum, five Newton-Schulz steps that push the update's singular values towards 1, decoupled weight decay and the
step scaled by 0.2·sqrt(max(rows, cols)) so that its RMS matches an AdamW step.  The Newton-Schulz products
(X·Xᵀ, A·A, B·X) are GEMMs: on the GPU they run on this package's tcgen05 kernel in bf16.
"""
from __future__ import annotations

import math

import torch

NS_COEFF = (3.4445, -4.7750, 2.0315)


def _mm_nt(a, b):
    """a · bᵀ."""
    if a.is_cuda and a.dtype == torch.bfloat16:
        from ..ops import basic
        if basic.gemm_ok(a.shape[0], b.shape[0], a.shape[1]):
            return basic.gemm(a.contiguous(), b.contiguous())
    return a @ b.t()


def _mm_nn(a, b):
    """a · b with b stored (inner, columns): fed to the GEMM as an MN-major operand, no transposing copy."""
    if a.is_cuda and a.dtype == torch.bfloat16:
        from ..ops import basic
        if basic.gemm_ok(a.shape[0], b.shape[1], a.shape[1]):
            return basic.gemm(a.contiguous(), b.contiguous(), b_mn=True)
    return a @ b


def orthogonalise(g, steps=5, eps=1e-7):
    """Approximate U·Vᵀ of g = U·S·Vᵀ by the quintic Newton-Schulz iteration (bf16 on the GPU, g's dtype on CPU)."""
    x = g.to(torch.bfloat16) if g.is_cuda else g.clone()
    tall = x.shape[0] > x.shape[1]
    if tall:
        x = x.t().contiguous()
    x = x / x.norm().clamp(min=eps)
    a, b, c = NS_COEFF
    for _ in range(steps):
        gram = _mm_nt(x, x)                               # (m, m), symmetric
        poly = b * gram + c * _mm_nt(gram, gram)
        x = a * x + _mm_nn(poly, x)
    return (x.t() if tall else x).to(g.dtype)


class MuonAdamW:
    def __init__(self, params, lr=1e-3, weight_decay=0.1, betas=(0.9, 0.95), mul=1.0, momentum=0.95, ns_steps=5):
        params = list(params)
        hidden = lambda p: p.dim() == 2 and p.shape[0] < 10000             # word tables are the 2-D tensors above that
        self.mats = [p for p in params if hidden(p)]
        rest = [p for p in params if not hidden(p)]
        self.mul, self.momentum, self.ns_steps, self.wd = mul, momentum, ns_steps, weight_decay
        self.buf = {id(p): torch.zeros_like(p, dtype=torch.float32) for p in self.mats}
        self.adam = torch.optim.AdamW(rest, lr=lr, betas=betas, weight_decay=weight_decay,
                                      fused=bool(rest) and rest[0].is_cuda) if rest else None
        self.param_groups = [dict(lr=lr)]

    @torch.no_grad()
    def step(self):
        lr = self.param_groups[0]["lr"]
        for p in self.mats:
            if p.grad is None:
                continue
            g = p.grad.float()
            m = self.buf[id(p)]
            m.lerp_(g, 1 - self.momentum)
            upd = orthogonalise(g.lerp(m, self.momentum), self.ns_steps)              # Nesterov look-ahead
            scale = 0.2 * math.sqrt(max(p.shape))                                     # RMS of an AdamW step
            p.mul_(1 - lr * self.mul * self.wd)
            p.add_(upd.to(p.dtype), alpha=-lr * self.mul * scale)
        if self.adam is not None:
            self.adam.param_groups[0]["lr"] = lr
            self.adam.step()

    def zero_grad(self, set_to_none=True):
        for p in self.mats:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()
        if self.adam is not None:
            self.adam.zero_grad(set_to_none=set_to_none)

    def state_dict(self):
        return {"muon": [self.buf[id(p)] for p in self.mats], "adam": self.adam.state_dict() if self.adam else None,
                "lr": self.param_groups[0]["lr"]}

    def load_state_dict(self, sd):
        for p, m in zip(self.mats, sd["muon"]):
            self.buf[id(p)].copy_(m)
        if self.adam is not None and sd.get("adam") is not None:
            self.adam.load_state_dict(sd["adam"])
        self.param_groups[0]["lr"] = sd.get("lr", self.param_groups[0]["lr"])
