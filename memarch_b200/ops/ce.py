"""Fused output projection + cross-entropy (+ pointer mixture, + sparse logit bias).

Behaviour of the reference's `_LinearCE`, `_LinearCESparse`, `_LinearCEMix` (fused_ops.py:39-167): rows are
processed in chunks; the logits of a chunk are produced by a GEMM, one row kernel turns them in place into
d(loss)/d(logits) while emitting the per-row loss, and the two gradient GEMMs (dh = G·W, dW += Gᵀ·h) run in the same
forward pass, so the N×V logits are never kept and never recomputed.  Backward only scales by the upstream grad.

GPU body: tcgen05 GEMMs (`gemm`, fp32 accumulation of dW across chunks inside the kernel) + `ce_rows` row kernel.
"""
from __future__ import annotations

import torch

from . import _ext, ref
from .basic import gemm, gemm_ok

CE_ROWS_CHUNK = 4096


def _ce_forward_cuda(h, w, y, gate, hit, cand, cval, chunk):
    C = _ext.C()
    N, d = h.shape
    V = w.shape[0]
    hd = h.to(torch.bfloat16).contiguous()
    wd = w.to(torch.bfloat16).contiguous()
    gh = torch.empty_like(hd)
    gw = torch.zeros(V, d, device=h.device, dtype=torch.float32)
    loss = torch.empty(N, device=h.device, dtype=torch.float32)
    dg = torch.empty(N, device=h.device, dtype=torch.float32) if gate is not None else None
    dcv = torch.empty(cval.shape, device=h.device, dtype=torch.float32) if cval is not None else None
    gf = gate.float().contiguous() if gate is not None else None
    hf = hit.float().contiguous() if hit is not None else None
    y = y.contiguous()
    logits = torch.empty(min(chunk, N), V, device=h.device, dtype=torch.bfloat16)
    for i in range(0, N, chunk):
        n = min(chunk, N - i)
        hc = hd[i:i + n]
        lg = logits[:n]
        gemm(hc, wd, out=lg)                                                # (n, V) bf16
        if cand is not None:
            lg.scatter_add_(-1, cand[i:i + n], cval[i:i + n].to(lg.dtype))
        C.ce_rows(lg, y[i:i + n], loss[i:i + n],
                  gf[i:i + n] if gf is not None else None, hf[i:i + n] if hf is not None else None,
                  dg[i:i + n] if dg is not None else None)
        _ext.count()
        if dcv is not None:
            dcv[i:i + n] = lg.gather(-1, cand[i:i + n]).float()
        gemm(lg, wd, b_mn=True, out=gh[i:i + n])                            # dh = G · W
        gemm(lg, hc, a_mn=True, b_mn=True, out=gw, out_dtype=torch.float32, accumulate=True)   # dW += Gᵀ · h
    return loss.sum(), gh, gw, dg, dcv


class _LinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, y, gate, hit, cand, cval, chunk, mm_dtype):
        if _ext.use_cuda(h) and gemm_ok(min(chunk, h.shape[0]), w.shape[0], h.shape[1]):
            total, gh, gw, dg, dcv = _ce_forward_cuda(h, w, y, gate, hit, cand, cval, chunk)
        else:
            total, gh, gw, _, dg, dcv = ref.linear_ce(h, w, y, None, gate, hit, cand, cval, chunk, mm_dtype)
        ctx.save_for_backward(gh, gw, dg if dg is not None else gh.new_zeros(0),
                              dcv if dcv is not None else gh.new_zeros(0))
        ctx.meta = (h.dtype, w.dtype, gate is not None, gate.dtype if gate is not None else None,
                    cval is not None, cval.dtype if cval is not None else None)
        return total

    @staticmethod
    def backward(ctx, go):
        gh, gw, dg, dcv = ctx.saved_tensors
        hdt, wdt, has_g, gdt, has_c, cdt = ctx.meta
        return ((gh * go).to(hdt), (gw * go).to(wdt), None,
                (dg * go).to(gdt) if has_g else None, None, None,
                (dcv * go).to(cdt) if has_c else None, None, None)


def linear_ce(h, w, y, gate=None, hit=None, cand=None, cval=None, chunk=CE_ROWS_CHUNK, mm_dtype=None):
    """Sum over rows of CE(h·Wᵀ, y); with `gate`/`hit` the pointer-mixture loss; with `cand`/`cval` a sparse
    additive logit bias.  h (..., d), w (V, d), y (...)."""
    h2 = h.reshape(-1, h.shape[-1])
    y1 = y.reshape(-1)
    if gate is not None:
        gate, hit = gate.reshape(-1), hit.reshape(-1)
    if cand is not None:
        cand, cval = cand.reshape(-1, cand.shape[-1]).long(), cval.reshape(-1, cval.shape[-1])
    return _LinearCE.apply(h2, w, y1, gate, hit, cand, cval, chunk, mm_dtype)


class _ChunkLSE(torch.autograd.Function):
    """(lse, target logit) per row with vocabulary chunks; logits live one chunk at a time both ways
    (full2.py:753-831)."""

    @staticmethod
    def forward(ctx, h, W, b, y, ch):
        lse, ly = ref.chunk_lse(h, W, b, y, ch)
        ctx.save_for_backward(h, W, b if b is not None else h.new_zeros(0), y, lse)
        ctx.ch, ctx.has_b = ch, b is not None
        return lse, ly

    @staticmethod
    def backward(ctx, g_lse, g_ly):
        h, W, b, y, lse = ctx.saved_tensors
        b = b if ctx.has_b else None
        hb, Wb = h.to(torch.bfloat16), W.to(torch.bfloat16)
        dh = torch.zeros(h.shape, device=h.device, dtype=torch.float32)
        dW, db = [], []
        for c0 in range(0, W.shape[0], ctx.ch):
            lo = (hb @ Wb[c0:c0 + ctx.ch].T).float()
            if b is not None:
                lo = lo + b[c0:c0 + ctx.ch].float()
            n = lo.shape[1]
            hit = torch.arange(c0, c0 + n, device=y.device)[None] == y[:, None]
            G = g_lse[:, None] * (lo - lse[:, None]).exp() + g_ly[:, None] * hit
            Gb = G.to(torch.bfloat16)
            dh = dh + (Gb @ Wb[c0:c0 + n]).float()
            dW.append((Gb.T @ hb).float())
            if b is not None:
                db.append(G.sum(0))
        return (dh.to(h.dtype), torch.cat(dW).to(W.dtype), torch.cat(db).to(b.dtype) if b is not None else None,
                None, None)


def chunk_ce(h, W, b, y, ch):
    return _ChunkLSE.apply(h, W, b, y, ch)
