"""Input embedding sum of the memarch model as one op: token row + gated rows of the lock finder's candidates +
phrase-table row.

Reference behaviour: the input side of `FullLM2.forward` (full2.py:1538-1600): `h = emb(x)`, `h += (emb(cand) *
sel[..., None]).sum(2)` (INDUCT_IN), `h += phr(idx)`.  GPU body: `csrc/embed.cu` (one gather-sum kernel forward; the
backward scatters the gradient rows into the tables with vector reductions and forms d sel on the way).  CPU body: the
PyTorch statement.
"""
from __future__ import annotations

import torch

from . import _ext


class _EmbedSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, emb, x, cand, sel, phr, pidx):
        C = _ext.C()
        xf = x.reshape(-1).contiguous()
        cf = cand.reshape(-1, cand.shape[-1]).contiguous() if cand is not None else None
        sf = sel.reshape(-1, sel.shape[-1]).float().contiguous() if sel is not None else None
        pf = pidx.reshape(-1).contiguous() if pidx is not None else None
        h = C.embed_sum_fwd(emb, xf, cf, sf, phr, pf)
        _ext.count()
        ctx.save_for_backward(emb, xf, cf, sf, pf)
        ctx.P = phr.shape[0] if phr is not None else 0
        ctx.sel_shape = sel.shape if sel is not None else None
        ctx.sel_dtype = sel.dtype if sel is not None else None
        return h.view(*x.shape, emb.shape[1])

    @staticmethod
    def backward(ctx, dh):
        emb, xf, cf, sf, pf = ctx.saved_tensors
        C = _ext.C()
        d = emb.shape[1]
        demb, dphr, dsel = C.embed_sum_bwd(dh.reshape(-1, d).float().contiguous(), emb, xf, cf, sf, int(ctx.P), pf)
        _ext.count()
        return (demb, None, None, dsel.view(ctx.sel_shape).to(ctx.sel_dtype) if ctx.sel_shape is not None else None,
                dphr if ctx.P else None, None)


def embed_sum(emb, x, cand=None, sel=None, phr=None, pidx=None):
    """emb[x] + Σ_k sel[..., k] · emb[cand[..., k]] + phr[pidx]; emb (V,d), phr (P,d), x / pidx (...), cand / sel (..., K)."""
    if (_ext.use_cuda(emb) and emb.dtype == torch.float32 and emb.shape[1] % 4 == 0 and emb.is_contiguous()
            and (phr is None or (phr.dtype == torch.float32 and phr.is_contiguous()))):
        return _EmbedSum.apply(emb, x, cand, sel, phr, pidx)
    h = torch.nn.functional.embedding(x, emb)
    if cand is not None:
        h = h + (torch.nn.functional.embedding(cand, emb) * sel[..., None].to(h.dtype)).sum(-2)
    if phr is not None:
        h = h + torch.nn.functional.embedding(pidx, phr).type_as(h)
    return h
