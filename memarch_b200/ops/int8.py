"""int8 matrix multiplication numerics (the reference's INT8_MM family, int8mm.py:1-111).

Scheme (SwitchBack / Jetfire style): forward `y = Q_row(x) · Q_row(W)ᵀ`, input gradient `dx = Q_row(g) · Q_col(W)`,
weight gradient in bf16 (the most sensitive sum: over all tokens).  Quantisation is symmetric, scale = max|·| / 127 per
input row and per output channel.  The integer values (|q| <= 127) are exact in bf16, so multiplying them on the bf16
tensor cores with fp32 accumulation equals an int8 multiply with int32 accumulation up to one rounding of the sum;
that is what runs here (through the tcgen05 GEMM on the GPU), which makes the *quality* of an int8 run measurable on
this hardware.  An `kind::i8` tensor-core path would change the speed, not these numbers.
"""
from __future__ import annotations

import torch

from . import _ext
from .basic import gemm, gemm_ok


def fq(x, dim):
    """Symmetric quantisation along `dim` -> (integer values held in bf16, fp32 scale shaped like the max)."""
    xf = x.float()
    s = xf.abs().amax(dim=dim, keepdim=True).clamp(min=1e-12) / 127.0
    q = torch.round(xf / s).clamp(-127, 127)
    return q.to(torch.bfloat16), s


def _mm_t(a, b):
    """a (M,K) · b (N,K)ᵀ with fp32 result; tcgen05 GEMM on the GPU."""
    if _ext.use_cuda(a):
        M, K = a.shape
        N = b.shape[0]
        if gemm_ok(M, N, K) and M >= 128:
            # integers up to 127 are exact in bf16 and their dot products are exact in the fp32 accumulator: the
            # result must leave the kernel in fp32 too, a bf16 store would round away the low digits
            out = torch.zeros(M, N, device=a.device, dtype=torch.float32)
            gemm(a.contiguous(), b.contiguous(), out=out, out_dtype=torch.float32, accumulate=True)
            return out
    return a.float() @ b.float().t()


def _bmm_exact(a, b):
    """Batched product of integer-valued bf16 operands with an exact fp32 result (a bf16 result would round it)."""
    return torch.bmm(a.float(), b.float())


class _I8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        qx, sx = fq(x2, 1)
        qw, sw = fq(w, 1)
        y = _mm_t(qx, qw) * sx * sw.t()
        ctx.save_for_backward(x2, w)
        ctx.shape, ctx.dt = x.shape, x.dtype
        return y.to(x.dtype).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, g):
        x2, w = ctx.saved_tensors
        g2 = g.reshape(-1, w.shape[0])
        qg, sg = fq(g2, 1)
        qw, sw = fq(w, 0)                                   # scale along the input axis
        dx = (_mm_t(qg, qw.t().contiguous()) * sg * sw).to(ctx.dt).reshape(ctx.shape)
        dw = (g2.to(torch.bfloat16).t() @ x2.to(torch.bfloat16)).to(w.dtype)
        return dx, dw


class _I8Bmm(torch.autograd.Function):
    """(E,C,K) @ (E,K,N): scale per input row and per output column of every expert."""

    @staticmethod
    def forward(ctx, x, w):
        qx, sx = fq(x, 2)
        qw, sw = fq(w, 1)
        y = _bmm_exact(qx, qw) * sx * sw
        ctx.save_for_backward(x, w)
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        qg, sg = fq(g, 2)
        qw, sw = fq(w, 2)
        dx = (_bmm_exact(qg, qw.transpose(1, 2)) * sg * sw.transpose(1, 2)).to(x.dtype)
        dw = torch.bmm(x.to(torch.bfloat16).transpose(1, 2), g.to(torch.bfloat16)).to(w.dtype)
        return dx, dw


def linear_i8(x, w, min_dim=256):
    if w.dim() == 2 and min(w.shape) >= min_dim and x.is_floating_point():
        return _I8Linear.apply(x, w)
    return torch.nn.functional.linear(x, w.to(x.dtype))


def bmm_i8(x, w, min_dim=256):
    if min(x.shape[-1], w.shape[-1]) >= min_dim and x.is_floating_point():
        return _I8Bmm.apply(x, w)
    return torch.bmm(x, w)
