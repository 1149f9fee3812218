"""int8 matrix multiplication numerics (the reference's INT8_MM family, int8mm.py:1-111).

Scheme (SwitchBack / Jetfire style): forward `y = Q_row(x) · Q_row(W)ᵀ`, input gradient `dx = Q_row(g) · Q_col(W)`,
weight gradient in bf16 (the most sensitive sum: over all tokens).  Quantisation is symmetric, scale = max|·| / 127 per
input row and per output channel.  On the GPU the products run on the int8 tensor cores (`csrc/gemm_i8.cu`:
`tcgen05.mma.kind::i8`, int32 accumulators, scales applied in the epilogue) after the row quantiser kernel; on CPU the
integer values are held in floating point (|q| <= 127 is exact) and multiplied there - the same numbers up to the
rounding of the result.
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


def i8_ok(M, N, K):
    """Shapes the int8 tensor-core GEMM takes: 16-byte row pitch of the int8 operands."""
    return K % 16 == 0 and K >= 32 and M >= 1 and N >= 1


def quant_mm(x, w, out_dtype=torch.bfloat16):
    """Q_row(x) · Q_row(w)ᵀ with the scales applied: x (M,K) or (G,M,K), w (N,K) or (G,N,K), floating point in,
    int8 tensor cores on the GPU."""
    C = _ext.C()
    qx, sx = C.quant_rows_i8(x.contiguous())
    qw, sw = C.quant_rows_i8(w.contiguous())
    _ext.count(3)
    return C.gemm_i8(qx, qw, sx, sw, out_dtype == torch.float32)


def quant_mm_stored(x, w_q, w_s, out_dtype=torch.bfloat16):
    """Q_row(x) · w_qᵀ with the scales applied, for weights already stored as int8: x (G,M,K) floating point,
    w_q (G,N,K) int8, w_s (G,N) fp32 scale of every output column."""
    C = _ext.C()
    qx, sx = C.quant_rows_i8(x.contiguous())
    _ext.count(2)
    return C.gemm_i8(qx, w_q, sx, w_s, out_dtype == torch.float32)


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
        ctx.save_for_backward(x2, w)
        ctx.shape, ctx.dt = x.shape, x.dtype
        if _ext.use_cuda(x2) and x2.dtype in (torch.bfloat16, torch.float32) and w.dtype == x2.dtype and i8_ok(x2.shape[0], w.shape[0], K):
            y = quant_mm(x2, w, torch.float32)
        else:
            qx, sx = fq(x2, 1)
            qw, sw = fq(w, 1)
            y = _mm_t(qx, qw) * sx * sw.t()
        return y.to(x.dtype).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, g):
        x2, w = ctx.saved_tensors
        g2 = g.reshape(-1, w.shape[0])
        if _ext.use_cuda(g2) and g2.dtype in (torch.bfloat16, torch.float32) and w.dtype == g2.dtype and i8_ok(g2.shape[0], w.shape[1], w.shape[0]):
            # rows of Wᵀ quantised = W quantised along its input axis
            dx = quant_mm(g2.contiguous(), w.t().contiguous(), torch.float32).to(ctx.dt).reshape(ctx.shape)
        else:
            qg, sg = fq(g2, 1)
            qw, sw = fq(w, 0)                                   # scale along the input axis
            dx = (_mm_t(qg, qw.t().contiguous()) * sg * sw).to(ctx.dt).reshape(ctx.shape)
        dw = (g2.to(torch.bfloat16).t() @ x2.to(torch.bfloat16)).to(w.dtype)
        return dx, dw


class _I8Bmm(torch.autograd.Function):
    """(E,C,K) @ (E,K,N): scale per input row and per output column of every expert."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        if _ext.use_cuda(x) and x.dtype in (torch.bfloat16, torch.float32) and w.dtype == x.dtype and i8_ok(x.shape[1], w.shape[2], x.shape[2]):
            # (E,K,N) weights: the GEMM wants the contraction contiguous, i.e. rows of Wᵀ (scale per output column)
            return quant_mm(x, w.transpose(1, 2).contiguous(), torch.float32).to(x.dtype)
        qx, sx = fq(x, 2)
        qw, sw = fq(w, 1)
        y = _bmm_exact(qx, qw) * sx * sw
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        if _ext.use_cuda(g) and g.dtype in (torch.bfloat16, torch.float32) and w.dtype == g.dtype and i8_ok(g.shape[1], w.shape[1], w.shape[2]):
            dx = quant_mm(g.contiguous(), w, torch.float32).to(x.dtype)          # rows of W: scale per input row
        else:
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
