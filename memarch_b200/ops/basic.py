"""Normalisation, activation and GEMM-shaped ops: autograd wrappers over the sm_100a kernels.

CUDA tensors take the hand-written kernels in `csrc/` (RMSNorm, relu², SwiGLU, tcgen05 GEMM); CPU tensors take the
PyTorch statement in `ref.py`.  Reference behaviour: `nn.RMSNorm` + bf16 autocast linears of the light blocks
(baseline.py:35-52, full.py:140-182), Triton SwiGLU (fused_ops.py:175-228), `_Relu2` (full.py:98-110).
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from . import _ext, ref

# What multiplies the *plain* linears (qkv/o/up/down of the light blocks): "tc" = this package's tcgen05 GEMM (the
# default), "lib" = cuBLAS (kept for A/B measurements).  The fused paths (experts, output head, attention,
# optimizer) always run this package's kernels.
PLAIN_GEMM = os.environ.get("MEMARCH_PLAIN_GEMM", "tc")


# ------------------------------------------------------------------------------------------------ RMSNorm
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, out_bf16):
        C = _ext.C()
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y, rstd = C.rmsnorm_fwd(x2, w.contiguous(), float(eps), bool(out_bf16))
        _ext.count()
        ctx.save_for_backward(x2, w, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        C = _ext.C()
        dx, dw, _ = C.rmsnorm_bwd(dy.reshape(x2.shape).contiguous(), x2, w.contiguous(), rstd, None, False)
        _ext.count(2)
        return dx.view(ctx.shape), dw.to(w.dtype), None, None


def rmsnorm(x, weight, eps=None, out_dtype=None):
    """RMSNorm in fp32 with one cast of the result.  `out_dtype` None keeps fp32 (CPU oracle) / x dtype."""
    if eps is None:
        eps = torch.finfo(torch.float32).eps if x.dtype in (torch.bfloat16, torch.float32) else torch.finfo(x.dtype).eps
    if _ext.use_cuda(x) and x.dtype in (torch.float32, torch.bfloat16) and x.shape[-1] % 8 == 0:
        want_bf16 = (out_dtype or x.dtype) == torch.bfloat16
        return _RMSNorm.apply(x, weight, eps, want_bf16)
    y = ref.rmsnorm(x, weight, eps)
    return y.to(out_dtype or x.dtype)


class _AddRMSNorm(torch.autograd.Function):
    """h = x + y (fp32 stream + bf16 branch) and n = rmsnorm(h)·w (bf16) in one kernel.  Backward folds the residual
    gradient into the norm's backward pass and emits the branch's bf16 gradient from the same kernel."""

    @staticmethod
    def forward(ctx, x, y, w, eps):
        C = _ext.C()
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        y2 = y.reshape(-1, shape[-1]).contiguous()
        h, n, rstd = C.add_rmsnorm_fwd(x2, y2, w.contiguous(), float(eps))
        _ext.count()
        ctx.save_for_backward(h, w, rstd)
        ctx.shape = shape
        return h.view(shape), n.view(shape)

    @staticmethod
    def backward(ctx, dh, dn):
        h, w, rstd = ctx.saved_tensors
        C = _ext.C()
        if dn is None:
            return dh, dh.to(torch.bfloat16), None, None
        add = dh.reshape(h.shape).contiguous().float() if dh is not None else None
        dx, dw, lo = C.rmsnorm_bwd(dn.reshape(h.shape).contiguous(), h, w.contiguous(), rstd, add, True)
        _ext.count(2)
        return dx.view(ctx.shape), lo.view(ctx.shape), dw.to(w.dtype), None


def add_rmsnorm(x, y, weight, eps=None):
    """(x + y, rmsnorm(x + y)·w): residual add fused with the following normalisation."""
    if eps is None:
        eps = torch.finfo(torch.float32).eps
    if _ext.use_cuda(x) and x.dtype == torch.float32 and y.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _AddRMSNorm.apply(x, y, weight, eps)
    h = x + y.to(x.dtype)
    return h, rmsnorm(h, weight, eps, out_dtype=torch.bfloat16 if x.is_cuda else None)


# ------------------------------------------------------------------------------------------------ activations
class _Relu2(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a):
        ctx.save_for_backward(a)
        _ext.count()
        return _ext.C().relu2_fwd(a.contiguous())

    @staticmethod
    def backward(ctx, dh):
        a, = ctx.saved_tensors
        _ext.count()
        return _ext.C().relu2_bwd(dh.contiguous(), a.contiguous())


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        _ext.count()
        return _ext.C().swiglu_fwd(gu.contiguous())

    @staticmethod
    def backward(ctx, dh):
        gu, = ctx.saved_tensors
        _ext.count()
        return _ext.C().swiglu_bwd(dh.contiguous(), gu.contiguous())


def relu2(a):
    if _ext.use_cuda(a) and a.dtype == torch.bfloat16:
        return _Relu2.apply(a)
    return ref.relu2(a)


def swiglu(gu):
    if _ext.use_cuda(gu) and gu.dtype == torch.bfloat16 and gu.shape[-1] % 16 == 0:
        return _SwiGLU.apply(gu)
    return ref.swiglu(gu)


class _ResidAdd(torch.autograd.Function):
    """fp32 residual stream + bf16 branch output in one pass; the branch gets its gradient in bf16."""

    @staticmethod
    def forward(ctx, x, y):
        _ext.count()
        return _ext.C().resid_add(x.contiguous(), y.contiguous())

    @staticmethod
    def backward(ctx, g):
        return g, g.to(torch.bfloat16)


def resid_add(x, y):
    """x + y with x the residual stream and y a block's branch output."""
    if _ext.use_cuda(x) and x.dtype == torch.float32 and y.dtype == torch.bfloat16 and x.numel() % 4 == 0:
        return _ResidAdd.apply(x, y)
    return x + y.to(x.dtype)


# ------------------------------------------------------------------------------------------------ GEMM
def gemm(a, b, *, a_mn=False, b_mn=False, out=None, out_dtype=torch.bfloat16, accumulate=False, epi=0,
         aux=None, out2=None, groups=1, counts=None, count_mode=0):
    """C[g] = A[g] · B[g]ᵀ on the tcgen05 tensor cores (bf16 in, fp32 accumulate in TMEM).

    Logical shapes per group: A (M,K), B (N,K), C (M,N).  Storage: an operand that is K-major is stored
    (rows, K) with K contiguous; `a_mn`/`b_mn` say the operand is stored (K, rows) with rows contiguous
    ("MN-major"), which is how a transposed view of a row-major matrix is fed without a transposing copy.
    `epi`: 0 plain, 1 relu² (out = relu(acc)², out2 = acc), 2 multiply by 2·relu(aux) (relu² backward),
    3 SwiGLU over column halves (B rows [n, H+n]), 4 per-row scale by aux (fp32 vector).
    `counts` (int32, one per group) with `count_mode` 1: only the first counts[g] rows of A[g] hold data (the rest is
    zero padding) - row tiles wholly past it are written as zeros without being computed; `count_mode` 2: only the
    first counts[g] positions of the contraction hold data - the k-blocks past it are not read.
    """
    C = _ext.C()
    _ext.count()
    m_, k_ = (a.shape[-1], a.shape[-2]) if a_mn else (a.shape[-2], a.shape[-1])
    n_ = b.shape[-1] if b_mn else b.shape[-2]
    _ext.count_flops(2 * m_ * n_ * k_ * max(1, int(groups)))
    return C.gemm(a, b, out, out2, aux, bool(a_mn), bool(b_mn), bool(accumulate), int(epi),
                  out_dtype == torch.float32, int(groups), counts, int(count_mode) if counts is not None else 0)


def gemm_ok(M, N, K):
    """Shapes the TMA descriptors accept: 16-byte row pitches (multiples of 8 bf16 elements)."""
    return K % 8 == 0 and N % 8 == 0 and M % 8 == 0 and K >= 16


class _Linear(torch.autograd.Function):
    """y = x · Wᵀ with W (out, in) bf16.  dx = dy · W (B operand MN-major), dW = dyᵀ · x (both MN-major)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return gemm(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy, w, b_mn=True)
        if ctx.needs_input_grad[1]:
            dw = gemm(dy, x, a_mn=True, b_mn=True)
        return dx, dw


# Set by the trainer when weights are stepped inside backward: callable(weight, bf16 gradient) -> True when it has
# consumed the gradient (stepped the weight), False to let autograd accumulate it as usual.
WEIGHT_GRAD_SINK = None


class _WeightBf16(torch.autograd.Function):
    """fp32 master weight -> the bf16 operand of the GEMMs.

    Forward hands out the weight's bf16 shadow, which the optimizer kernel rewrites together with the weight
    (`Instinct` passes `p._bf16_shadow` to `instinct_step`), so no per-step cast kernel runs; the shadow is rebuilt
    whenever the weight was changed by anything else (its version counter moved).  Backward gives the bf16 weight
    gradient straight to `WEIGHT_GRAD_SINK` - the optimizer step of this weight, inside backward, reading the
    gradient in bf16 - instead of casting it to fp32 for `.grad`; declined gradients flow on as usual."""

    @staticmethod
    def forward(ctx, w):
        ctx.w = w
        sh = getattr(w, "_bf16_shadow", None)
        if sh is None or sh.shape != w.shape:
            sh = w.detach().to(torch.bfloat16)
            w._bf16_shadow, w._shadow_ver = sh, w._version
        elif getattr(w, "_shadow_ver", None) != w._version:
            sh.copy_(w.detach())                   # refreshed in place: the buffer may be one that other ranks write into
            w._shadow_ver = w._version
        return sh.detach()

    @staticmethod
    def backward(ctx, g):
        sink = WEIGHT_GRAD_SINK
        if sink is not None and sink(ctx.w, g):
            return None
        return g


def weight_bf16(w, direct=False):
    """bf16 view of a weight for a GEMM.  `direct`: the weight is used once per step, so its gradient may go
    straight to the optimizer (see `_WeightBf16`)."""
    if w.dtype == torch.bfloat16:
        return w
    if direct and w.requires_grad and torch.is_grad_enabled() and w.is_leaf:
        return _WeightBf16.apply(w)
    sh = getattr(w, "_bf16_shadow", None)
    if sh is not None and not torch.is_grad_enabled() and getattr(w, "_shadow_ver", None) == w._version and sh.shape == w.shape:
        return sh                                   # evaluation: the shadow the optimizer keeps is the cast
    return w.to(torch.bfloat16)


class _LinearAct(torch.autograd.Function):
    """h = act(x · Wᵀ) with the activation in the GEMM epilogue (SwiGLU over the column halves of W's output, or
    relu²); the pre-activation is kept for the backward pass, which is one activation-backward kernel and the two
    gradient GEMMs."""

    @staticmethod
    def forward(ctx, x, w, swi):
        M, N = x.shape[0], w.shape[0]
        pre = torch.empty(M, N, device=x.device, dtype=torch.bfloat16)
        h = torch.empty(M, N // 2 if swi else N, device=x.device, dtype=torch.bfloat16)
        gemm(x, w, out=h, out2=pre, epi=3 if swi else 1)
        ctx.save_for_backward(x, w, pre)
        ctx.swi = swi
        return h

    @staticmethod
    def backward(ctx, dh):
        x, w, pre = ctx.saved_tensors
        C = _ext.C()
        _ext.count()
        dpre = C.swiglu_bwd(dh.contiguous(), pre) if ctx.swi else C.relu2_bwd(dh.contiguous(), pre)
        dx = gemm(dpre, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = gemm(dpre, x, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None
        return dx, dw, None


# SwiGLU backward inside the input-gradient GEMM's epilogue (2H pre-activations in, 2H gradients out per H accumulator
# columns): 0.97 ms at (32768, 8192, 2048) against 0.74 + 0.43 ms for the plain GEMM plus the elementwise kernel.  (With
# exp + IEEE division for the sigmoid it took 1.6 ms - one epilogue warp per scheduler cannot hide that dependent
# chain; the hardware tanh made it pay.)  relu² backward: 0.80 ms fused against 0.74 + 0.25 ms.
FUSE_DSWIGLU = True


class _FFN(torch.autograd.Function):
    """y = act(x · Wupᵀ) · Wdownᵀ as one autograd node, so that the backward of the activation rides in the epilogue
    of the GEMM that produces its input gradient: dpre = act'(pre) ∘ (dy · Wdown) is one GEMM (SwiGLU: both halves
    written side by side; relu²: times 2·relu(pre)), with no (rows, hidden) gradient tensor written and re-read."""

    @staticmethod
    def forward(ctx, x, w_up, w_down, swi):
        M, N = x.shape[0], w_up.shape[0]
        pre = torch.empty(M, N, device=x.device, dtype=torch.bfloat16)
        h = torch.empty(M, N // 2 if swi else N, device=x.device, dtype=torch.bfloat16)
        gemm(x, w_up, out=h, out2=pre, epi=3 if swi else 1)
        y = gemm(h, w_down)
        ctx.save_for_backward(x, w_up, w_down, pre, h)
        ctx.swi = swi
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w_up, w_down, pre, h = ctx.saved_tensors
        dy = dy.contiguous()
        if ctx.swi and not FUSE_DSWIGLU:
            dpre = _ext.C().swiglu_bwd(gemm(dy, w_down, b_mn=True), pre)
        else:
            dpre = gemm(dy, w_down, b_mn=True, epi=5 if ctx.swi else 2, aux=pre)
        d_down = gemm(dy, h, a_mn=True, b_mn=True) if ctx.needs_input_grad[2] else None
        dx = gemm(dpre, w_up, b_mn=True) if ctx.needs_input_grad[0] else None
        d_up = gemm(dpre, x, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None
        return dx, d_up, d_down, None


def ffn(x, w_up, w_down, act, direct=False):
    """act(x · Wupᵀ) · Wdownᵀ with act in {"swiglu", "relu2"} - the feed-forward half of a light block."""
    if _ext.use_cuda(x) and PLAIN_GEMM == "tc":
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)
        M, K = x2.shape
        N, D = w_up.shape[0], w_down.shape[0]
        H = N // 2 if act == "swiglu" else N
        if (gemm_ok(M, N, K) and gemm_ok(M, D, H) and M >= 256 and N % 16 == 0 and H % 8 == 0
                and w_down.shape[1] == H):
            y = _FFN.apply(x2.contiguous(), weight_bf16(w_up, direct).contiguous(), weight_bf16(w_down, direct).contiguous(),
                           act == "swiglu")
            return y.view(*x.shape[:-1], D)
    return linear(linear_act(x, w_up, act, direct=direct), w_down, direct=direct)


def linear_act(x, w, act, direct=False):
    """act(x · Wᵀ), act in {"swiglu", "relu2"}: one GEMM with the activation fused on the GPU."""
    if _ext.use_cuda(x) and PLAIN_GEMM == "tc":
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)
        wd = weight_bf16(w, direct)
        M, K = x2.shape
        N = wd.shape[0]
        if gemm_ok(M, N, K) and M >= 128 and N % 16 == 0:
            h = _LinearAct.apply(x2.contiguous(), wd.contiguous(), act == "swiglu")
            return h.view(*x.shape[:-1], h.shape[-1])
    y = linear(x, w, direct=direct)
    return relu2(y) if act == "relu2" else swiglu(y)


def linear(x, w, dtype=None, direct=False):
    """x (..., in) times W (out, in)ᵀ in `dtype` (bf16 on the GPU, the tensors' own dtype on CPU).  `direct`: see
    `weight_bf16`."""
    if _ext.use_cuda(x):
        dt = dtype or torch.bfloat16
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != dt:
            x2 = x2.to(dt)
        wd = weight_bf16(w, direct) if dt == torch.bfloat16 else (w if w.dtype == dt else w.to(dt))
        M, K = x2.shape
        N = wd.shape[0]
        if PLAIN_GEMM == "tc" and dt == torch.bfloat16 and gemm_ok(M, N, K) and M >= 128:
            y = _Linear.apply(x2.contiguous(), wd.contiguous())
        else:
            y = F.linear(x2, wd)
        return y.view(*x.shape[:-1], N)
    if dtype is not None and dtype != x.dtype:
        return F.linear(x.to(dtype), w.to(dtype))
    return F.linear(x, w.to(x.dtype))
