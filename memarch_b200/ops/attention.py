"""Causal / sliding-window attention with RoPE for the light and final blocks.

Reference behaviour: `F.scaled_dot_product_attention(rope(q), rope(k), v, is_causal=True)` when the text fits the
window (full.py:156-157); block-masked window attention `kv <= q and q - kv < window` otherwise (FlexAttention with
an O(T) block list, full2.py:153-181; two-block variants lm.py:448-554).

GPU body: `rope_qk` kernel (rotation of the q and k thirds of the packed qkv activations, `rope_merge_bwd` packs and
rotates the three gradients back in one pass) followed by the attention core: the library flash kernel by default
(`MEMARCH_ATTN=lib`), or the own tcgen05 forward kernel `attn_fwd_tc` (`MEMARCH_ATTN=own`, head dim 64: block list from
window arithmetic, no mask tensor, exact LSE; its backward recomputes through the library).
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from . import _ext, ref

ATTN_CORE = os.environ.get("MEMARCH_ATTN", "lib")
OWN_WINDOW_EVAL = os.environ.get("MEMARCH_ATTN_EVAL", "own") == "own"
OWN_BWD = os.environ.get("MEMARCH_ATTN_BWD", "own") == "own"
WINDOW_BODY = os.environ.get("MEMARCH_WINDOW", "flash")        # library body of windowed attention with backward: flash | block


_tables = {}


def rope_tables(T, hd, device):
    """(T, hd/2) fp32 cos / sin tables, built once per (T, hd, device)."""
    key = (T, hd, str(device))
    if key not in _tables:
        cos, sin = ref.rope_angles(T, hd, device)
        _tables[key] = (cos.contiguous(), sin.contiguous())
    return _tables[key]


class _RopeQK(torch.autograd.Function):
    """Rotate the q and k slices of qkv (B,T,3,H,hd); v passes through.  Backward rotates the grads back."""

    @staticmethod
    def forward(ctx, qkv, half):
        ctx.half = half
        cos, sin = rope_tables(qkv.shape[1], qkv.shape[4], qkv.device)
        _ext.count()
        return _ext.C().rope_qk(qkv.contiguous(), cos, sin, 1.0, bool(half))

    @staticmethod
    def backward(ctx, g):
        cos, sin = rope_tables(g.shape[1], g.shape[4], g.device)
        _ext.count()
        return _ext.C().rope_qk(g.contiguous(), cos, sin, -1.0, bool(ctx.half)), None


class _RopeSplit(torch.autograd.Function):
    """Rotate q,k and hand q,k,v to the attention core as (B,H,T,hd) views of one packed tensor.  Backward takes the
    three separate gradients (any batch/head/token strides), rotates back and packs them in one pass."""

    @staticmethod
    def forward(ctx, qkv, half):
        ctx.half = half
        cos, sin = rope_tables(qkv.shape[1], qkv.shape[4], qkv.device)
        _ext.count()
        r = _ext.C().rope_qk(qkv.contiguous(), cos, sin, 1.0, bool(half))
        return r[:, :, 0].transpose(1, 2), r[:, :, 1].transpose(1, 2), r[:, :, 2].transpose(1, 2)

    @staticmethod
    def backward(ctx, dq, dk, dv):
        cos, sin = rope_tables(dq.shape[2], dq.shape[3], dq.device)
        fix = lambda t: t if (t.stride(3) == 1 and t.stride(0) % 8 == 0 and t.stride(1) % 8 == 0 and t.stride(2) % 8 == 0) \
            else t.contiguous()
        _ext.count()
        return _ext.C().rope_merge_bwd(fix(dq), fix(dk), fix(dv), cos, sin, bool(ctx.half)), None


class _OwnAttn(torch.autograd.Function):
    """Attention core on the own tcgen05 kernels (`csrc/attn_tc.cu`, `csrc/attn_bwd_tc.cu`): S = QKt, O = PV and the five
    backward products on the tensor cores with TMEM accumulators, softmax by one thread per row, block lists from
    window arithmetic, exact LSE.  `MEMARCH_ATTN_BWD=lib` makes backward recompute through the library instead."""

    @staticmethod
    def forward(ctx, q, k, v, window):
        C = _ext.C()
        qc, kc, vc = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse = C.attn_fwd_tc(qc, kc, vc, int(window), float(q.shape[-1]) ** -0.5)
        _ext.count()
        ctx.save_for_backward(qc, kc, vc, o, lse)
        ctx.window = int(window)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        if OWN_BWD:
            do = do.contiguous()
            delta = (do.float() * o.float()).sum(-1)
            dq, dk, dv = _ext.C().attn_bwd_tc(q, k, v, do, lse, delta, ctx.window, float(q.shape[-1]) ** -0.5)
            _ext.count()
            return dq.to(q.dtype), dk, dv, None
        q, k, v = (t.detach().requires_grad_() for t in (q, k, v))
        with torch.enable_grad():
            o2 = F.scaled_dot_product_attention(q, k, v, is_causal=True) if ctx.window == 0 else _lib_window(q, k, v, ctx.window)
        dq, dk, dv = torch.autograd.grad(o2, (q, k, v), do)
        return dq, dk, dv, None


def own_attention(q, k, v, window=0):
    """q, k, v (B,H,T,64) bf16 with RoPE applied -> o (B,H,T,64); `window` 0 = plain causal."""
    return _OwnAttn.apply(q, k, v, int(window or 0))


def _lib_window(q, k, v, window):
    """Two-block dense-mask window attention through SDPA: each block of `window` queries sees itself and the
    previous block (2·window keys); linear cost in T."""
    B, H, T, D = q.shape
    W = window
    nb = -(-T // W)
    pad = nb * W - T
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, pad)) for t in (q, k, v))
    qb, kb, vb = (t.reshape(B, H, nb, W, D) for t in (q, k, v))
    prev = lambda t: torch.cat([torch.zeros_like(t[:, :, :1]), t[:, :, :-1]], 2)
    kk, vv = torch.cat([prev(kb), kb], 3), torch.cat([prev(vb), vb], 3)
    i = torch.arange(W, device=q.device)[:, None]
    j = torch.arange(2 * W, device=q.device)[None]
    ok = (j > i) & (j <= i + W)
    first = torch.arange(nb, device=q.device)[:, None, None] > 0
    mask = ok[None] & (first | (j >= W)[None])
    qb, kk, vv = qb.reshape(B, H * nb, W, D), kk.reshape(B, H * nb, 2 * W, D), vv.reshape(B, H * nb, 2 * W, D)
    mask = mask[None].expand(H, nb, W, 2 * W).reshape(1, H * nb, W, 2 * W)
    out = F.scaled_dot_product_attention(qb, kk, vv, attn_mask=mask)
    return out.reshape(B, H, nb * W, D)[:, :, :T]


_flash_window_ok = [None]


def _flash_window(q, k, v, window):
    """Sliding-window causal attention through the library flash kernel's own window arguments (key j is visible to
    query i iff 0 <= i - j < window): cost proportional to the window, forward and backward.  q, k, v (B,H,T,hd).
    Falls back to the two-block dense-mask form if this build of the library has no windowed flash kernel."""
    if _flash_window_ok[0] is not False and WINDOW_BODY == "flash":
        try:
            T = q.shape[2]
            o = torch.ops.aten._flash_attention_forward(
                q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), None, None, T, T, 0.0, True, False,
                scale=None, window_size_left=int(window) - 1, window_size_right=0)[0]
            _flash_window_ok[0] = True
            return o.transpose(1, 2)
        except Exception:   # noqa: BLE001 - older library: no window arguments / unsupported head size
            if _flash_window_ok[0] is True:
                raise
            _flash_window_ok[0] = False
    return _lib_window(q, k, v, window)


def attention(qkv, window=None, rope_half=False, qk_norm=False):
    """qkv (B,T,3,H,hd) -> (B,T,H·hd).  `window` None or >= T means plain causal."""
    B, T, _, H, hd = qkv.shape
    win = None if (window is None or window >= T) else int(window)
    if _ext.use_cuda(qkv) and qkv.dtype == torch.bfloat16 and not qk_norm and hd % 8 == 0:
        q, k, v = _RopeSplit.apply(qkv, rope_half)
        # own tcgen05 kernel: everywhere when asked for; by default where it is the faster one, i.e. sliding-window
        # attention without a backward pass (evaluation / generation at long context: only the blocks under the window
        # are visited, 3.4x faster than the dense-mask library form at T = 16k, window 256)
        no_grad = not (torch.is_grad_enabled() and qkv.requires_grad)
        if hd == 64 and (ATTN_CORE == "own" or (ATTN_CORE == "lib" and win is not None and no_grad and OWN_WINDOW_EVAL)):
            return own_attention(q, k, v, win or 0).transpose(1, 2).reshape(B, T, H * hd)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True) if win is None else _flash_window(q, k, v, win)
        return o.transpose(1, 2).reshape(B, T, H * hd)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    o = ref.window_attention(q, k, v, win, rope_half, qk_norm=qk_norm)
    return o.reshape(B, T, H * hd)
