"""MoE data movement and expert FFN ops.

Reference behaviour: capacity slotting by cumulative rank, slot table gather `xpad[table]`, `bmm` experts with
SwiGLU or relu², weighted `index_add` combine (full2.py:532-602, 1102-1110), and the gather-only inverse pair
`_SlotGather` / `_CombineW` (full2.py:283-328) whose backward needs no scatter-add.

GPU bodies: `gather_rows` (slot <- token, optional per-row scale), `gather_sum_rows` (token <- its k slots, weighted,
fp32 accumulate), `row_dot` (slot-weight grads) and the grouped tcgen05 GEMMs with the activation in the epilogue.
"""
from __future__ import annotations

import os

import torch

from . import _ext, ref
from .basic import gemm, gemm_ok, relu2, swiglu


# ------------------------------------------------------------------------------------------------ dispatch
class _SlotGather(torch.autograd.Function):
    """xe[s] = x[table[s]] (empty slot -> 0).  Backward: dx[n] = Σ_j dxe[flat_idx[n, j]] in fp32."""

    @staticmethod
    def forward(ctx, x, table, flat_idx):
        ctx.save_for_backward(table, flat_idx)
        ctx.N = x.shape[0]
        if _ext.use_cuda(x):
            _ext.count()
            return _ext.C().gather_rows(x.contiguous(), table, None)
        N = x.shape[0]
        m = (table < N)[:, None]
        return torch.where(m, x[table.clamp(max=N - 1)], x.new_zeros(()))

    @staticmethod
    def backward(ctx, g):
        table, fi = ctx.saved_tensors
        if _ext.use_cuda(g):
            _ext.count()
            return _ext.C().gather_sum_rows(g.contiguous(), fi, None, ctx.N), None, None
        EC = g.shape[0]
        mk = (fi < EC)[..., None]
        dx = torch.where(mk, g[fi.clamp(max=EC - 1)], g.new_zeros(())).float().sum(1).to(g.dtype)
        return dx, None, None


class _CombineW(torch.autograd.Function):
    """out[n] = Σ_j ye[fi[n,j]] · wtab[fi[n,j]] (fp32 sum).  Backward: dye[s] = wtab[s]·go[table[s]],
    dwtab[s] = <go[table[s]], ye[s]>."""

    @staticmethod
    def forward(ctx, ye, wtab, fi, table, N):
        ctx.save_for_backward(ye, wtab, fi, table)
        ctx.N = N
        if _ext.use_cuda(ye):
            _ext.count()
            return _ext.C().gather_sum_rows(ye.contiguous(), fi, wtab.float().contiguous(), N)
        EC = ye.shape[0]
        c = fi.clamp(max=EC - 1)
        mk = fi < EC
        wg = torch.where(mk, wtab[c], wtab.new_zeros(()))
        return (ye[c].float() * wg[..., None].float()).sum(1).to(ye.dtype)

    @staticmethod
    def backward(ctx, go):
        ye, wtab, fi, table = ctx.saved_tensors
        N = ctx.N
        if _ext.use_cuda(go):
            C = _ext.C()
            go = go.contiguous()
            dye = C.gather_rows(go, table, wtab.float().contiguous())
            dw = C.row_dot(go, table, ye.contiguous())
            _ext.count(2)
            return dye, dw.to(wtab.dtype), None, None, None
        m = (table < N)[:, None]
        gs = torch.where(m, go[table.clamp(max=N - 1)], go.new_zeros(()))
        dye = (gs.float() * wtab[:, None].float()).to(ye.dtype)
        dw = (gs.float() * ye.float()).sum(-1).to(wtab.dtype)
        return dye, dw, None, None, None


def slot_gather(x, table, flat_idx):
    return _SlotGather.apply(x, table, flat_idx)


def combine(ye, wtab, flat_idx, table, N):
    return _CombineW.apply(ye, wtab, flat_idx, table, N)


# ------------------------------------------------------------------------------------------------ expert FFN
class _ExpertFFN(torch.autograd.Function):
    """(E,C,d) -> relu²/SwiGLU FFN -> (E,C,d) on grouped tcgen05 GEMMs, activation in the up-GEMM epilogue.

    `train_w` False (frozen bank) skips both weight-gradient GEMMs.  `counts` (int32, E): filled places per expert;
    the places after them are zero rows, so the GEMMs skip their row tiles (forward, input gradients) and their
    k-blocks (weight gradients) - the dropless form of the same arithmetic.
    """

    @staticmethod
    def forward(ctx, xe, up, down, act, train_w, counts):
        E, Cn, d = xe.shape
        xe = xe.contiguous()
        cm = 1 if counts is not None and Cn >= 256 else 0
        kw = dict(groups=E, counts=counts if cm else None, count_mode=cm)
        if act == "relu2":
            H = up.shape[2]
            h = torch.empty(E, Cn, H, device=xe.device, dtype=torch.bfloat16)
            a = torch.empty_like(h)
            gemm(xe, up, b_mn=True, out=h, out2=a, epi=1, **kw)
        elif up.shape[2] % 16 == 0 and Cn >= 256:
            H = up.shape[2] // 2
            h = torch.empty(E, Cn, H, device=xe.device, dtype=torch.bfloat16)
            a = torch.empty(E, Cn, 2 * H, device=xe.device, dtype=torch.bfloat16)
            gemm(xe, up, b_mn=True, out=h, out2=a, epi=3, **kw)                # SwiGLU in the epilogue
        else:
            a = gemm(xe, up, b_mn=True, **kw)
            h = _ext.C().swiglu_fwd(a)
            _ext.count()
        y = gemm(h, down, b_mn=True, **kw)
        ctx.save_for_backward(xe, up, down, a, h, counts if cm else None)
        ctx.act, ctx.train_w = act, train_w
        return y

    @staticmethod
    def backward(ctx, dy):
        xe, up, down, a, h, counts = ctx.saved_tensors
        E = xe.shape[0]
        dy = dy.contiguous()
        cm = 1 if counts is not None else 0
        kw = dict(groups=E, counts=counts, count_mode=cm)
        if ctx.act == "relu2":
            da = gemm(dy, down, epi=2, aux=a, **kw)                            # dh · 2relu(a)
        else:
            dh = gemm(dy, down, **kw)
            da = _ext.C().swiglu_bwd(dh, a)
            _ext.count()
        dxe = gemm(da, up, **kw) if ctx.needs_input_grad[0] else None
        dup = ddown = None
        if ctx.train_w:
            kw = dict(groups=E, counts=counts, count_mode=2 * cm)
            # weight gradients contract over the places: the pair kernel needs >= 256 output rows (H, d)
            ddown = gemm(h, dy, a_mn=True, b_mn=True, **(kw if h.shape[2] >= 256 else dict(groups=E)))
            dup = gemm(xe, da, a_mn=True, b_mn=True, **(kw if xe.shape[2] >= 256 else dict(groups=E)))
        return dxe, dup, ddown, None, None, None


def expert_ffn(xe, up, down, act="swiglu", train_w=True, counts=None):
    """xe (E,C,d); up (E,d,H); down (E,H',d).  bf16 on the GPU; CPU: plain bmm in the input dtype.
    `counts` (int32 per expert, optional): rows of xe[e] past counts[e] are zero padding and are not computed."""
    E, Cn, d = xe.shape
    if (_ext.use_cuda(xe) and xe.dtype == torch.bfloat16 and up.dtype == torch.bfloat16
            and gemm_ok(Cn if Cn % 8 == 0 else 8, up.shape[2], d) and down.shape[1] % 8 == 0):
        return _ExpertFFN.apply(xe, up, down, act, train_w and up.requires_grad, counts)
    h = torch.bmm(xe, up.to(xe.dtype))
    h = relu2(h) if act == "relu2" else swiglu(h)
    return torch.bmm(h, down.to(xe.dtype))


# ------------------------------------------------------------------------------------------------ routing
class _Route(torch.autograd.Function):
    """Fused router tail on the GPU: softmax, top-k_max, budget mask, renormalised weights and the two per-expert
    sums of the auxiliary loss in one kernel; backward in one kernel (`csrc/select.cu`)."""

    @staticmethod
    def forward(ctx, logits, real, k_tok, k_max):
        C = _ext.C()
        probs, top_e, w, e_flat, cnt, psum = C.moe_route_fwd(logits.contiguous(), real.contiguous(), k_tok.contiguous(), int(k_max))
        _ext.count()
        ctx.save_for_backward(probs, top_e, k_tok, real)
        ctx.mark_non_differentiable(top_e, e_flat, cnt)
        return w, psum, top_e, e_flat, cnt, probs

    @staticmethod
    def backward(ctx, dw, dpsum, _a, _b, _c, dprobs):
        probs, top_e, k_tok, real = ctx.saved_tensors
        dl = _ext.C().moe_route_bwd(probs, top_e, k_tok.contiguous(), real.contiguous(), dw.contiguous().float(),
                                    dprobs.contiguous().float() if dprobs is not None else None,
                                    dpsum.contiguous().float() if dpsum is not None else None)
        _ext.count()
        return dl, None, None, None


def moe_route(xf, router_w, real, k_tok, k_max, E):
    """(probs, top_e, keep, w, e_flat, aux) - the CUDA kernel on the GPU, `ref.moe_route` elsewhere."""
    if _ext.use_cuda(xf) and E <= 128 and k_max <= 8:
        logits = (xf.to(router_w.dtype) @ router_w.T).float()
        w, psum, top_e, e_flat, cnt, probs = _Route.apply(logits, real, k_tok, k_max)
        pm = psum / real.sum().clamp(min=1)
        aux = E * (cnt / cnt.sum().clamp(min=1) * pm).sum()
        keep = torch.arange(k_max, device=xf.device)[None] < k_tok[:, None]
        return probs, top_e, keep, w, e_flat, aux
    return ref.moe_route(xf, router_w, real, k_tok, k_max, E)


def route_and_slot(xf, router_w, real, k_tok, k_max, E, C, want_counts=False):
    """Router + capacity slotting.  Returns (w (N,k), table, wtab, flat_idx, aux, dropped, probs) and, with
    `want_counts`, the filled places per expert (int32 on the GPU, None on CPU) as an eighth value."""
    probs, top_e, keep, w, e_flat, aux = moe_route(xf, router_w, real, k_tok, k_max, E)
    counts = None
    with torch.no_grad():
        if _ext.use_cuda(xf):
            table, flat_idx, dropped, counts = _ext.C().moe_slots(e_flat.contiguous(), int(E), int(C))
            _ext.count()
        else:
            table, _, flat_idx, dropped = ref.moe_slots(e_flat, w.detach(), E, C)
    ok = flat_idx < E * C
    if not _ext.use_cuda(xf) and os.environ.get("CHECK") == "1":
        # CHECK=1 (CPU only): every choice that got a place and that place point at each other (full2.py:567-570)
        tok = torch.arange(flat_idx.shape[0], device=xf.device)[:, None].expand_as(flat_idx)
        assert bool((table[flat_idx[ok]] == tok[ok]).all()), "slot table and inverse table disagree"
        assert int((table < flat_idx.shape[0]).sum()) == int(ok.sum()), "filled places and placed choices differ"
    # slot weights as a differentiable gather-free scatter: wtab[flat_idx[n,j]] = w[n,j]
    wtab = torch.zeros(E * C + 1, device=xf.device, dtype=w.dtype).scatter(
        0, flat_idx.reshape(-1), (w * ok).reshape(-1))[:-1]
    if want_counts:
        return w, table, wtab, flat_idx, aux, dropped, probs, counts
    return w, table, wtab, flat_idx, aux, dropped, probs
