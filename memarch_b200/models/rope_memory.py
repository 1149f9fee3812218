"""Anchor-routed long-range attention ("rope memory"; the reference's JAX port, rope.py:1-500).

Anchors are the surprising tokens.  Every anchor owns the span of text from itself to the next anchor (at most
`span_cap` tokens) and is found by its first `links` keys.  A query scores every earlier anchor by its best link,
opens its top-`K` anchors and attends with ONE softmax over its local window (`win` tokens, causal) and the tokens of
the opened spans that lie before the window.  The cost per token does not depend on the text length: window + K spans.

Routing is exact (every query against every anchor's links) and runs under `no_grad`; with `rgrad` the routing score of
an opened anchor is added as a bias to all keys of its span, which is how the choice receives a gradient.
Reading is the dense-mask formulation (scores against all T keys, spans as a mask), chunked over queries with
recomputation: the same numbers as the gathered form and no gather capacity to overflow.  Spans of different anchors
never overlap, so every token enters the softmax at most once.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..ops import ref


@dataclass(frozen=True)
class RopeCfg:
    K: int = 4                  # anchors opened per query
    links: int = 8              # keys that represent an anchor in the search
    win: int = 64               # local causal window
    span_cap: int = 256         # longest span read after an anchor
    excl_win: bool = True       # an anchor opens only once its span start has left the window
    rgrad: bool = True          # routing score as a bias on the span's keys
    rgrad_scale: float = 1.0
    chunk: int = 256            # queries per recomputed chunk


def anchors_from_surprise(s, tau, A, top=False):
    """s (B,T) with s[:,0] forced to be an anchor.  Returns own (B,T) = index of the anchor that owns each position,
    apos (B,A) anchor positions in order, avalid (B,A).  Over the cap: the first A in order, or with `top` the A most
    surprising."""
    B, T = s.shape
    anchor = s > tau
    anchor[:, 0] = True
    if top and A < T:
        ti = torch.where(anchor, s, torch.full_like(s, -float("inf"))).topk(A, -1).indices
        sel = torch.zeros_like(anchor).scatter(1, ti, True)
        keep = anchor & sel
    else:
        keep = anchor & (anchor.long().cumsum(1) <= A)
    own = keep.long().cumsum(1) - 1
    pos = torch.arange(T, device=s.device)
    order = ((~keep).long() * T + pos).argsort(dim=-1, stable=True)
    if A <= T:
        apos = order[:, :A]
        avalid = keep.gather(1, apos)
    else:
        apos = F.pad(order, (0, A - T))
        avalid = F.pad(keep.gather(1, order), (0, A - T))
    return own, apos, avalid


def next_anchor(apos, avalid, T):
    """Position of the next valid anchor, or T for the last / invalid ones."""
    nv = torch.cat([avalid[:, 1:], torch.zeros_like(avalid[:, :1])], 1)
    na = torch.cat([apos[:, 1:], apos[:, :1]], 1)
    return torch.where(nv, na, torch.full_like(apos, T))


@torch.no_grad()
def route_exact(q, k, own, apos, avalid, cfg: RopeCfg):
    """q, k (B,H,T,hd).  Returns tidx (B,H,T,K) anchor numbers, tval (valid), tpos (position of the best link)."""
    B, H, T, hd = q.shape
    A = apos.shape[1]
    kk, L = min(cfg.K, A), min(cfg.links, cfg.span_cap)
    lp = apos[:, :, None] + torch.arange(L, device=q.device)
    inb = lp < T
    lp = lp.clamp(max=T - 1)
    own_lp = own.gather(1, lp.reshape(B, A * L)).view(B, A, L)
    lval = inb & avalid[:, :, None] & (own_lp == torch.arange(A, device=q.device)[None, :, None])
    kl = k.gather(2, lp.reshape(B, 1, A * L, 1).expand(B, H, A * L, hd)).view(B, H, A, L, hd)
    nxt = next_anchor(apos, avalid, T)
    nx = torch.maximum(nxt, apos + cfg.win) if cfg.excl_win else nxt
    qi = torch.arange(T, device=q.device)
    tidx = torch.zeros(B, H, T, kk, dtype=torch.long, device=q.device)
    tval = torch.zeros(B, H, T, kk, dtype=torch.bool, device=q.device)
    tpos = torch.zeros(B, H, T, kk, dtype=torch.long, device=q.device)
    for c0 in range(0, T, cfg.chunk):
        qc = q[:, :, c0:c0 + cfg.chunk].float()
        s = torch.einsum("bhmd,bhald->bhmal", qc, kl.float()) / math.sqrt(hd)
        s = s.masked_fill(~lval[:, None, None], -float("inf"))
        s_a, best_l = s.max(-1)
        ok = avalid[:, None, :] & (nx[:, None, :] <= qi[None, c0:c0 + cfg.chunk, None])
        s_a = s_a.masked_fill(~ok[:, None], -float("inf"))
        top_v, top_i = s_a.topk(kk, -1)
        val = top_v > -float("inf")
        lpa = lp[:, None, None].expand(B, H, qc.shape[2], A, L).gather(-1, best_l[..., None]).squeeze(-1)
        tidx[:, :, c0:c0 + cfg.chunk] = torch.where(val, top_i, torch.zeros_like(top_i))
        tval[:, :, c0:c0 + cfg.chunk] = val
        tpos[:, :, c0:c0 + cfg.chunk] = torch.where(val, lpa.gather(-1, top_i), torch.zeros_like(top_i))
    return tidx, tval, tpos


def _read_chunk(qc, kr, v, k0, q0c, c0, st, en, tval, tpos, W, rgrad, rgrad_scale):
    B, H, C, hd = qc.shape
    T = kr.shape[2]
    sc = 1.0 / math.sqrt(hd)
    qi = c0 + torch.arange(C, device=qc.device)
    t = torch.arange(T, device=qc.device)
    in_k = (st[..., None] <= t) & (t < en[..., None]) & tval[..., None]           # (B,H,C,K,T)
    s = torch.einsum("bhcd,bhtd->bhct", qc.float(), kr.float()) * sc
    if rgrad:
        kb = k0.gather(2, tpos.reshape(B, H, -1, 1).expand(-1, -1, -1, hd)).view(B, H, C, -1, hd)
        rsel = torch.einsum("bhcd,bhckd->bhck", q0c.float(), kb.float()) * sc
        gb = torch.where(tval, rsel * rgrad_scale, torch.zeros_like(rsel))
        s_span = s + torch.einsum("bhck,bhckt->bhct", gb, in_k.float())
    else:
        s_span = s
    span = in_k.any(-2)
    dist = qi[:, None] - t[None, :]
    win = (dist >= 0) & (dist < W)
    s_all = torch.where(win[None, None], s, torch.where(span, s_span, torch.full_like(s, -float("inf"))))
    p = s_all.softmax(-1)
    out = torch.einsum("bhct,bhtd->bhcd", p, v.float()).to(v.dtype)
    share = (p * (span & ~win[None, None])).sum(-1).detach()
    return out, share


def rope_attention(qr, kr, v, own, apos, avalid, cfg: RopeCfg, routed=None):
    """qr, kr rotated queries / keys, v values, all (B,H,T,hd).  Returns (out (B,H,T,hd), share of softmax mass that
    went to opened spans, (tidx, tval, tpos))."""
    B, H, T, hd = qr.shape
    tidx, tval, tpos = route_exact(qr, kr, own, apos, avalid, cfg) if routed is None else routed
    nxt = next_anchor(apos, avalid, T)
    outs, shares = [], []
    qi_all = torch.arange(T, device=qr.device)
    for c0 in range(0, T, cfg.chunk):
        sl = slice(c0, c0 + cfg.chunk)
        ti = tidx[:, :, sl]
        st = apos.gather(1, ti.reshape(B, -1)).view_as(ti)
        nx = nxt.gather(1, ti.reshape(B, -1)).view_as(ti)
        en = torch.minimum(torch.minimum(nx, st + cfg.span_cap), (qi_all[sl] - cfg.win + 1)[None, None, :, None])
        args = (qr[:, :, sl], kr, v, kr.detach(), qr[:, :, sl].detach(), c0, st, en, tval[:, :, sl] & (en > st),
                tpos[:, :, sl], cfg.win, cfg.rgrad, cfg.rgrad_scale)
        if torch.is_grad_enabled() and qr.requires_grad:
            o, sh = checkpoint(_read_chunk, *args, use_reentrant=False)
        else:
            o, sh = _read_chunk(*args)
        outs.append(o)
        shares.append(sh)
    return torch.cat(outs, 2), torch.cat(shares, 2).mean(), (tidx, tval, tpos)


class RopeMemoryAttention(nn.Module):
    """Attention layer with the routed read: drop-in for a light block's attention at long context."""

    def __init__(self, d, heads, cfg: RopeCfg = RopeCfg()):
        super().__init__()
        self.heads, self.cfg = heads, cfg
        self.qkv = nn.Linear(d, 3 * d, bias=False)
        self.o = nn.Linear(d, d, bias=False)
        self.stats = {}

    def forward(self, x, surprise, tau, cap=0.25, routed=None):
        B, T, D = x.shape
        hd = D // self.heads
        q, k, v = self.qkv(x).view(B, T, 3, self.heads, hd).permute(2, 0, 3, 1, 4)
        cos, sin = ref.rope_angles(T, hd, x.device)
        q, k = ref.apply_rope(q, cos, sin, False), ref.apply_rope(k, cos, sin, False)
        with torch.no_grad():
            own, apos, avalid = anchors_from_surprise(surprise.clone(), tau, max(1, round(T * cap)))
        out, share, route = rope_attention(q, k, v, own, apos, avalid, self.cfg, routed)
        self.stats["rope_share"] = share
        return self.o(out.transpose(1, 2).reshape(B, T, D)), route
