"""Anchor-routed long-range attention ("rope memory"; the reference's JAX port, rope.py:1-500).

Anchors are the surprising tokens.  Every anchor owns the span of text from itself to the next anchor (at most
`span_cap` tokens) and is found by its first `links` keys.  A query scores every earlier anchor by its best link,
opens its top-`K` anchors and attends with ONE softmax over its local window (`win` tokens, causal) and the tokens of
the opened spans that lie before the window.  The cost per token does not depend on the text length: window + K spans.

Routing runs under `no_grad`, either exact (every query against every anchor's links) or two-level (`route_hier`:
groups of anchors ranked per block of queries, exact scores among the anchors of the kept groups only); with `rgrad`
the routing score of an opened anchor is added as a bias to all keys of its span, which is how the choice receives a
gradient.
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
    route: str = "hier"         # "hier": two-level search over groups of anchors; "exact": every anchor
    G: int = 64                 # hier: anchors per group
    NB: int = 16                # hier: groups kept per block of queries
    BM: int = 64                # hier: queries per block
    excl_win: bool = True       # an anchor opens only once its span start has left the window
    rgrad: bool = True          # routing score as a bias on the span's keys
    rgrad_scale: float = 1.0
    chunk: int = 256            # queries per recomputed chunk
    route_bf16: bool = False    # exact search with bf16 operands (fp32 accumulate): on a GPU the scores are one tensor-core
                                # GEMM per chunk and the choice is the `rope_route_topk` kernel
    mgrad: bool = False         # the share of mass on opened spans keeps its gradient (a penalty may push it up)


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


def _links(k, own, apos, avalid, L):
    """The first L keys of every anchor's own span: kl (B,H,A,L,hd), lval (B,A,L) which of them exist, lp (B,A,L)
    their positions."""
    B, H, T, hd = k.shape
    A = apos.shape[1]
    lp = apos[:, :, None] + torch.arange(L, device=k.device)
    inb = lp < T
    lp = lp.clamp(max=T - 1)
    own_lp = own.gather(1, lp.reshape(B, A * L)).view(B, A, L)
    lval = inb & avalid[:, :, None] & (own_lp == torch.arange(A, device=k.device)[None, :, None])
    kl = k.gather(2, lp.reshape(B, 1, A * L, 1).expand(B, H, A * L, hd)).view(B, H, A, L, hd)
    return kl, lval, lp


def _open_from(apos, avalid, T, cfg):
    """First query position that may open each anchor: once its span is complete and (excl_win) has left the window."""
    nxt = next_anchor(apos, avalid, T)
    return torch.maximum(nxt, apos + cfg.win) if cfg.excl_win else nxt


def _best_of(qc, kl, lval, lp, ok, kk, hd):
    """Score queries qc (..., M, hd) against link keys kl (..., N, L, hd) of N anchors, keep each anchor's best link,
    mask by ok (..., M, N) and take the top kk.  lval / lp (..., N, L) broadcast over heads.
    Returns (slot in N, valid, position of the best link), each (..., M, kk)."""
    s = torch.einsum("...md,...nld->...mnl", qc.float(), kl.float()) / math.sqrt(hd)
    s = s.masked_fill(~lval[..., None, :, :], -float("inf"))
    s_a, best_l = s.max(-1)
    s_a = s_a.masked_fill(~ok, -float("inf"))
    top_v, top_i = s_a.topk(kk, -1)
    val = top_v > -float("inf")
    lpa = lp[..., None, :, :].expand(*s.shape).gather(-1, best_l[..., None]).squeeze(-1)
    zero = torch.zeros_like(top_i)
    return torch.where(val, top_i, zero), val, torch.where(val, lpa.gather(-1, top_i), zero)


@torch.no_grad()
def route_exact(q, k, own, apos, avalid, cfg: RopeCfg):
    """q, k (B,H,T,hd).  Returns tidx (B,H,T,K) anchor numbers, tval (valid), tpos (position of the best link)."""
    B, H, T, hd = q.shape
    A = apos.shape[1]
    kk, L = min(cfg.K, A), min(cfg.links, cfg.span_cap)
    kl, lval, lp = _links(k, own, apos, avalid, L)
    nx = _open_from(apos, avalid, T, cfg)
    if cfg.route_bf16:
        if q.is_cuda and kk <= 8 and (A * L) % 8 == 0 and hd % 8 == 0 and hd >= 16 and cfg.chunk % 8 == 0 and T % 8 == 0:
            return _route_exact_kernel(q, kl, lval, lp, avalid, nx, kk, cfg.chunk)
        q, kl = q.to(torch.bfloat16).float(), kl.to(torch.bfloat16).float()     # the same operands, PyTorch statement
    qi = torch.arange(T, device=q.device)
    out = []
    for c0 in range(0, T, cfg.chunk):
        ok = avalid[:, None, :] & (nx[:, None, :] <= qi[None, c0:c0 + cfg.chunk, None])
        out.append(_best_of(q[:, :, c0:c0 + cfg.chunk], kl, lval[:, None], lp[:, None], ok[:, None], kk, hd))
    return tuple(torch.cat(t, 2) for t in zip(*out))


def _route_exact_kernel(q, kl, lval, lp, avalid, nx, kk, chunk):
    """Scores of a chunk of queries against all link keys as ONE grouped tensor-core GEMM (a group per batch x head,
    bf16 operands, fp32 result), then `rope_route_topk` (csrc/rope_route.cu): best existing link per anchor the query
    may open, K best anchors, no (B,H,M,A,L) tensor of masked scores in between."""
    from ..ops import _ext, gemm
    B, H, T, hd = q.shape
    A, L = lval.shape[1], lval.shape[2]
    klb = kl.to(torch.bfloat16).reshape(B * H, A * L, hd).contiguous()
    lval8, av8 = lval.to(torch.uint8).contiguous(), avalid.to(torch.uint8).contiguous()
    lp32, nx32 = lp.to(torch.int32).contiguous(), nx.clamp(max=2 ** 31 - 1).to(torch.int32).contiguous()
    out = []
    for c0 in range(0, T, chunk):
        qc = q[:, :, c0:c0 + chunk].to(torch.bfloat16).reshape(B * H, -1, hd).contiguous()
        S = gemm(qc, klb, groups=B * H, out_dtype=torch.float32)
        ti, tv, tp = _ext.C().rope_route_topk(S, lval8, lp32, av8, nx32, H, kk, c0, 1.0 / math.sqrt(hd))
        _ext.count()
        M = qc.shape[1]
        out.append((ti.view(B, H, M, kk), tv.view(B, H, M, kk).bool(), tp.view(B, H, M, kk)))
    return tuple(torch.cat(t, 2) for t in zip(*out))


@torch.no_grad()
def route_hier(q, k, own, apos, avalid, cfg: RopeCfg):
    """Two-level search (rope.py:147-262 of the reference's JAX port): the cost per query does not grow with the
    number of anchors.

    Anchors are taken `G` at a time in order; a group is known by the mean of its link keys.  Queries are taken `BM`
    at a time; a block looks only at groups all of whose anchors were complete before the block began, ranks them by
    the mean query of the PREVIOUS block (every query of that block lies in the past of every query of this one, so
    nothing leaks backwards in time) and keeps the best `NB`.  The anchors after the last complete group, including
    the ones that appear while the block runs (at most one per query), are always candidates.  Each query is then
    scored exactly against the candidates only, with the same rule for which anchors may open as the exact search.
    When `NB` covers all complete groups the result is that of the exact search."""
    B, H, T, hd = q.shape
    A = apos.shape[1]
    dev = q.device
    kk, L = min(cfg.K, A), min(cfg.links, cfg.span_cap)
    G, BM = cfg.G, cfg.BM
    NG = -(-A // G)
    nb = min(cfg.NB, NG)
    kl, lval, lp = _links(k, own, apos, avalid, L)
    nxt = next_anchor(apos, avalid, T)
    nx = _open_from(apos, avalid, T, cfg)

    # level 1: one key per group of anchors, one query per block of queries
    pad = NG * G - A
    w = F.pad(lval, (0, 0, 0, pad)).view(B, 1, NG, G * L, 1).float()
    gkey = (F.pad(kl, (0, 0, 0, 0, 0, pad)).view(B, H, NG, G * L, hd).float() * w).sum(3) / w.sum(3).clamp(min=1.0)
    NMB = -(-T // BM)
    qp = F.pad(q, (0, 0, 0, NMB * BM - T)).view(B, H, NMB, BM, hd)
    m0 = torch.arange(NMB, device=dev) * BM
    last = (m0 + BM).clamp(max=T) - 1
    qmean = qp.float().sum(3) / (last - m0 + 1).float()[None, None, :, None]
    gsc = torch.einsum("bhnd,bhgd->bhng", qmean, gkey)
    gsc = torch.cat([torch.zeros_like(gsc[:, :, :1]), gsc[:, :, :-1]], 2)
    done = (avalid[:, None, :] & (nxt[:, None, :] <= m0[None, :, None])).sum(-1)             # (B,NMB)
    nfg = done // G
    g = torch.arange(NG, device=dev)
    gok = g < nfg[..., None]
    if cfg.excl_win:
        out_of_win = (avalid[:, None, :] & (apos[:, None, :] + cfg.win <= last[None, :, None])).sum(-1)
        gok = gok & (g * G < out_of_win[..., None])
    top_gv, top_gi = gsc.masked_fill(~gok[:, None], -float("inf")).topk(nb, -1)               # (B,H,NMB,nb)

    # candidates of a block: the anchors of its groups, then the tail after the last complete group
    ar = torch.arange(G, device=dev)
    grp = (top_gi[..., None] * G + ar).flatten(-2)
    grp_ok = ((top_gv > -float("inf"))[..., None] & ((top_gi[..., None] * G + ar) < A)).flatten(-2)
    tail = (nfg[:, None, :, None] * G + torch.arange(G + BM, device=dev)).expand(B, H, NMB, G + BM)
    cand = torch.cat([grp, tail], -1)
    cand_ok = torch.cat([grp_ok, tail < A], -1)
    cand = torch.where(cand_ok, cand, torch.zeros_like(cand))
    Cn = cand.shape[-1]

    # level 2: exact scores against the candidates, a few blocks at a time
    per = max(1, min(max(1, cfg.chunk // BM), (1 << 26) // max(1, B * H * Cn * L * hd)))
    out = []
    for b0 in range(0, NMB, per):
        ca, cv = cand[:, :, b0:b0 + per], cand_ok[:, :, b0:b0 + per]
        n = ca.shape[2]
        flat = ca.reshape(B, H, n * Cn)
        kl_c = kl.gather(2, flat[..., None, None].expand(B, H, n * Cn, L, hd)).view(B, H, n, Cn, L, hd)
        pick = lambda t: t[:, None].expand(B, H, *t.shape[1:]).gather(
            2, flat.view(B, H, n * Cn, *([1] * (t.dim() - 2))).expand(B, H, n * Cn, *t.shape[2:])
        ).view(B, H, n, Cn, *t.shape[2:])
        qi = (m0[b0:b0 + per, None] + torch.arange(BM, device=dev))                          # (n,BM)
        ok = cv[:, :, :, None, :] & pick(avalid)[:, :, :, None, :] & (pick(nx)[:, :, :, None, :] <= qi[None, None, :, :, None])
        slot, val, pos = _best_of(qp[:, :, b0:b0 + per], kl_c, pick(lval), pick(lp), ok, kk, hd)
        idx = ca[:, :, :, None, :].expand(B, H, n, BM, Cn).gather(-1, slot)
        out.append((torch.where(val, idx, torch.zeros_like(idx)), val, pos))
    return tuple(torch.cat(t, 2).view(B, H, NMB * BM, kk)[:, :, :T] for t in zip(*out))


def route(q, k, own, apos, avalid, cfg: RopeCfg):
    if cfg.route == "exact":
        return route_exact(q, k, own, apos, avalid, cfg)
    if cfg.route == "hier":
        return route_hier(q, k, own, apos, avalid, cfg)
    raise ValueError(f"unknown route mode {cfg.route!r}")


def mask_route(tidx, tval, apos, qmask=None, docs=None):
    """Queries outside `qmask` (B,T) open nothing and read their window only; with `docs` (B,T) document numbers an
    anchor of another document than the query's is not opened (rope.py:277-287)."""
    if qmask is not None:
        tval = tval & qmask[:, None, :, None]
    if docs is not None:
        B, H, T, K = tidx.shape
        da = docs.gather(1, apos).gather(1, tidx.reshape(B, -1)).view(B, H, T, K)
        tval = tval & (da == docs[:, None, :, None])
    return tval


def _read_chunk(qc, kr, v, k0, q0c, c0, st, en, tval, tpos, W, rgrad, rgrad_scale, mgrad=False):
    B, H, C, hd = qc.shape
    T = kr.shape[2]
    sc = 1.0 / math.sqrt(hd)
    qi = c0 + torch.arange(C, device=qc.device)
    t = torch.arange(T, device=qc.device)
    s = torch.einsum("bhcd,bhtd->bhct", qc.float(), kr.float()) * sc
    gb = None
    if rgrad:
        kb = k0.gather(2, tpos.reshape(B, H, -1, 1).expand(-1, -1, -1, hd)).view(B, H, C, -1, hd)
        rsel = torch.einsum("bhcd,bhckd->bhck", q0c.float(), kb.float()) * sc
        gb = torch.where(tval, rsel * rgrad_scale, torch.zeros_like(rsel))
    # one opened anchor at a time: the (query, anchor, key) table never exists, only (query, key) ones
    span = torch.zeros_like(s, dtype=torch.bool)
    s_span = s
    for j in range(st.shape[-1]):
        inside = (st[..., j, None] <= t) & (t < en[..., j, None]) & tval[..., j, None]
        span = span | inside
        if gb is not None:
            s_span = s_span + gb[..., j, None] * inside
    dist = qi[:, None] - t[None, :]
    win = (dist >= 0) & (dist < W)
    s_all = torch.where(win[None, None], s, torch.where(span, s_span, torch.full_like(s, -float("inf"))))
    p = s_all.softmax(-1)
    out = torch.einsum("bhct,bhtd->bhcd", p, v.float()).to(v.dtype)
    share = (p * (span & ~win[None, None])).sum(-1)
    return out, share if mgrad else share.detach()


def rope_attention(qr, kr, v, own, apos, avalid, cfg: RopeCfg, routed=None, qmask=None, docs=None, want_mass=False):
    """qr, kr rotated queries / keys, v values, all (B,H,T,hd).  Returns (out (B,H,T,hd), share of softmax mass that
    went to opened spans, (tidx, tval, tpos)).  `routed` reuses another layer's choice; `qmask` / `docs` as in
    `mask_route`.  `want_mass` adds a fourth result: that share per position (B,T), mean over heads."""
    B, H, T, hd = qr.shape
    tidx, tval, tpos = route(qr, kr, own, apos, avalid, cfg) if routed is None else routed
    tval = mask_route(tidx, tval, apos, qmask, docs)
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
                tpos[:, :, sl], cfg.win, cfg.rgrad, cfg.rgrad_scale, cfg.mgrad)
        if torch.is_grad_enabled() and qr.requires_grad:
            o, sh = checkpoint(_read_chunk, *args, use_reentrant=False)
        else:
            o, sh = _read_chunk(*args)
        outs.append(o)
        shares.append(sh)
    mass = torch.cat(shares, 2)
    if want_mass:
        return torch.cat(outs, 2), mass.mean().detach(), (tidx, tval, tpos), mass.mean(1)
    return torch.cat(outs, 2), mass.mean().detach(), (tidx, tval, tpos)


class RopeMemoryAttention(nn.Module):
    """Attention layer with the routed read: drop-in for a light block's attention at long context."""

    def __init__(self, d, heads, cfg: RopeCfg = RopeCfg()):
        super().__init__()
        self.heads, self.cfg = heads, cfg
        self.qkv = nn.Linear(d, 3 * d, bias=False)
        self.o = nn.Linear(d, d, bias=False)
        self.stats = {}

    def forward(self, x, surprise, tau, cap=0.25, routed=None, qmask=None, docs=None):
        B, T, D = x.shape
        hd = D // self.heads
        q, k, v = self.qkv(x).view(B, T, 3, self.heads, hd).permute(2, 0, 3, 1, 4)
        cos, sin = ref.rope_angles(T, hd, x.device)
        q, k = ref.apply_rope(q, cos, sin, False), ref.apply_rope(k, cos, sin, False)
        with torch.no_grad():
            own, apos, avalid = anchors_from_surprise(surprise.clone(), tau, max(1, round(T * cap)))
        out, share, route = rope_attention(q, k, v, own, apos, avalid, self.cfg, routed, qmask, docs)
        self.stats["rope_share"] = share
        return self.o(out.transpose(1, 2).reshape(B, T, D)), route
