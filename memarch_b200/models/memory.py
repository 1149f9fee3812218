"""Independent fixed-size memory of entity cards: a fresh bank (full-width contents) and a dim bank (compressed
contents, weaker at read time), written by novelty × importance and read per text segment.

Semantics follow the reference's `mem2.Memory` (mem2.py:51-238) and `mem3.VolumeMemory` (mem3.py:22-146); parameter
names are identical (`norm_w, face, content, importance, gate, down, up, norm_r, norm_c, query, value, out,
dim_weight, focus_gate`).  The code is organised differently: every write is split into a *plan* (discrete,
no-grad decisions: which words are bright, which card each updates or which place it takes, what is demoted,
promoted, pruned) and an *apply* (differentiable masked row writes done by scatter with averaging instead of
one-hot einsums).  The plan is what the GPU `mem_plan` kernel computes with the card state resident on chip.

State per text: fc (Fn,d) fresh contents, dc (Dmax,d/4) dim contents, faces (S,nf,df) chain of faces per card,
pos bookmark, valid, bright, uses, touched; S = Fn + Dmax.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


def scale_grad(x, s):
    """Same value, gradient × s: a card is read by many later segments and their grads must not avalanche."""
    if s == 1.0:
        return x
    return x * s + x.detach() * (1 - s)


def masked_put(t, idx, val, mask):
    """t[b, idx[b,w]] = val[b,w] where mask[b,w]; several writers of one place are averaged; switched-off writers
    touch nothing (so no gradient reaches them).  t (B,C,...), idx/mask (B,W), val (B,W,...)."""
    B, C = t.shape[:2]
    W = idx.shape[1]
    mf = mask.to(torch.float32)
    cnt = torch.zeros(B, C, device=t.device, dtype=torch.float32).scatter_add_(1, idx, mf)
    hit = cnt > 0
    tail = t.shape[2:]
    shp = (B, C) + (1,) * len(tail)
    if not t.is_floating_point():
        vf = val.to(torch.float32).reshape(B, W, -1) * mf[..., None]
        acc = torch.zeros(B, C, vf.shape[-1], device=t.device, dtype=torch.float32)
        acc = acc.scatter_add(1, idx[..., None].expand(-1, -1, vf.shape[-1]), vf)
        new = (acc / cnt.clamp(min=1)[..., None]).round().reshape(B, C, *tail).to(t.dtype)
        return torch.where(hit.view(shp), new, t)
    vf = val.to(t.dtype).reshape(B, W, -1) * mf[..., None].to(t.dtype)
    acc = torch.zeros(B, C, vf.shape[-1], device=t.device, dtype=t.dtype)
    acc = acc.scatter_add(1, idx[..., None].expand(-1, -1, vf.shape[-1]), vf)
    new = (acc / cnt.clamp(min=1)[..., None].to(t.dtype)).reshape(B, C, *tail)
    return t * (~hit).view(shp).to(t.dtype) + new


def _rows(t, idx):
    """t (B,C,...) rows at idx (B,W) -> (B,W,...)."""
    B = t.shape[0]
    ar = torch.arange(B, device=t.device)[:, None]
    return t[ar, idx]


def _count_before(mask):
    """Inclusive running count of True along the last axis (exact integer prefix sum)."""
    return mask.long().cumsum(-1)


class _ReadScores(torch.autograd.Function):
    """Fused card scores + softmax on the GPU (`csrc/memops.cu`): face normalisation, best link of the chain, dim
    penalty, empty-card mask and the softmax over cards in one kernel; backward in one kernel."""

    @staticmethod
    def forward(ctx, q, faces, valid, dim_pen, Fn, scale):
        from ..ops import _ext
        sc, w, best = _ext.C().mem_read_fwd(q.contiguous(), faces.contiguous(), valid.contiguous(),
                                            dim_pen.reshape(()).float(), int(Fn), float(scale))
        _ext.count()
        ctx.save_for_backward(q, faces, valid, w, best)
        ctx.meta = (int(Fn), float(scale))
        ctx.mark_non_differentiable(best)
        return sc, w

    @staticmethod
    def backward(ctx, dsc, dw):
        from ..ops import _ext
        q, faces, valid, w, best = ctx.saved_tensors
        Fn, scale = ctx.meta
        dq, dfa, dpen = _ext.C().mem_read_bwd(q.contiguous(), faces.contiguous(), valid.contiguous(), w, best,
                                              dw.contiguous().float() if dw is not None else torch.zeros_like(w),
                                              dsc.contiguous().float() if dsc is not None else None, Fn, scale)
        _ext.count()
        return dq, dfa, None, dpen.to(q.dtype), None, None


class CardMemory(nn.Module):
    META = ("faces", "pos", "valid", "bright", "uses", "touched")

    def __init__(self, d, fresh=64, dim=192, dim_max=256, faces=2, d_face=64, d_dim=None, write=32, focus=8,
                 match=0.8, w_use=2.0, w_age=1e-3, lean=True, **_):
        super().__init__()
        self.d, self.Fn, self.Dn, self.Dmax = d, fresh, dim, dim_max
        self.nf, self.df, self.W, self.K = faces, d_face, write, focus
        self.match, self.w_use, self.w_age, self.lean = match, w_use, w_age, lean
        dc = d_dim or d // 4
        self.norm_w = nn.RMSNorm(d)
        self.face = nn.Linear(d, d_face, bias=False)
        self.content = nn.Linear(d, d, bias=False)
        self.importance = nn.Linear(d, 1)
        self.gate = nn.Linear(2 * d, 1)
        self.down = nn.Linear(d, dc, bias=False)
        self.up = nn.Linear(dc, d, bias=False)
        self.norm_r = nn.RMSNorm(d)
        self.norm_c = nn.RMSNorm(d)
        self.query = nn.Linear(d, d_face, bias=False)
        self.value = nn.Linear(d, d, bias=False)
        self.out = nn.Linear(d, d, bias=False)
        self.dim_weight = nn.Parameter(torch.tensor(-0.5))
        self.focus_gate = nn.Linear(2 * d, 1)

    # -------------------------------------------------------------------------------------------- state
    def init_state(self, B, device, dtype=torch.float32):
        S = self.Fn + self.Dmax
        z = lambda *s, dt=torch.float32: torch.zeros(*s, device=device, dtype=dt)
        return dict(fc=z(B, self.Fn, self.d, dt=dtype), dc=z(B, self.Dmax, self.down.out_features, dt=dtype),
                    faces=z(B, S, self.nf, self.df, dt=dtype), pos=z(B, S, dt=torch.long),
                    valid=z(B, S, dt=torch.bool), bright=z(B, S), uses=z(B, S), touched=z(B, S))

    def contents(self, st):
        """Contents of every card at full width (dim cards expanded from their compressed form)."""
        return torch.cat([st["fc"], self.up(st["dc"])], 1)

    _contents = contents

    def score(self, st, now):
        sc = st["bright"] + self.w_use * st["uses"] - self.w_age * (now - st["touched"])
        return sc.masked_fill(~st["valid"], -1e9)

    # -------------------------------------------------------------------------------------------- read
    def card_scores(self, q, faces, valid):
        """Best cosine over a card's chain of faces, × sqrt(d_face); dim cards get the learned penalty."""
        fa = F.normalize(faces, dim=-1)
        sc = torch.einsum("bsf,bclf->bscl", q, fa).amax(-1) * math.sqrt(self.df)
        dimw = F.logsigmoid(self.dim_weight)
        sc = torch.cat([sc[..., :self.Fn], sc[..., self.Fn:] + dimw], -1)
        return sc.masked_fill(~valid[:, None], -1e4)

    def read(self, h, st, grad_scale=1.0):
        """h (B,S,d) words of the segment -> (addition to h, detached read weight of every card)."""
        n = self.norm_r(h)
        q = F.normalize(self.query(n), dim=-1)
        from ..ops import _ext
        if (_ext.use_cuda(q) and q.dtype == torch.float32 and st["faces"].dtype == torch.float32
                and self.df % 32 == 0 and self.df <= 128 and self.nf <= 255):
            sc, w = _ReadScores.apply(q, scale_grad(st["faces"], grad_scale), st["valid"],
                                      F.logsigmoid(self.dim_weight), self.Fn, math.sqrt(self.df))
        else:
            sc = self.card_scores(q, scale_grad(st["faces"], grad_scale), st["valid"])
            any_card = st["valid"].any(-1)[:, None, None]
            w = F.softmax(sc.float(), -1).type_as(h) * any_card
        vals = self.value(self.norm_c(scale_grad(self.contents(st), grad_scale)))
        mem = torch.einsum("bsc,bcd->bsd", w, vals)
        k = min(self.K, st["touched"].shape[1])
        fidx = st["touched"].masked_fill(~st["valid"], -1e9).topk(k, -1).indices
        fsc = sc.gather(-1, fidx[:, None].expand(-1, sc.shape[1], -1))
        fw = F.softmax(fsc.float(), -1).type_as(h) * st["valid"].gather(1, fidx).any(-1)[:, None, None]
        foc = torch.einsum("bsk,bkd->bsd", fw, _rows(vals, fidx))
        g = torch.sigmoid(self.focus_gate(torch.cat([n, foc], -1)))
        return self.out(g * foc + (1 - g) * mem), w.detach()

    # -------------------------------------------------------------------------------------------- write: shared steps
    def _words(self, h):
        """What a segment offers to the memory: (normed state, face, importance) of every word."""
        n = self.norm_w(h)
        return n, self.face(n), torch.sigmoid(self.importance(n))

    @staticmethod
    def _count_reads(st, w_read, now):
        """Cards this segment looked at: their use count grows, a card read with weight > 0.5 counts as touched now."""
        st = dict(st)
        if w_read is not None:
            used = w_read.float().sum(1).detach()
            st["uses"] = st["uses"] + used
            st["touched"] = torch.where(used > 0.5, torch.zeros_like(st["touched"]) + now, st["touched"])
        return st

    def _candidates(self, f, imp, st, W):
        """The W words worth writing: new (unlike every card's faces) and important.  For each of them the most
        similar card and whether it is similar enough to be an update.  -> (brightness of all words, cand, best, upd)"""
        fa = F.normalize(st["faces"], dim=-1)
        alike = lambda q: torch.einsum("bsf,bclf->bscl", F.normalize(q, dim=-1).type_as(fa), fa).amax(-1)
        known = alike(f).masked_fill(~st["valid"][:, None], -1).amax(-1)
        bright = (1 - known.clamp(min=0)) * imp.squeeze(-1).float()
        cand = bright.topk(W, -1).indices
        best_cos, best = alike(_rows(f, cand)).masked_fill(~st["valid"][:, None], -2).max(-1)
        return bright, cand, best, best_cos > self.match

    def _bank_order(self, st, now):
        """Strength of the cards in the fresh and in the dim bank (empty places weakest of all)."""
        strength, Fn, ok = self.score(st, now), self.Fn, st["valid"]
        empty = torch.full_like(strength, -2e9)
        return torch.where(ok, strength, empty)[:, :Fn], torch.where(ok, strength, empty)[:, Fn:]

    def _promotion(self, w_read, st, key_f, like):
        """A dim card that this segment read a lot (total weight > 1) trades places with the weakest fresh card."""
        B, Fn = like.shape[0], self.Fn
        if w_read is None:
            zero = torch.zeros(B, dtype=torch.long, device=like.device)
            return torch.zeros(B, dtype=torch.bool, device=like.device), zero, zero
        heat = w_read.float().sum(1)[:, Fn:].masked_fill(~st["valid"][:, Fn:], 0)
        hot_v, hot = heat.max(-1)
        return hot_v > 1.0, hot, key_f.argmin(-1)

    def _swap(self, fc, dc, meta, promote, hot, weak):
        """Exchange the hot dim card and the weak fresh card (contents through the compression, every meta field)."""
        pm, hf, wf = promote[:, None], hot[:, None], weak[:, None]
        up_c, down_c = self.up(_rows(dc, hf)), self.down(_rows(fc, wf))
        fc, dc = masked_put(fc, wf, up_c, pm), masked_put(dc, hf, down_c, pm)
        hfull = hf + self.Fn
        for k, t in meta.items():
            a, b = _rows(t, wf), _rows(t, hfull)
            meta[k] = masked_put(masked_put(t, wf, b, pm), hfull, a, pm)
        return fc, dc, meta

    def _dim_strength(self, meta, now):
        return (meta["bright"] + self.w_use * meta["uses"] - self.w_age * (now - meta["touched"]))[:, self.Fn:]

    # -------------------------------------------------------------------------------------------- write
    @torch.no_grad()
    def plan_write(self, f, imp, st, now, w_read):
        """Discrete decisions of one write (no gradients): returns a dict of index/mask tensors."""
        bright, cand, best, upd = self._candidates(f, imp, st, min(self.W, f.shape[1]))
        is_new = ~upd
        key_f, key_d = self._bank_order(st, now)
        # a new card takes the weakest fresh place; a card that sat there moves to the weakest dim place
        slot = key_f.argsort(dim=-1, stable=True).gather(1, (_count_before(is_new) - 1).clamp(min=0))
        demote = is_new & _rows(st["valid"], slot)
        dslot = key_d.argsort(dim=-1, stable=True).gather(1, (_count_before(demote) - 1).clamp(min=0))
        promote, hot, weak = self._promotion(w_read, st, key_f, f)
        return dict(bright=bright, cand=cand, best=best, upd=upd, is_new=is_new, slot=slot, demote=demote,
                    dslot=dslot, promote=promote, hot=hot, weak=weak)

    def write(self, h, positions, st, now, w_read=None):
        """h (B,S,d) word states in context; positions (B,S); w_read (B,S,C) how this segment read the cards."""
        Fn = self.Fn
        n, f, imp = self._words(h)
        c_all = None if self.lean else self.content(n) * imp
        st = self._count_reads(st, w_read, now)
        p = self.plan_write(f, imp, st, now, w_read)
        cand, best, upd, is_new, slot, demote, dslot = (p[k] for k in
                                                        ("cand", "best", "upd", "is_new", "slot", "demote", "dslot"))
        fw, pw, bw = _rows(f, cand), _rows(positions, cand), p["bright"].gather(1, cand)
        cw = self.content(_rows(n, cand)) * _rows(imp, cand) if self.lean else _rows(c_all, cand)
        old = _rows(self.contents(st), best)
        g = torch.sigmoid(self.gate(torch.cat([cw, old], -1)))
        new_val = old + g * (cw - old)

        fc, dc = st["fc"], st["dc"]
        meta = {k: st[k] for k in self.META}
        # 1) displaced fresh card -> dim bank (compressed)
        dfull = dslot + Fn
        dc = masked_put(dc, dslot, self.down(_rows(fc, slot)), demote)
        meta = {k: masked_put(t, dfull, _rows(t, slot), demote) for k, t in meta.items()}
        # 2) new cards in fresh places
        fc = masked_put(fc, slot, cw, is_new)
        chain0 = torch.cat([fw[:, :, None], torch.zeros_like(fw)[:, :, None].expand(-1, -1, self.nf - 1, -1)], 2)
        now_w = torch.zeros_like(bw) + now
        for k, v in (("faces", chain0), ("pos", pw), ("valid", torch.ones_like(is_new)), ("bright", bw),
                     ("uses", torch.zeros_like(bw)), ("touched", now_w)):
            meta[k] = masked_put(meta[k], slot, v, is_new)
        # 3) update of existing cards: content blended through the gate, new image heads the chain of faces
        is_f, is_d = upd & (best < Fn), upd & (best >= Fn)
        fc = masked_put(fc, best.clamp(max=Fn - 1), new_val, is_f)
        dc = masked_put(dc, (best - Fn).clamp(min=0), self.down(new_val), is_d)
        chain = torch.cat([fw[:, :, None], _rows(meta["faces"], best)[:, :, :-1]], 2)
        meta["faces"] = masked_put(meta["faces"], best, chain, upd)
        meta["pos"] = masked_put(meta["pos"], best, pw, upd)
        meta["bright"] = masked_put(meta["bright"], best, torch.maximum(bw, _rows(meta["bright"], best)), upd)
        meta["touched"] = masked_put(meta["touched"], best, now_w, upd)
        # 4) swap: hot dim card <-> weakest fresh card
        fc, dc, meta = self._swap(fc, dc, meta, p["promote"], p["hot"], p["weak"])
        # 5) prune the dim bank back to `dim` strongest once it reaches its ceiling
        with torch.no_grad():
            valid = meta["valid"]
            over = valid[:, Fn:].sum(1) > self.Dmax - self.W
            sc = self._dim_strength(meta, now).masked_fill(~valid[:, Fn:], -1e9)
            keep = sc.argsort(dim=-1, descending=True, stable=True).argsort(dim=-1, stable=True) < self.Dn
            meta["valid"] = torch.cat([valid[:, :Fn], torch.where(over[:, None], valid[:, Fn:] & keep, valid[:, Fn:])], 1)
        return dict(fc=fc, dc=dc, **meta)


class VolumeMemory(CardMemory):
    """Memory v3: capacity counted in pieces, a card is any number of pieces sharing a card id; a new fact about a
    known entity adds a piece to its card; pruning merges the weakest dim piece into another piece of the same
    card ("two facts -> gist") and drops it only when it has no mate (mem3.py:22-146)."""

    META = CardMemory.META + ("card",)

    def init_state(self, B, device, dtype=torch.float32):
        st = super().init_state(B, device, dtype)
        C = self.Fn + self.Dmax
        st["card"] = torch.full((B, C), -1, dtype=torch.long, device=device)
        st["next_id"] = torch.zeros(B, dtype=torch.long, device=device)
        return st

    def write(self, h, positions, st, now, w_read=None):
        B, S, d = h.shape
        Fn = self.Fn
        dev = h.device
        n, f, imp = self._words(h)
        c = self.content(n) * imp
        st = self._count_reads(st, w_read, now)
        with torch.no_grad():
            W = min(self.W, S, Fn)
            bright, cand, best, upd = self._candidates(f, imp, st, W)
            # a piece about a known card carries that card's id, anything else starts a new card
            cid = torch.where(upd, st["card"].gather(1, best), st["next_id"][:, None] + torch.arange(W, device=dev))
            key_f, key_d = self._bank_order(st, now)
            slot = key_f.argsort(dim=-1, stable=True)[:, :W]          # every written piece takes a fresh place
            demote = _rows(st["valid"], slot)
            dslot = key_d.argsort(dim=-1, stable=True).gather(1, (_count_before(demote) - 1).clamp(min=0))
            promote, hot, weak = self._promotion(w_read, st, key_f, f)
        fw, cw, pw, bw = _rows(f, cand), _rows(c, cand), _rows(positions, cand), bright.gather(1, cand)
        fc, dc = st["fc"], st["dc"]
        meta = {k: st[k] for k in self.META}
        yes = torch.ones_like(upd)
        dfull = dslot + Fn
        dc = masked_put(dc, dslot, self.down(_rows(fc, slot)), demote)
        meta = {k: masked_put(t, dfull, _rows(t, slot), demote) for k, t in meta.items()}
        # the new image becomes the first face on ALL pieces of the matched card
        old_face = _rows(meta["faces"], best)
        chain = torch.where(upd[..., None, None],
                            torch.cat([fw[:, :, None], old_face[:, :, :-1]], 2),
                            torch.cat([fw[:, :, None], torch.zeros_like(old_face[:, :, :-1])], 2))
        same = (meta["card"][:, None, :] == cid[:, :, None]) & upd[:, :, None] & meta["valid"][:, None, :]
        last = (same.long() * (torch.arange(W, device=dev) + 1)[None, :, None]).amax(1) - 1
        has = last >= 0
        pick = _rows(chain, last.clamp(min=0))
        meta["faces"] = torch.where(has[..., None, None], pick.type_as(meta["faces"]), meta["faces"])
        meta["touched"] = torch.where(has, torch.zeros_like(meta["touched"]) + now, meta["touched"])
        fc = masked_put(fc, slot, cw, yes)
        now_w = torch.zeros_like(bw) + now
        for k, v in (("faces", chain), ("pos", pw), ("valid", yes), ("bright", bw), ("uses", torch.zeros_like(bw)),
                     ("touched", now_w), ("card", cid)):
            meta[k] = masked_put(meta[k], slot, v, yes)
        next_id = st["next_id"] + W
        fc, dc, meta = self._swap(fc, dc, meta, promote, hot, weak)
        with torch.no_grad():
            valid = meta["valid"]
            vd = valid[:, Fn:]
            over = vd.sum(1) > self.Dmax - self.W
            sc = self._dim_strength(meta, now).masked_fill(~vd, 1e9)
            rank = sc.argsort(dim=-1, stable=True).argsort(dim=-1, stable=True)
            drop = over[:, None] & vd & (rank < (vd.sum(1, keepdim=True) - self.Dn))
            cd = meta["card"][:, Fn:]
            mate = (cd[:, :, None] == cd[:, None, :]) & vd[:, None, :] & ~drop[:, None, :]
            mate = mate & ~torch.eye(self.Dmax, dtype=torch.bool, device=dev)[None]
            to = mate.float().argmax(-1)
            merge = drop & mate.any(-1)
            self.last_merge = merge.float().sum(1).mean()
            self.last_drop = drop.float().sum(1).mean()
        mw = merge.to(dc.dtype)
        add = torch.zeros_like(dc).scatter_add(1, to[..., None].expand(-1, -1, dc.shape[-1]), dc * mw[..., None])
        cnt = torch.zeros(B, self.Dmax, device=dev, dtype=dc.dtype).scatter_add(1, to, mw)[..., None]
        dc = (dc + add) / (1 + cnt)
        meta["valid"] = torch.cat([valid[:, :Fn], valid[:, Fn:] & ~drop], 1)
        return dict(fc=fc, dc=dc, next_id=next_id, **meta)
