"""Earlier generations of the model family, kept because the registry names are part of the public surface and the
long-context / ablation experiments compare against them (lm.py:63-807, full.py:185-352 of the reference):

  cards / tail        attention-free: short causal convolution per layer, optional bookmark cards
  img_sampled / full  transformer whose output goes through frozen word images (sampled or full softmax)
  plan<K> / planw<K> / planwc<K> / planwimg<K>
                      planner (once per K-token thought) + speaker (every token; own thought or a 2K window; cards)
  sketch<K>           planner emits a sketch (M vectors) and a word menu; the speaker picks from the menu
  surp<NN> / surpc / surpq / surpp / surpcx / surpimg, S300[pcq]_<NN>
                      thinking on surprises: heavy *attention* blocks on anchors only (threshold / cap / quota /
                      packed selection, situation cards, word-image output)
  F300 / F300ck / Fsmall / T300ck
                      full model v1: windowed light blocks, anchor-causal heavy blocks, bookmark re-reading of raw
                      text at anchors; the checkpointed transformer control

Parameter names match the reference, so its checkpoints load.  These models run on the library attention path
(boolean masks through SDPA): they are baselines and ablations, not the product model; the product's hot ops are in
`memarch.py`.
"""
from __future__ import annotations

import math
import os

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..ops import ref
from .blocks import LightBlock, TransformerLM, _cdt


# ------------------------------------------------------------------------------------------------ building blocks
class MaskedBlock(LightBlock):
    """Light block whose attention takes an explicit boolean mask (True = may look) and optional RoPE positions."""

    def forward(self, x, mask=None, pos=None):                  # noqa: D102 - signature differs from LightBlock on purpose
        B, T, D = x.shape
        hd = D // self.heads
        n1 = ops.rmsnorm(x, self.n1.weight, self.n1.eps, out_dtype=_cdt(x))
        q, k, v = ops.linear(n1, self.qkv.weight).view(B, T, 3, self.heads, hd).permute(2, 0, 3, 1, 4)
        cos, sin = ref.rope_angles(T, hd, x.device, pos=pos)
        q, k = ref.apply_rope(q, cos, sin, self.rope_half), ref.apply_rope(k, cos, sin, self.rope_half)
        if mask is None:
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        else:
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        x = x + ops.linear(a.transpose(1, 2).reshape(B, T, D), self.o.weight).to(x.dtype)
        n2 = ops.rmsnorm(x, self.n2.weight, self.n2.eps, out_dtype=_cdt(x))
        return x + ops.linear(self._act(ops.linear(n2, self.up.weight)), self.down.weight).to(x.dtype)


class FFN(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.norm = nn.RMSNorm(d)
        self.up = nn.Linear(d, 8 * d, bias=False)
        self.down = nn.Linear(4 * d, d, bias=False)

    def forward(self, x):
        n = ops.rmsnorm(x, self.norm.weight, self.norm.eps, out_dtype=_cdt(x))
        return x + ops.linear(ops.swiglu(ops.linear(n, self.up.weight)), self.down.weight).to(x.dtype)


class Tail(nn.Module):
    """Sees only the last `width` tokens: depthwise causal convolution, gated."""

    def __init__(self, d, width=4):
        super().__init__()
        self.width = width
        self.norm = nn.RMSNorm(d)
        self.conv = nn.Conv1d(d, d, width, groups=d)
        self.gate = nn.Linear(d, d, bias=False)
        self.out = nn.Linear(d, d, bias=False)

    def forward(self, x):
        n = self.norm(x)
        c = self.conv(F.pad(n.transpose(1, 2), (self.width - 1, 0))).transpose(1, 2)
        return x + self.out(c * F.silu(self.gate(n)))


def bookmark_read(reader, x, n, book, mark, w, qpos):
    """Shared tail of both card readers: from every chosen bookmark read up to R raw tokens of `book` with
    ACT-style halting; returns (x + projected reading, expected tokens read)."""
    B, Tq, K = mark.shape
    T, Db, R = book.shape[1], book.shape[-1], reader.max_read
    rpos = mark[..., None] + torch.arange(R, device=x.device)
    readable = rpos <= qpos[None, :, None, None]
    rpos = rpos.clamp(max=T - 1)
    v = book.gather(1, rpos.reshape(B, -1, 1).expand(-1, -1, Db)).view(B, Tq, K, R, Db) + reader.offset
    halt = torch.sigmoid(reader.halt_v(v).squeeze(-1) + reader.halt_h(n)[:, :, None])
    halt = torch.where(readable, halt, torch.ones_like(halt))
    halt = torch.cat([halt[..., :-1], torch.ones_like(halt[..., -1:])], -1)
    survive = torch.cumprod(torch.cat([torch.ones_like(halt[..., :1]), 1 - halt[..., :-1]], -1), -1)
    read = ((survive * halt * readable)[..., None] * v).sum(-2)
    got = (w[..., None] * read).sum(-2)
    cost = (w * (survive * readable).sum(-1)).sum(-1).mean()
    return x + reader.out(got), cost


class _ReaderBase(nn.Module):
    def __init__(self, d, d_book, top_k, max_read, d_face):
        super().__init__()
        self.top_k, self.max_read, self.d_face = top_k, max_read, d_face
        self.norm = nn.RMSNorm(d)
        self.face = nn.Linear(d, d_face, bias=False)
        self.query = nn.Linear(d, d_face, bias=False)
        self.offset = nn.Parameter(torch.randn(max_read, d_book) * 0.02)
        self.halt_v = nn.Linear(d_book, 1)
        self.halt_h = nn.Linear(d, 1, bias=False)
        self.out = nn.Linear(d_book, d, bias=False)


class CardRead(_ReaderBase):
    """Every earlier token is a card: find by face, re-read raw text at its bookmark (lm.py:80-125)."""

    def __init__(self, d, d_book, top_k=4, max_read=4, d_face=64):
        super().__init__(d, d_book, top_k, max_read, d_face)

    def forward(self, x, book):
        x, book = x.float(), book.float()
        B, T, _ = x.shape
        n = self.norm(x)
        scores = self.query(n) @ self.face(n).transpose(1, 2) / math.sqrt(self.d_face)
        pos = torch.arange(T, device=x.device)
        scores = scores.masked_fill(pos[None, :] >= pos[:, None], -1e4)
        top_s, top_i = scores.topk(min(self.top_k, T), -1)
        w = F.softmax(top_s.float(), -1).type_as(x) * (top_s > -1e3)
        return bookmark_read(self, x, n, book, top_i, w, pos)


class AnchorCardRead(_ReaderBase):
    """Cards are the anchors after the heavy layers; computed in chunks of `chunk` words with recomputation so
    the word x card table never lives whole (full.py:185-239)."""

    def __init__(self, d, d_book=128, top_k=4, max_read=4, d_face=64, chunk=4096):
        super().__init__(d, d_book, top_k, max_read, d_face)
        self.chunk = chunk

    def forward(self, x, book, cards, idx, valid):
        outs, costs = [], []
        for s in range(0, x.shape[1], self.chunk):
            a = (x[:, s:s + self.chunk].float(), s, book.float(), cards.float(), idx, valid)
            o, c = checkpoint(self._part, *a, use_reentrant=False) if self.training else self._part(*a)
            outs.append(o)
            costs.append(c)
        return torch.cat(outs, 1), torch.stack(costs).mean()

    def _part(self, x, start, book, cards, idx, valid):
        B, Tq, _ = x.shape
        n = self.norm(x)
        faces = self.face(self.norm(cards))
        scores = self.query(n) @ faces.transpose(1, 2) / math.sqrt(self.d_face)
        qpos = torch.arange(start, start + Tq, device=x.device)
        ok = valid[:, None, :] & (idx[:, None, :] < qpos[None, :, None])
        scores = scores.masked_fill(~ok, -1e4)
        k = min(self.top_k, scores.shape[-1])
        top_s, top_j = scores.topk(k, -1)
        w = F.softmax(top_s, -1) * (top_s > -1e3)
        mark = idx.gather(1, top_j.reshape(B, -1)).view(B, Tq, k)
        return bookmark_read(self, x, n, book, mark, w, qpos)


class CardsLM(nn.Module):
    def __init__(self, vocab, d=512, layers=8, d_book=128, card_layers=(3, 6), use_cards=True):
        super().__init__()
        self.emb = nn.Embedding(vocab, d)
        self.book = nn.Embedding(vocab, d_book)
        self.tails = nn.ModuleList(Tail(d) for _ in range(layers))
        self.ffns = nn.ModuleList(FFN(d) for _ in range(layers))
        self.cards = nn.ModuleDict({str(i): CardRead(d, d_book) for i in card_layers} if use_cards else {})
        self.norm = nn.RMSNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)

    def forward(self, x, prep=None):
        h = self.emb(x)
        book = self.book(x) if len(self.cards) else None
        cost = torch.zeros((), device=x.device)
        for i, (tail, ffn) in enumerate(zip(self.tails, self.ffns)):
            h = tail(h)
            if str(i) in self.cards:
                h, c = self.cards[str(i)](h, book)
                cost = cost + c
            h = ffn(h)
        return self.head(self.norm(h)), cost

    def train_loss(self, out, y, train=True):
        return F.cross_entropy(out.float().view(-1, out.shape[-1]), y.reshape(-1))


# ------------------------------------------------------------------------------------------------ word images
def load_word_images(vocab, width=768):
    """Frozen word images.  The reference takes GPT-2's embedding table from the hub (lm.py:166-176); offline the
    table comes from `WORD_IMAGES` (a .pt / .npy of shape (n, width)) or, failing that, a seeded random table."""
    path = os.environ.get("WORD_IMAGES")
    if path and os.path.exists(path):
        import numpy as np
        t = torch.load(path) if path.endswith(".pt") else torch.from_numpy(np.load(path))
        out = torch.zeros(vocab, t.shape[1])
        out[:min(vocab, len(t))] = t[:vocab].float()
        return out
    g = torch.Generator().manual_seed(768)
    return torch.randn(vocab, width, generator=g) * 0.1


class ImageOut(nn.Module):
    """Output through fixed word images: the model emits "what I want to say", compared with the images; sampled
    training uses the right word + `n_neg` frequency-corrected negatives, evaluation always the full vocabulary."""

    def __init__(self, d, vocab, sampled, n_neg=1024, n_real=50257):
        super().__init__()
        self.sampled, self.n_neg, self.n_real = sampled, n_neg, min(n_real, vocab)
        img = load_word_images(vocab)
        self.register_buffer("img", img / img.norm(dim=-1, keepdim=True).mean())
        self.proj = nn.Linear(d, img.shape[1], bias=False)
        self.register_buffer("log_q", torch.full((vocab,), -math.log(self.n_real)))

    def set_unigram(self, counts):
        q = (counts.float() + 1) / (counts.float() + 1)[:self.n_real].sum()
        q[self.n_real:] = 1e-12
        self.log_q.copy_(q.log())

    def logits(self, h):
        lo = self.proj(h) @ self.img.T.type_as(h)
        lo[..., self.n_real:] = -1e4
        return lo

    def loss(self, h, y, train):
        if not (train and self.sampled):
            return F.cross_entropy(self.logits(h).float().view(-1, self.img.shape[0]), y.reshape(-1))
        z = self.proj(h).reshape(-1, self.img.shape[1])
        y = y.reshape(-1)
        neg = torch.multinomial(self.log_q.exp(), self.n_neg, replacement=True)
        pos_lo = (z * self.img[y].type_as(z)).sum(-1, keepdim=True) - self.log_q[y, None]
        neg_lo = z @ self.img[neg].T.type_as(z) - self.log_q[neg][None]
        neg_lo = neg_lo.masked_fill(neg[None] == y[:, None], -1e4)
        lo = torch.cat([pos_lo, neg_lo], -1).float()
        return F.cross_entropy(lo, torch.zeros(len(y), dtype=torch.long, device=y.device))


class PlainTransformerLM(nn.Module):
    """Transformer returning logits (the shape the prototypes share); `blocks` as in the reference."""

    def __init__(self, vocab, d=512, layers=8, heads=8, ckpt=False):
        super().__init__()
        self.ckpt = ckpt
        self.emb = nn.Embedding(vocab, d)
        self.blocks = nn.ModuleList(MaskedBlock(d, heads) for _ in range(layers))
        self.norm = nn.RMSNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)

    def hidden(self, x):
        h = self.emb(x)
        for b in self.blocks:
            h = checkpoint(b, h, use_reentrant=False) if self.ckpt and self.training else b(h)
        return self.norm(h)

    def forward(self, x, prep=None):
        return self.head(self.hidden(x)), torch.zeros((), device=x.device)

    def train_loss(self, out, y, train=True):
        return F.cross_entropy(out.float().view(-1, out.shape[-1]), y.reshape(-1))


class ImageTransformerLM(PlainTransformerLM):
    def __init__(self, vocab, sampled):
        super().__init__(vocab)
        del self.head
        self.out = ImageOut(self.norm.normalized_shape[0], vocab, sampled)

    def forward(self, x, prep=None):
        return self.hidden(x), torch.zeros((), device=x.device)

    def train_loss(self, h, y, train=True):
        return self.out.loss(h, y, train)


# ------------------------------------------------------------------------------------------------ planner / speaker
def _window_mask(T, window, device):
    pos = torch.arange(T, device=device)
    dist = pos[:, None] - pos[None, :]
    return (dist >= 0) & (dist < window)


class _ThoughtPool(nn.Module):
    """Shared front: embed, add in-thought position, squeeze every K-token thought to one vector (4-query pooling),
    run the planner over thoughts (thought j sees thoughts < j after the shift)."""

    def _init_front(self, vocab, k, d, p_layers, heads):
        self.k = k
        self.emb = nn.Embedding(vocab, d)
        self.pos = nn.Parameter(torch.randn(k, d) * 0.02)
        self.pool_q = nn.Parameter(torch.randn(4, d) * 0.02)
        self.pool_out = nn.Linear(4 * d, d, bias=False)
        self.start = nn.Parameter(torch.randn(d) * 0.02)
        self.planner = nn.ModuleList(MaskedBlock(d, heads) for _ in range(p_layers))
        self.p_norm = nn.RMSNorm(d)

    def _plan(self, x):
        B, T = x.shape
        k, n = self.k, T // self.k
        e = self.emb(x).view(B, n, k, -1) + self.pos
        att = torch.einsum("bnkd,qd->bnqk", e, self.pool_q).softmax(-1)
        p = self.pool_out(torch.einsum("bnqk,bnkd->bnqd", att, e).flatten(2))
        for b in self.planner:
            p = b(p)
        return e, self.p_norm(p)

    def _shift(self, p):
        return torch.cat([self.start.expand(p.shape[0], 1, -1).type_as(p), p[:, :-1]], 1)


class PlannerSpeakerLM(_ThoughtPool):
    def __init__(self, vocab, k, d=512, p_layers=8, s_layers=3, heads=8, window=0, cards=False):
        super().__init__()
        self.window = window
        self._init_front(vocab, k, d, p_layers, heads)
        self.intent = nn.Linear(d, d, bias=False)
        self.book = nn.Embedding(vocab, 128) if cards else None
        self.cards = CardRead(d, 128) if cards else None
        self.speaker = nn.ModuleList(MaskedBlock(d, heads) for _ in range(s_layers))
        self.norm = nn.RMSNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)

    def forward(self, x, prep=None):
        B, T = x.shape
        k, n = self.k, T // self.k
        e, p = self._plan(x)
        plan = self._shift(self.intent(p))
        h = e + plan[:, :, None]
        cost = torch.zeros((), device=x.device)
        if self.window:
            h = h.reshape(B, T, -1)
            mask = _window_mask(T, self.window, x.device)
            for i, b in enumerate(self.speaker):
                h = b(h, mask)
                if i == 0 and self.cards is not None:
                    h, cost = self.cards(h, self.book(x))
            return self.head(self.norm(h)), cost
        h = h.reshape(B * n, k, -1)
        for b in self.speaker:
            h = b(h)
        return self.head(self.norm(h.view(B, T, -1))), cost

    def train_loss(self, out, y, train=True):
        return F.cross_entropy(out.float().view(-1, out.shape[-1]), y.reshape(-1))


class ImagePlannerLM(nn.Module):
    def __init__(self, vocab, k):
        super().__init__()
        self.core = PlannerSpeakerLM(vocab, k=k, window=2 * k)
        del self.core.head
        self.core.head = nn.Identity()
        self.out = ImageOut(512, vocab, sampled=True)

    def forward(self, x, prep=None):
        return self.core(x)

    def train_loss(self, h, y, train=True):
        return self.out.loss(h, y, train)


class SketchLM(_ThoughtPool):
    def __init__(self, vocab, k=32, d=512, p_layers=8, s_layers=3, heads=8, M=8, menu=256):
        super().__init__()
        self.M, self.n_menu, self.window = M, min(menu, vocab), 2 * k
        self._init_front(vocab, k, d, p_layers, heads)
        self.sketch = nn.Linear(d, M * d, bias=False)
        self.menu_head = nn.Linear(d, vocab, bias=False)
        self.speaker = nn.ModuleList(MaskedBlock(d, heads) for _ in range(s_layers))
        self.c_norm = nn.ModuleList(nn.RMSNorm(d) for _ in range(s_layers))
        self.c_q = nn.ModuleList(nn.Linear(d, d, bias=False) for _ in range(s_layers))
        self.c_out = nn.ModuleList(nn.Linear(d, d, bias=False) for _ in range(s_layers))
        self.norm = nn.RMSNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)
        self.other = nn.Linear(d, 1)
        self.stats = {}

    def forward(self, x, prep=None):
        B, T = x.shape
        k, n, M = self.k, T // self.k, self.M
        e, p = self._plan(x)
        p = self._shift(p)
        sk = self.sketch(p).view(B, n, M, -1)
        menu_logits = self.menu_head(p)
        menu_idx = menu_logits.detach().float().topk(self.n_menu, -1).indices
        h = (e + sk.mean(2)[:, :, None]).reshape(B, T, -1)
        mask = _window_mask(T, self.window, x.device)
        scale = 1 / math.sqrt(h.shape[-1])
        for blk, cn, cq, co in zip(self.speaker, self.c_norm, self.c_q, self.c_out):
            h = blk(h, mask)
            q = cq(cn(h)).view(B, n, k, -1)
            a = (torch.einsum("bnkd,bnmd->bnkm", q, sk) * scale).softmax(-1)
            h = h + co(torch.einsum("bnkm,bnmd->bnkd", a, sk).reshape(B, T, -1))
        return (self.norm(h), menu_idx, menu_logits), torch.zeros((), device=x.device)

    def train_loss(self, out, y, train=True):
        hn, menu_idx, menu_logits = out
        B, T, d = hn.shape
        k, n = self.k, T // self.k
        yb, hb = y.reshape(B, n, k), hn.view(B, n, k, d)
        menu_loss = -F.log_softmax(menu_logits.float(), -1).gather(-1, yb).mean()
        hit = menu_idx[:, :, None, :] == yb[..., None]
        inmenu, slot = hit.any(-1), hit.float().argmax(-1)
        Wm = self.head.weight[menu_idx]
        lo = torch.cat([torch.einsum("bnkd,bnmd->bnkm", hb, Wm.type_as(hb)), self.other(hb)], -1).float()
        tgt = torch.where(inmenu, slot, torch.full_like(slot, self.n_menu))
        logp_menu = F.log_softmax(lo, -1)
        miss = ~inmenu
        self.stats["miss"] = miss.float().mean()
        nm = int(miss.sum())
        tok_menu = menu_idx[:, :, None, :].expand(B, n, k, self.n_menu)
        full = None
        if nm:                                                   # full vocabulary only for words outside the menu
            full = (hb[miss] @ self.head.weight.T.type_as(hb)).float().scatter(1, tok_menu[miss], -1e4)
        if train:
            loss = F.nll_loss(logp_menu.view(-1, self.n_menu + 1), tgt.view(-1))
            if nm:
                loss = loss + F.cross_entropy(full, yb[miss], reduction="sum") / y.numel()
            return loss + 0.5 * menu_loss
        lp = logp_menu.gather(-1, tgt[..., None]).squeeze(-1)
        if nm:
            lp = lp.clone()
            lp[miss] = lp[miss] + F.log_softmax(full, -1).gather(-1, yb[miss][:, None]).squeeze(-1)
        return -lp.mean()


# ------------------------------------------------------------------------------------------------ surprise models
def _light_surprise(l_head, lh, x, rows=None):
    """-log p(x_t) under the light head, in row groups so that B x T x V never lives whole."""
    B, T = x.shape
    s = torch.full((B, T), 1e4, device=x.device)
    step = rows or max(1, B // 4)
    for i in range(0, B, step):
        for j in range(0, T - 1, 8192):
            lo = l_head(lh[i:i + step, j:min(j + 8192, T - 1)])
            tgt = x[i:i + step, j + 1:j + 1 + lo.shape[1], None]
            s[i:i + lo.shape[0], j + 1:j + 1 + lo.shape[1]] = (torch.logsumexp(lo, -1) - lo.gather(-1, tgt).squeeze(-1)).float()
    return s


def _first_anchors(anchor, C):
    """The first C anchors of every text in order: (idx (B,C), valid (B,C))."""
    T = anchor.shape[1]
    keep = anchor & (anchor.cumsum(1) <= C)
    pos = torch.arange(T, device=anchor.device)
    idx = ((~keep).long() * T + pos).argsort(dim=-1, stable=True)[:, :C]
    return idx, keep.gather(1, idx)


def _anchor_mask(valid):
    A = valid.shape[1]
    causal = torch.ones(A, A, dtype=torch.bool, device=valid.device).tril()
    return ((causal[None] & valid[:, None, :]) | torch.eye(A, dtype=torch.bool, device=valid.device)[None])[:, None]


class SurpriseLM(nn.Module):
    def __init__(self, vocab, d=512, light=2, heavy=8, final=1, heads=8, frac=0.2, images=False, packed=False,
                 select="threshold", chunk=128, cap=0.25, sit_cards=0):
        super().__init__()
        self.sit_cards = sit_cards
        if sit_cards:
            self.sit_keys = nn.Parameter(torch.randn(sit_cards, d) * 0.02)
            self.sit_gain = nn.Parameter(torch.zeros(sit_cards, d))
        self.frac, self.packed, self.select, self.chunk, self.cap = frac, packed, select, chunk, cap
        self.emb = nn.Embedding(vocab, d)
        self.light = nn.ModuleList(MaskedBlock(d, heads) for _ in range(light))
        self.l_norm = nn.RMSNorm(d)
        self.l_head = nn.Sequential(nn.Linear(d, 128, bias=False), nn.Linear(128, vocab, bias=False))
        self.heavy = nn.ModuleList(MaskedBlock(d, heads) for _ in range(heavy))
        self.final = nn.ModuleList(MaskedBlock(d, heads) for _ in range(final))
        self.norm = nn.RMSNorm(d)
        self.out = ImageOut(d, vocab, sampled=False) if images else None
        self.head = None if images else nn.Linear(d, vocab, bias=False)
        self.register_buffer("tau", torch.tensor(5.0))
        self.stats = {}

    def forward(self, x, prep=None):
        B, T = x.shape
        h = self.emb(x)
        if self.sit_cards:                     # situation at word t = mean of what was read up to t (no look-ahead)
            tri = torch.ones(T, T, device=x.device).tril_()
            sit = (tri / tri.sum(1, keepdim=True)).type_as(h) @ h.detach()
            p = (F.normalize(sit, dim=-1) @ F.normalize(self.sit_keys, dim=-1).T * 8).softmax(-1)
            h = h * (1 + (p @ self.sit_gain).type_as(h))
        for b in self.light:
            h = b(h)
        lh = self.l_norm(h)
        with torch.no_grad():
            s = _light_surprise(self.l_head, lh.detach(), x)
            anchor = s > self.tau                                # chosen with the old threshold
            if self.training:
                self.tau.mul_(0.9).add_(0.1 * ref.tau_quantile(s, self.frac))
            self.stats["anchors"] = anchor.float().mean()
        if self.select != "threshold":
            h = self._heavy_static(h, s, anchor)
        elif self.packed:
            h = self._heavy_packed(h, anchor)
        else:
            h = self._heavy_padded(h, anchor)
        for b in self.final:
            h = b(h)
        hn = self.norm(h)
        logits = self.out.logits(hn) if self.out is not None else self.head(hn)
        return (logits, lh), torch.zeros((), device=x.device)

    def _think(self, h, idx, valid):
        d = h.shape[-1]
        a_in = h.gather(1, idx[..., None].expand(-1, -1, d))
        a, mask = a_in, _anchor_mask(valid)
        for b in self.heavy:
            a = b(a, mask)
        return h.scatter_add(1, idx[..., None].expand(-1, -1, d), (a - a_in) * valid[..., None])

    def _heavy_static(self, h, s, anchor):
        B, T, _ = h.shape
        with torch.no_grad():
            if self.select == "quota" and self.training:
                k = max(1, round(self.chunk * self.frac))
                top = s.view(B, T // self.chunk, self.chunk).topk(k, -1).indices.sort(-1).values
                idx = (top + torch.arange(0, T, self.chunk, device=h.device)[None, :, None]).view(B, -1)
                valid = torch.ones_like(idx, dtype=torch.bool)
            else:
                idx, valid = _first_anchors(anchor, max(1, round(T * self.cap)))
            self.stats["anchors"] = valid.float().mean() * idx.shape[1] / T
        return self._think(h, idx, valid)

    def _heavy_padded(self, h, anchor):
        with torch.no_grad():
            A = max(1, int(anchor.sum(1).max()))                 # variable width: one host read per step
            idx, valid = _first_anchors(anchor, A)
        return self._think(h, idx, valid)

    def _heavy_packed(self, h, anchor):
        """All anchors of the batch in one dense sequence; mask = same text and not later; RoPE by the anchor's
        number in its own text.  Length is rounded up to a multiple of 512 so that few shapes occur."""
        B, T, d = h.shape
        with torch.no_grad():
            flat = anchor.reshape(-1).nonzero().squeeze(1)
            N = flat.numel()
            Np = max(512, -(-N // 512) * 512)
            seq = flat // T
            counts = anchor.sum(1)
            pos = torch.arange(N, device=h.device) - (counts.cumsum(0) - counts)[seq]
            pad = Np - N
            seq_p = torch.cat([seq, -1 - torch.arange(pad, device=h.device)])
            pos_p = torch.cat([pos, torch.zeros(pad, dtype=torch.long, device=h.device)])
            idx_p = torch.cat([flat, torch.zeros(pad, dtype=torch.long, device=h.device)])
            q = torch.arange(Np, device=h.device)
            mask = (seq_p[:, None] == seq_p[None, :]) & (q[None, :] <= q[:, None])
        flat_h = h.reshape(B * T, d)
        a_in = flat_h[idx_p][None]
        a = a_in
        for blk in self.heavy:
            a = blk(a, mask[None, None], pos_p)
        return flat_h.index_add(0, flat, (a - a_in)[0, :N]).view(B, T, d)

    def train_loss(self, out, y, train=True):
        logits, lh = out
        V = logits.shape[-1]
        loss = F.cross_entropy(logits.float().view(-1, V), y.reshape(-1))
        if train:               # the light part learns to predict, or surprise means nothing (every 4th position)
            l_logits = self.l_head(lh[:, ::4])
            loss = loss + 0.3 * F.cross_entropy(l_logits.float().reshape(-1, V), y[:, ::4].reshape(-1))
        return loss


class FullLM(nn.Module):
    """Full model v1: windowed light blocks, heavy *attention* blocks over the text's earlier anchors, windowed final
    blocks, bookmark re-reading with the anchors as cards (full.py:242-330)."""

    def __init__(self, vocab, d=1024, light=4, heavy=14, final=2, heads=16, frac=0.2, cap=0.25, window=2048, ckpt=False):
        super().__init__()
        self.frac, self.cap, self.window, self.ckpt = frac, cap, window, ckpt
        self.emb = nn.Embedding(vocab, d)
        self.book = nn.Embedding(vocab, 128)
        self.light = nn.ModuleList(LightBlock(d, heads) for _ in range(light))
        self.l_norm = nn.RMSNorm(d)
        self.l_head = nn.Sequential(nn.Linear(d, 128, bias=False), nn.Linear(128, vocab, bias=False))
        self.heavy = nn.ModuleList(MaskedBlock(d, heads) for _ in range(heavy))
        self.final = nn.ModuleList(LightBlock(d, heads) for _ in range(final))
        self.cards = AnchorCardRead(d)
        self.norm = nn.RMSNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)
        self.register_buffer("tau", torch.tensor(5.0))
        self.stats = {}

    def _run(self, blk, *a):
        return checkpoint(blk, *a, use_reentrant=False) if self.ckpt and self.training else blk(*a)

    def forward(self, x, prep=None):
        B, T = x.shape
        A = max(1, round(T * self.cap))
        win = self.window if T > self.window else None
        h = self.emb(x)
        for b in self.light:
            h = self._run(b, h, win)
        lh = self.l_norm(h)
        with torch.no_grad():
            s = _light_surprise(self.l_head, lh.detach(), x, rows=max(1, min(B, 32768 // T)))
            anchor = s > self.tau
            if self.training:
                self.tau.mul_(0.9).add_(0.1 * ref.tau_quantile(s, self.frac))
            idx, valid = _first_anchors(anchor, A)
            mask = _anchor_mask(valid)
            self.stats["anchors"] = valid.float().mean() * A / T
        d = h.shape[-1]
        a_in = h.gather(1, idx[..., None].expand(-1, -1, d))
        a = a_in
        for b in self.heavy:
            a = self._run(b, a, mask)
        h = h.scatter_add(1, idx[..., None].expand(-1, -1, d), (a - a_in) * valid[..., None])
        for b in self.final:
            h = self._run(b, h, win)
        h, cost = self.cards(h, self.book(x), a, idx, valid)
        return (self.norm(h), lh), cost

    def _ce_part(self, hn, y):
        return F.cross_entropy(self.head(hn).float().view(-1, self.head.out_features), y.reshape(-1), reduction="sum")

    def train_loss(self, out, y, train=True):
        hn, lh = out
        V = self.head.out_features
        loss = 0
        for j in range(0, hn.shape[1], 8192):                    # 8k-token chunks with recomputation
            part = (hn[:, j:j + 8192], y[:, j:j + 8192])
            loss = loss + (checkpoint(self._ce_part, *part, use_reentrant=False) if self.training else self._ce_part(*part))
        loss = loss / y.numel()
        if train:
            l_logits = self.l_head(lh[:, ::4])
            loss = loss + 0.3 * F.cross_entropy(l_logits.float().reshape(-1, V), y[:, ::4].reshape(-1))
        return loss


# ------------------------------------------------------------------------------------------------ registry
def build_legacy(name, vocab):
    S300 = dict(d=1024, light=4, heavy=14, final=2, heads=16)
    if name == "F300":
        return FullLM(vocab)
    if name == "F300ck":
        return FullLM(vocab, ckpt=True)
    if name == "T300ck":
        return PlainTransformerLM(vocab, d=1024, layers=16, heads=16, ckpt=True)
    if name == "Fsmall":
        return FullLM(vocab, d=256, light=1, heavy=2, final=1, heads=4, window=64)
    for pre, kw in (("S300p_", dict(packed=True)), ("S300c_", dict(select="cap")), ("S300q_", dict(select="quota")),
                    ("S300_", {})):
        if name.startswith(pre):
            return SurpriseLM(vocab, frac=int(name[len(pre):]) / 100, **S300, **kw)
    for pre, kw in (("surpcx", dict(select="cap", sit_cards=4)), ("surpc", dict(select="cap")),
                    ("surpq", dict(select="quota")), ("surpp", dict(packed=True)), ("surpimg", dict(images=True)),
                    ("surp", {})):
        if name.startswith(pre):
            return SurpriseLM(vocab, frac=int(name[len(pre):]) / 100, **kw)
    if name.startswith("sketch"):
        return SketchLM(vocab, k=int(name[6:]))
    if name.startswith("planwimg"):
        return ImagePlannerLM(vocab, k=int(name[8:]))
    if name.startswith("planwc"):
        k = int(name[6:])
        return PlannerSpeakerLM(vocab, k=k, window=2 * k, cards=True)
    if name.startswith("planw"):
        k = int(name[5:])
        return PlannerSpeakerLM(vocab, k=k, window=2 * k)
    if name.startswith("plan"):
        return PlannerSpeakerLM(vocab, k=int(name[4:]))
    if name == "img_sampled":
        return ImageTransformerLM(vocab, sampled=True)
    if name == "img_full":
        return ImageTransformerLM(vocab, sampled=False)
    if name == "cards":
        return CardsLM(vocab)
    if name == "tail":
        return CardsLM(vocab, use_cards=False)
    raise ValueError(f"unknown model name {name!r}")
