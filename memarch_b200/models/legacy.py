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

The families are assembled from one small toolkit - token losses, anchor pickers, "think on the picked words", a
bookmark reader, thought pooling - and a pattern table (`FAMILIES`) instead of one class per experiment.  Parameter
names match the reference, so its checkpoints load.  These models run on the library attention path (boolean masks
through SDPA): they are baselines and ablations, not the product model; the product's hot ops are in `memarch.py`.
"""
from __future__ import annotations

import math
import os
import re

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..ops import ref
from .blocks import DenseFFN, LightBlock, TransformerLM, _cdt   # noqa: F401 - TransformerLM re-exported for callers


# ------------------------------------------------------------------------------------------------ toolkit: losses
def token_ce(logits, y, reduction="mean"):
    """Cross-entropy of (.., V) logits against (..) targets, in fp32."""
    return F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), y.reshape(-1), reduction=reduction)


def light_head_aux(l_head, lh, y, weight=0.3, every=4):
    """The light part must learn to predict or its surprise means nothing: its own loss on every 4th position."""
    return weight * token_ce(l_head(lh[:, ::every]), y[:, ::every])


def no_cost(x):
    return torch.zeros((), device=x.device)


def maybe_ckpt(on, fn, *a):
    return checkpoint(fn, *a, use_reentrant=False) if on else fn(*a)


class ProtoLM(nn.Module):
    """What every prototype shares with the trainer: `forward(x, prep) -> (out, read cost)`, `train_loss(out, y)`."""

    def train_loss(self, out, y, train=True):
        return token_ce(out, y)


# ------------------------------------------------------------------------------------------------ toolkit: blocks
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


def stack(kind, n, *a):
    return nn.ModuleList(kind(*a) for _ in range(n))


def band_mask(T, width, device):
    """True where a word may look: itself and the `width - 1` words before it."""
    t = torch.arange(T, device=device)
    back = t[:, None] - t[None, :]
    return (back >= 0) & (back < width)


class ShortConv(nn.Module):
    """Token mixing without attention: a gated depthwise convolution over the last `width` words."""

    def __init__(self, d, width=4):
        super().__init__()
        self.width = width
        self.norm = nn.RMSNorm(d)
        self.conv = nn.Conv1d(d, d, width, groups=d)
        self.gate = nn.Linear(d, d, bias=False)
        self.out = nn.Linear(d, d, bias=False)

    def forward(self, x):
        n = self.norm(x)
        past = F.pad(n.transpose(1, 2), (self.width - 1, 0))           # left padding only: causal
        mixed = self.conv(past).transpose(1, 2) * F.silu(self.gate(n))
        return x + self.out(mixed)


# ------------------------------------------------------------------------------------------------ toolkit: bookmarks
class BookmarkReader(nn.Module):
    """Find cards by their face, then re-read up to `max_read` raw tokens of the shelf (`book`) from each chosen
    card's bookmark, with a learned stop after every token (lm.py:80-125, full.py:185-239).

    `cards=None`: every earlier word is a card (its own state is its face, its position its bookmark).  Otherwise
    the cards are given states with bookmarks `idx` and flags `valid`, and the words are served in chunks with
    recomputation so that the word x card table never lives whole."""

    def __init__(self, d, d_book=128, top_k=4, max_read=4, d_face=64, chunk=4096):
        super().__init__()
        self.top_k, self.max_read, self.d_face, self.chunk = top_k, max_read, d_face, chunk
        self.norm = nn.RMSNorm(d)
        self.face = nn.Linear(d, d_face, bias=False)
        self.query = nn.Linear(d, d_face, bias=False)
        self.offset = nn.Parameter(torch.randn(max_read, d_book) * 0.02)
        self.halt_v = nn.Linear(d_book, 1)
        self.halt_h = nn.Linear(d, 1, bias=False)
        self.out = nn.Linear(d_book, d, bias=False)

    def _choose(self, n, faces, allowed):
        """Scores of the words' queries against the card faces -> (weights (B,Tq,k), chosen cards (B,Tq,k))."""
        sc = (self.query(n) @ faces.transpose(1, 2) / math.sqrt(self.d_face)).masked_fill(~allowed, -1e4)
        best, pick = sc.topk(min(self.top_k, sc.shape[-1]), -1)
        return F.softmax(best.float(), -1).type_as(n) * (best > -1e3), pick

    def _read(self, x, n, book, mark, w, qpos):
        """x + what was read; expected number of tokens read per word."""
        B, Tq, K = mark.shape
        width = book.shape[-1]
        at = mark[..., None] + torch.arange(self.max_read, device=x.device)          # (B,Tq,K,R) text positions
        seen = at <= qpos[None, :, None, None]                                       # not beyond the reading word
        at = at.clamp(max=book.shape[1] - 1)
        v = book.gather(1, at.reshape(B, -1, 1).expand(-1, -1, width)).view(B, Tq, K, self.max_read, width) + self.offset
        stop = torch.sigmoid(self.halt_v(v).squeeze(-1) + self.halt_h(n)[:, :, None])
        stop = torch.where(seen, stop, torch.ones_like(stop))
        stop = torch.cat([stop[..., :-1], torch.ones_like(stop[..., -1:])], -1)      # the last token always stops
        going = torch.cumprod(torch.cat([torch.ones_like(stop[..., :1]), 1 - stop[..., :-1]], -1), -1)
        per_card = ((going * stop * seen)[..., None] * v).sum(-2)
        expected = (w * (going * seen).sum(-1)).sum(-1).mean()
        return x + self.out((w[..., None] * per_card).sum(-2)), expected

    def over_text(self, x, book):
        x, book = x.float(), book.float()
        T = x.shape[1]
        n = self.norm(x)
        t = torch.arange(T, device=x.device)
        w, pick = self._choose(n, self.face(n), (t[None, :] < t[:, None])[None])
        return self._read(x, n, book, pick, w, t)

    def over_cards(self, x, book, cards, idx, valid):
        parts = []
        for s in range(0, x.shape[1], self.chunk):
            a = (x[:, s:s + self.chunk].float(), s, book.float(), cards.float(), idx, valid)
            parts.append(maybe_ckpt(self.training, self._cards_part, *a))
        return torch.cat([o for o, _ in parts], 1), torch.stack([c for _, c in parts]).mean()

    def _cards_part(self, x, start, book, cards, idx, valid):
        B, Tq, _ = x.shape
        n = self.norm(x)
        qpos = torch.arange(start, start + Tq, device=x.device)
        allowed = valid[:, None, :] & (idx[:, None, :] < qpos[None, :, None])
        w, pick = self._choose(n, self.face(self.norm(cards)), allowed)
        return self._read(x, n, book, idx.gather(1, pick.reshape(B, -1)).view(B, Tq, -1), w, qpos)

    def forward(self, x, book, cards=None, idx=None, valid=None):
        return self.over_text(x, book) if cards is None else self.over_cards(x, book, cards, idx, valid)


# ------------------------------------------------------------------------------------------------ toolkit: anchors
def surprise_of(l_head, lh, x, rows=None):
    """-log p(next word) under the light head, by groups of rows so that B x T x V never lives whole; 1e4 where
    nothing precedes."""
    B, T = x.shape
    out = torch.full((B, T), 1e4, device=x.device)
    rows = rows or max(1, B // 4)
    for r0 in range(0, B, rows):
        for t0 in range(0, T - 1, 8192):
            t1 = min(t0 + 8192, T - 1)
            lo = l_head(lh[r0:r0 + rows, t0:t1])
            hit = lo.gather(-1, x[r0:r0 + rows, t0 + 1:t1 + 1, None]).squeeze(-1)
            out[r0:r0 + rows, t0 + 1:t1 + 1] = (torch.logsumexp(lo, -1) - hit).float()
    return out


def pick_first(flag, C):
    """The first C flagged words of every text, in order: (positions (B,C), which of them are real)."""
    T = flag.shape[1]
    keep = flag & (flag.cumsum(1) <= C)
    order = ((~keep).long() * T + torch.arange(T, device=flag.device)).argsort(dim=-1, stable=True)[:, :C]
    return order, keep.gather(1, order)


def pick_quota(s, chunk, k):
    """The k most surprising words of every chunk of `chunk` words, in text order."""
    B, T = s.shape
    top = s.view(B, T // chunk, chunk).topk(k, -1).indices.sort(-1).values
    idx = (top + torch.arange(0, T, chunk, device=s.device)[None, :, None]).view(B, -1)
    return idx, torch.ones_like(idx, dtype=torch.bool)


def earlier_picked(valid):
    """Attention mask among the picked words: a word sees the real picked words up to itself (and always itself)."""
    A = valid.shape[1]
    lower = torch.ones(A, A, dtype=torch.bool, device=valid.device).tril()
    return ((lower[None] & valid[:, None, :]) | torch.eye(A, dtype=torch.bool, device=valid.device)[None])[:, None]


def think_on(h, idx, valid, blocks, run=None):
    """Run `blocks` on the picked words only and add what changed back into the stream.  Returns (h, picked states)."""
    at = idx[..., None].expand(-1, -1, h.shape[-1])
    before = h.gather(1, at)
    a, mask = before, earlier_picked(valid)
    for b in blocks:
        a = b(a, mask) if run is None else run(b, a, mask)
    return h.scatter_add(1, at, (a - before) * valid[..., None]), a


def think_packed(h, flag, blocks):
    """All flagged words of the batch as ONE dense sequence: a word sees the earlier flagged words of its own text,
    RoPE counts the flagged words of that text.  The length is rounded up to a multiple of 512 (few shapes)."""
    B, T, d = h.shape
    with torch.no_grad():
        where = flag.reshape(-1).nonzero().squeeze(1)
        N = where.numel()
        pad = max(512, -(-N // 512) * 512) - N
        text = where // T
        per_text = flag.sum(1)
        number = torch.arange(N, device=h.device) - (per_text.cumsum(0) - per_text)[text]
        zeros = torch.zeros(pad, dtype=torch.long, device=h.device)
        text_p = torch.cat([text, -1 - torch.arange(pad, device=h.device)])       # every padding slot is its own text
        slot = torch.arange(N + pad, device=h.device)
        mask = (text_p[:, None] == text_p[None, :]) & (slot[None, :] <= slot[:, None])
        rope_pos, src = torch.cat([number, zeros]), torch.cat([where, zeros])
    flat = h.reshape(B * T, d)
    before = flat[src][None]
    a = before
    for b in blocks:
        a = b(a, mask[None, None], rope_pos)
    return flat.index_add(0, where, (a - before)[0, :N]).view(B, T, d)


# ------------------------------------------------------------------------------------------------ word images
def load_word_images(vocab, width=768):
    """Frozen word images.  The reference takes GPT-2's embedding table from the hub (lm.py:166-176); offline the
    table comes from `WORD_IMAGES` (a .pt / .npy of shape (n, width)) or, failing that, a seeded random table."""
    path = os.environ.get("WORD_IMAGES")
    if path and os.path.exists(path):
        import numpy as np
        t = torch.load(path) if path.endswith(".pt") else torch.from_numpy(np.load(path))
        table = torch.zeros(vocab, t.shape[1])
        table[:min(vocab, len(t))] = t[:vocab].float()
        return table
    return torch.randn(vocab, width, generator=torch.Generator().manual_seed(768)) * 0.1


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
        c = counts.float() + 1
        q = c / c[:self.n_real].sum()
        q[self.n_real:] = 1e-12
        self.log_q.copy_(q.log())

    def logits(self, h):
        lo = self.proj(h) @ self.img.T.type_as(h)
        lo[..., self.n_real:] = -1e4                               # padding rows of the vocabulary are no words
        return lo

    def loss(self, h, y, train):
        if not (train and self.sampled):
            return token_ce(self.logits(h), y)
        want = self.proj(h).reshape(-1, self.img.shape[1])
        y = y.reshape(-1)
        others = torch.multinomial(self.log_q.exp(), self.n_neg, replacement=True)
        right = (want * self.img[y].type_as(want)).sum(-1, keepdim=True) - self.log_q[y, None]
        wrong = want @ self.img[others].T.type_as(want) - self.log_q[others][None]
        wrong = wrong.masked_fill(others[None] == y[:, None], -1e4)           # a sampled "negative" that is the answer
        return F.cross_entropy(torch.cat([right, wrong], -1).float(), torch.zeros_like(y))


# ------------------------------------------------------------------------------------------------ families
class CardsLM(ProtoLM):
    def __init__(self, vocab, d=512, layers=8, d_book=128, card_layers=(3, 6), use_cards=True):
        super().__init__()
        self.emb, self.book = nn.Embedding(vocab, d), nn.Embedding(vocab, d_book)
        self.tails, self.ffns = stack(ShortConv, layers, d), stack(DenseFFN, layers, d)
        self.cards = nn.ModuleDict({str(i): BookmarkReader(d, d_book) for i in (card_layers if use_cards else ())})
        self.norm, self.head = nn.RMSNorm(d), nn.Linear(d, vocab, bias=False)

    def forward(self, x, prep=None):
        h, cost = self.emb(x), no_cost(x)
        shelf = self.book(x) if len(self.cards) else None
        for i, (mix, ffn) in enumerate(zip(self.tails, self.ffns)):
            h = mix(h)
            if str(i) in self.cards:
                h, c = self.cards[str(i)](h, shelf)
                cost = cost + c
            h = ffn(h)
        return self.head(self.norm(h)), cost


class PlainTransformerLM(ProtoLM):
    """Transformer returning logits (the shape the prototypes share); `images`: the head is the word-image output
    and the model returns the state that goes into it."""

    def __init__(self, vocab, d=512, layers=8, heads=8, ckpt=False, images=None):
        super().__init__()
        self.ckpt = ckpt
        self.emb, self.blocks, self.norm = nn.Embedding(vocab, d), stack(MaskedBlock, layers, d, heads), nn.RMSNorm(d)
        if images is None:
            self.head = nn.Linear(d, vocab, bias=False)
        else:
            self.out = ImageOut(d, vocab, sampled=images)

    def hidden(self, x):
        h = self.emb(x)
        for b in self.blocks:
            h = maybe_ckpt(self.ckpt and self.training, b, h)
        return self.norm(h)

    def forward(self, x, prep=None):
        h = self.hidden(x)
        return (self.head(h) if hasattr(self, "head") else h), no_cost(x)

    def train_loss(self, out, y, train=True):
        return self.out.loss(out, y, train) if hasattr(self, "out") else token_ce(out, y)


def ImageTransformerLM(vocab, sampled):
    return PlainTransformerLM(vocab, images=bool(sampled))


class ThoughtLM(ProtoLM):
    """Front shared by the planner models: embed, add the position inside the thought, squeeze every K-word thought
    to one vector (attention pooling with four learned queries), run the planner over the thoughts.  After `later`
    thought j carries what the planner knew BEFORE it (a learned vector for the first)."""

    def _front(self, vocab, k, d, p_layers, heads):
        self.k = k
        self.emb = nn.Embedding(vocab, d)
        self.pos = nn.Parameter(torch.randn(k, d) * 0.02)
        self.pool_q = nn.Parameter(torch.randn(4, d) * 0.02)
        self.pool_out = nn.Linear(4 * d, d, bias=False)
        self.start = nn.Parameter(torch.randn(d) * 0.02)
        self.planner, self.p_norm = stack(MaskedBlock, p_layers, d, heads), nn.RMSNorm(d)

    def thoughts(self, x):
        B, T = x.shape
        words = self.emb(x).view(B, T // self.k, self.k, -1) + self.pos
        look = torch.einsum("bnkd,qd->bnqk", words, self.pool_q).softmax(-1)
        p = self.pool_out(torch.einsum("bnqk,bnkd->bnqd", look, words).flatten(2))
        for b in self.planner:
            p = b(p)
        return words, self.p_norm(p)

    def later(self, p):
        return torch.cat([self.start.expand(p.shape[0], 1, -1).type_as(p), p[:, :-1]], 1)


class PlannerSpeakerLM(ThoughtLM):
    def __init__(self, vocab, k, d=512, p_layers=8, s_layers=3, heads=8, window=0, cards=False, images=False):
        super().__init__()
        self.window = window
        self._front(vocab, k, d, p_layers, heads)
        self.intent = nn.Linear(d, d, bias=False)
        self.book = nn.Embedding(vocab, 128) if cards else None
        self.cards = BookmarkReader(d, 128) if cards else None
        self.speaker, self.norm = stack(MaskedBlock, s_layers, d, heads), nn.RMSNorm(d)
        self.head = nn.Identity() if images else nn.Linear(d, vocab, bias=False)

    def forward(self, x, prep=None):
        B, T = x.shape
        words, p = self.thoughts(x)
        h = words + self.later(self.intent(p))[:, :, None]
        cost = no_cost(x)
        if not self.window:                                      # the speaker sees its own thought only
            h = h.reshape(B * (T // self.k), self.k, -1)
            for b in self.speaker:
                h = b(h)
            return self.head(self.norm(h.view(B, T, -1))), cost
        h = h.reshape(B, T, -1)
        mask = band_mask(T, self.window, x.device)
        for i, b in enumerate(self.speaker):
            h = b(h, mask)
            if i == 0 and self.cards is not None:
                h, cost = self.cards(h, self.book(x))
        return self.head(self.norm(h)), cost


class ImagePlannerLM(nn.Module):
    def __init__(self, vocab, k):
        super().__init__()
        self.core = PlannerSpeakerLM(vocab, k=k, window=2 * k, images=True)
        self.out = ImageOut(512, vocab, sampled=True)

    def forward(self, x, prep=None):
        return self.core(x)

    def train_loss(self, h, y, train=True):
        return self.out.loss(h, y, train)


class SketchLM(ThoughtLM):
    def __init__(self, vocab, k=32, d=512, p_layers=8, s_layers=3, heads=8, M=8, menu=256):
        super().__init__()
        self.M, self.n_menu, self.window = M, min(menu, vocab), 2 * k
        self._front(vocab, k, d, p_layers, heads)
        self.sketch = nn.Linear(d, M * d, bias=False)
        self.menu_head = nn.Linear(d, vocab, bias=False)
        self.speaker = stack(MaskedBlock, s_layers, d, heads)
        self.c_norm = nn.ModuleList(nn.RMSNorm(d) for _ in range(s_layers))
        self.c_q = nn.ModuleList(nn.Linear(d, d, bias=False) for _ in range(s_layers))
        self.c_out = nn.ModuleList(nn.Linear(d, d, bias=False) for _ in range(s_layers))
        self.norm, self.head, self.other = nn.RMSNorm(d), nn.Linear(d, vocab, bias=False), nn.Linear(d, 1)
        self.stats = {}

    def forward(self, x, prep=None):
        B, T = x.shape
        n = T // self.k
        words, p = self.thoughts(x)
        p = self.later(p)
        sk = self.sketch(p).view(B, n, self.M, -1)               # the thought's sketch: M vectors
        menu_logits = self.menu_head(p)
        menu = menu_logits.detach().float().topk(self.n_menu, -1).indices
        h = (words + sk.mean(2)[:, :, None]).reshape(B, T, -1)
        mask, scale = band_mask(T, self.window, x.device), h.shape[-1] ** -0.5
        for blk, cn, cq, co in zip(self.speaker, self.c_norm, self.c_q, self.c_out):
            h = blk(h, mask)
            look = (torch.einsum("bnkd,bnmd->bnkm", cq(cn(h)).view(B, n, self.k, -1), sk) * scale).softmax(-1)
            h = h + co(torch.einsum("bnkm,bnmd->bnkd", look, sk).reshape(B, T, -1))      # every word consults the sketch
        return (self.norm(h), menu, menu_logits), no_cost(x)

    def train_loss(self, out, y, train=True):
        hn, menu, menu_logits = out
        B, T, d = hn.shape
        n, S = T // self.k, self.n_menu
        yb, hb = y.reshape(B, n, self.k), hn.view(B, n, self.k, d)
        planner_term = -F.log_softmax(menu_logits.float(), -1).gather(-1, yb).mean()
        same = menu[:, :, None, :] == yb[..., None]
        on_menu, slot = same.any(-1), same.float().argmax(-1)
        # the speaker chooses among the menu's words plus one "something else" slot
        small = torch.cat([torch.einsum("bnkd,bnmd->bnkm", hb, self.head.weight[menu].type_as(hb)), self.other(hb)], -1)
        logp = F.log_softmax(small.float(), -1)
        tgt = torch.where(on_menu, slot, torch.full_like(slot, S))
        off = ~on_menu
        self.stats["miss"] = off.float().mean()
        rest = None
        if int(off.sum()):                                       # full vocabulary only for words outside the menu
            taken = menu[:, :, None, :].expand(B, n, self.k, S)[off]
            rest = (hb[off] @ self.head.weight.T.type_as(hb)).float().scatter(1, taken, -1e4)
        if train:
            loss = F.nll_loss(logp.view(-1, S + 1), tgt.view(-1))
            if rest is not None:
                loss = loss + F.cross_entropy(rest, yb[off], reduction="sum") / y.numel()
            return loss + 0.5 * planner_term
        lp = logp.gather(-1, tgt[..., None]).squeeze(-1)
        if rest is not None:
            lp = lp.clone()
            lp[off] = lp[off] + F.log_softmax(rest, -1).gather(-1, yb[off][:, None]).squeeze(-1)
        return -lp.mean()


class AnchorLM(ProtoLM):
    """Thinking on surprises, both generations: light blocks on every word, a light head whose error picks the
    anchors (running threshold `tau`), heavy ATTENTION blocks on the anchors, final blocks.

    `SurpriseLM` options: `select` threshold (variable count, padded to the batch maximum) / cap / quota, `packed`,
    situation cards, word-image output.  `FullLM` (`reread=True`): windowed light and final blocks, the anchors as
    cards of a bookmark reader, chunked loss with recomputation."""

    def __init__(self, vocab, d=512, light=2, heavy=8, final=1, heads=8, frac=0.2, images=False, packed=False,
                 select="threshold", chunk=128, cap=0.25, sit_cards=0, reread=False, window=0, ckpt=False):
        super().__init__()
        self.frac, self.packed, self.select, self.chunk, self.cap = frac, packed, select, chunk, cap
        self.sit_cards, self.reread, self.window, self.ckpt = sit_cards, reread, window, ckpt
        if sit_cards:
            self.sit_keys = nn.Parameter(torch.randn(sit_cards, d) * 0.02)
            self.sit_gain = nn.Parameter(torch.zeros(sit_cards, d))
        outer = LightBlock if reread else MaskedBlock
        self.emb = nn.Embedding(vocab, d)
        self.light = stack(outer, light, d, heads)
        self.l_norm = nn.RMSNorm(d)
        self.l_head = nn.Sequential(nn.Linear(d, 128, bias=False), nn.Linear(128, vocab, bias=False))
        self.heavy, self.final = stack(MaskedBlock, heavy, d, heads), stack(outer, final, d, heads)
        self.norm = nn.RMSNorm(d)
        if reread:
            self.book, self.cards = nn.Embedding(vocab, 128), BookmarkReader(d)
        self.out = ImageOut(d, vocab, sampled=False) if images else None
        self.head = None if images else nn.Linear(d, vocab, bias=False)
        self.register_buffer("tau", torch.tensor(5.0))
        self.stats = {}

    def _run(self, blk, *a):
        return maybe_ckpt(self.ckpt and self.training, blk, *a)

    def _situation(self, h):
        """Situation of word t = mean of the input up to t (no look-ahead); soft choice among `sit_cards` learned
        situations, each with its own per-channel gain on the input."""
        T = h.shape[1]
        tri = torch.ones(T, T, device=h.device).tril_()
        sit = (tri / tri.sum(1, keepdim=True)).type_as(h) @ h.detach()
        p = (F.normalize(sit, dim=-1) @ F.normalize(self.sit_keys, dim=-1).T * 8).softmax(-1)
        return h * (1 + (p @ self.sit_gain).type_as(h))

    def _pick(self, s, flag, T):
        """Which words think: (idx, valid), or None for the packed form."""
        if self.reread or self.select == "cap" or (self.select == "quota" and not self.training):
            return pick_first(flag, max(1, round(T * self.cap)))
        if self.select == "quota":
            return pick_quota(s, self.chunk, max(1, round(self.chunk * self.frac)))
        if self.packed:
            return None
        return pick_first(flag, max(1, int(flag.sum(1).max())))  # variable width: one host read per step

    def forward(self, x, prep=None):
        B, T = x.shape
        win = (self.window if T > self.window else None,) if self.reread else ()
        h = self.emb(x)
        if self.sit_cards:
            h = self._situation(h)
        for b in self.light:
            h = self._run(b, h, *win)
        lh = self.l_norm(h)
        with torch.no_grad():
            s = surprise_of(self.l_head, lh.detach(), x, rows=max(1, min(B, 32768 // T)) if self.reread else None)
            flag = s > self.tau                                  # chosen with the threshold before its update
            if self.training:
                self.tau.mul_(0.9).add_(0.1 * ref.tau_quantile(s, self.frac))
            picked = self._pick(s, flag, T)
            static = picked is not None and (self.reread or self.select != "threshold")
            self.stats["anchors"] = (picked[1].float().mean() * picked[0].shape[1] / T) if static else flag.float().mean()
        if picked is None:
            h, states = think_packed(h, flag, self.heavy), None
        else:
            h, states = think_on(h, *picked, self.heavy, self._run if self.reread else None)
        for b in self.final:
            h = self._run(b, h, *win)
        if self.reread:
            h, cost = self.cards(h, self.book(x), states, *picked)
            return (self.norm(h), lh), cost
        hn = self.norm(h)
        return (self.out.logits(hn) if self.out is not None else self.head(hn), lh), no_cost(x)

    def _head_sum(self, hn, y):
        return token_ce(self.head(hn), y, "sum")

    def train_loss(self, out, y, train=True):
        first, lh = out
        if self.reread:                                          # states in: 8k-token chunks with recomputation
            loss = sum(maybe_ckpt(self.training, self._head_sum, first[:, j:j + 8192], y[:, j:j + 8192])
                       for j in range(0, first.shape[1], 8192)) / y.numel()
        else:
            loss = token_ce(first, y)
        return loss + light_head_aux(self.l_head, lh, y) if train else loss


def SurpriseLM(vocab, **kw):
    return AnchorLM(vocab, **kw)


def FullLM(vocab, d=1024, light=4, heavy=14, final=2, heads=16, frac=0.2, cap=0.25, window=2048, ckpt=False):
    return AnchorLM(vocab, d=d, light=light, heavy=heavy, final=final, heads=heads, frac=frac, cap=cap, window=window,
                    ckpt=ckpt, reread=True)


# ------------------------------------------------------------------------------------------------ registry
_S300 = dict(d=1024, light=4, heavy=14, final=2, heads=16)
_PCT = lambda m: int(m.group(1)) / 100       # noqa: E731
_K = lambda m: int(m.group(1))               # noqa: E731

# (pattern, builder(vocab, match)); first match wins
FAMILIES = [
    (r"F300", lambda v, m: FullLM(v)),
    (r"F300ck", lambda v, m: FullLM(v, ckpt=True)),
    (r"Fsmall", lambda v, m: FullLM(v, d=256, light=1, heavy=2, final=1, heads=4, window=64)),
    (r"T300ck", lambda v, m: PlainTransformerLM(v, d=1024, layers=16, heads=16, ckpt=True)),
    (r"S300p_(\d+)", lambda v, m: SurpriseLM(v, frac=_PCT(m), packed=True, **_S300)),
    (r"S300c_(\d+)", lambda v, m: SurpriseLM(v, frac=_PCT(m), select="cap", **_S300)),
    (r"S300q_(\d+)", lambda v, m: SurpriseLM(v, frac=_PCT(m), select="quota", **_S300)),
    (r"S300_(\d+)", lambda v, m: SurpriseLM(v, frac=_PCT(m), **_S300)),
    (r"surpcx(\d+)", lambda v, m: SurpriseLM(v, frac=_PCT(m), select="cap", sit_cards=4)),
    (r"surpc(\d+)", lambda v, m: SurpriseLM(v, frac=_PCT(m), select="cap")),
    (r"surpq(\d+)", lambda v, m: SurpriseLM(v, frac=_PCT(m), select="quota")),
    (r"surpp(\d+)", lambda v, m: SurpriseLM(v, frac=_PCT(m), packed=True)),
    (r"surpimg(\d+)", lambda v, m: SurpriseLM(v, frac=_PCT(m), images=True)),
    (r"surp(\d+)", lambda v, m: SurpriseLM(v, frac=_PCT(m))),
    (r"sketch(\d+)", lambda v, m: SketchLM(v, k=_K(m))),
    (r"planwimg(\d+)", lambda v, m: ImagePlannerLM(v, k=_K(m))),
    (r"planwc(\d+)", lambda v, m: PlannerSpeakerLM(v, k=_K(m), window=2 * _K(m), cards=True)),
    (r"planw(\d+)", lambda v, m: PlannerSpeakerLM(v, k=_K(m), window=2 * _K(m))),
    (r"plan(\d+)", lambda v, m: PlannerSpeakerLM(v, k=_K(m))),
    (r"img_sampled", lambda v, m: ImageTransformerLM(v, sampled=True)),
    (r"img_full", lambda v, m: ImageTransformerLM(v, sampled=False)),
    (r"cards", lambda v, m: CardsLM(v)),
    (r"tail", lambda v, m: CardsLM(v, use_cards=False)),
]


def build_legacy(name, vocab):
    for pattern, make in FAMILIES:
        m = re.fullmatch(pattern, name)
        if m:
            return make(vocab, m)
    raise ValueError(f"unknown model name {name!r}")
