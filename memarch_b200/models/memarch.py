"""MemArchLM: the product model (the reference's FullLM2, full2.py:1269-1997).

    light window layers -> memory read (focus + cards) -> light window layers
      -> surprise -> anchors (threshold + per-text cap) -> heavy layers on anchors only (no attention)
      -> final window layers -> re-reading at bookmarks + recognition -> output head

`forward(x[, prep]) -> ((hn, lh), cost)`, `train_loss(out, y, train)`, `prep(x)`, `table_rows(x)`,
`before_step(step)`, `rebank(step)`, `.stats` (device tensors, no host sync) - the reference's public surface.
Parameter and buffer names equal the reference's so `state_dict`s interchange.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..config import ModelConfig
from ..ops import ref
from .blocks import DenseFFN, LightBlock, _cdt, run_blocks
from .memory import CardMemory, VolumeMemory
from .moe import AnchorMoE
from .reread import Reread

_BUCKET_MUL = -2960836687051489901       # odd 64-bit multiplier (0xD6E8FEB86659FD93 as a signed number)
_BUCKET_W = 8                             # keys per bucket: one 64-byte row


def bucket_table(keys, width=_BUCKET_W):
    """Phrase keys -> (bucket rows of keys (M, width), rows of their numbers, M - 1).  A key lives in the row its hash
    names, anywhere among the row's `width` places: a lookup is ONE hash and one 64-byte row to compare, no second
    probe and no chain.  Built without a Python loop over the keys: sort by bucket, number the keys inside their
    bucket, and double the table in the rare case that a bucket overflows (at one key per bucket on average the chance
    that any of 2^18 buckets gets more than eight is below 1e-3).  Stands where the reference has a two-choice cuckoo
    table (full2.py:126-150); the tables are not part of a checkpoint, so the layout is free."""
    n = len(keys)
    M = 1 << max(8, int(np.ceil(np.log2(max(n, 1)))))
    while True:
        with np.errstate(over="ignore"):
            bucket = ((keys * np.int64(_BUCKET_MUL)) >> 40) & (M - 1)
        order = np.argsort(bucket, kind="stable")
        b_sorted = bucket[order]
        place = np.arange(n) - np.searchsorted(b_sorted, b_sorted, side="left")
        if n == 0 or place.max() < width:
            break
        M *= 2
    rows = np.full((M, width), -(1 << 62), dtype=np.int64)               # no key is that negative
    numbers = np.zeros((M, width), dtype=np.int64)
    rows[b_sorted, place] = keys[order]
    numbers[b_sorted, place] = order
    return rows, numbers, M - 1


class HeavyCtxAttn(nn.Module):
    """Optional: before a heavy layer every anchor looks back into the light states of the words up to itself
    (cross-attention without positions; zero-initialised output, so the model starts as if it were absent).
    (full2.py:1245-1266)"""

    def __init__(self, d, heads=8):
        super().__init__()
        self.h = heads
        self.nq, self.nk = nn.RMSNorm(d), nn.RMSNorm(d)
        self.q, self.kv, self.o = (nn.Linear(d, n * d, bias=False) for n in (1, 2, 1))
        nn.init.zeros_(self.o.weight)

    def _heads(self, t, parts):
        """(B, L, parts * D) -> parts tensors (B, heads, L, D / heads)"""
        B, L, _ = t.shape
        return t.view(B, L, parts, self.h, -1).permute(2, 0, 3, 1, 4)

    def forward(self, a, ctx, idx):
        (q,) = self._heads(self.q(self.nq(a)), 1)
        k, v = self._heads(self.kv(self.nk(ctx)), 2)
        word = torch.arange(ctx.shape[1], device=a.device)
        may_see = (word[None, None, :] <= idx[:, :, None])[:, None]            # anchor at position p sees words <= p
        y = F.scaled_dot_product_attention(q, k.type_as(q), v.type_as(q), attn_mask=may_see)
        return a + self.o(y.transpose(1, 2).flatten(2))


class _HostPrep:
    """CPU copies of the buffers that `MemArchLM.prep` reads, with that method and its helpers borrowed."""

    _TABLES = ("phr_keys", "phr_hkey", "phr_hval", "phr4_keys", "lock_bucket", "sp_E", "sp_H", "sp_lp", "sp_lse")

    def __init__(self, model):
        self.vocab = model.vocab
        for name in self._TABLES:
            if hasattr(model, name):
                setattr(self, name, getattr(model, name).detach().cpu())
        for name in ("phr_V", "phr_hmask"):
            if hasattr(model, name):
                setattr(self, name, getattr(model, name))
        for flag in ("phr", "phr4", "ind_a", "lock_w"):          # only their presence is asked for
            if hasattr(model, flag):
                setattr(self, flag, True)

    def __call__(self, x):
        return self.prep(x.cpu())


class MemArchLM(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.cfg = cfg
        c = cfg
        vocab, d = c.vocab, c.d
        self.vocab, self.frac, self.cap, self.window, self.seg = vocab, c.frac, c.cap, c.window, c.seg
        self.use_memory = c.use_memory
        self.emb = nn.Embedding(vocab, d)
        self.book = nn.Embedding(vocab, 128)
        blk = lambda: LightBlock(d, c.heads, c.blk, c.light_ffn, c.light_moe, rope_half=c.rope_half)
        self.light_a = nn.ModuleList(blk() for _ in range(c.light_a))
        mk = dict(vars(c.memory))
        volume = mk.pop("volume")
        self.memory = (VolumeMemory if volume else CardMemory)(d, **mk)
        self.light_b = nn.ModuleList(blk() for _ in range(c.light_b))
        self.l_norm = nn.RMSNorm(d)
        self.l_head = nn.Sequential(nn.Linear(d, 128, bias=False), nn.Linear(128, vocab, bias=False))
        self.moe = c.moe and not c.fish_n
        w_dtype = torch.bfloat16 if c.bf16_experts else torch.float32
        self._fish_aux = None
        self._hfull = -1
        self._mix = self._tongue = None
        self._vp = None
        self._surp = None                                # the light head's surprise of the last forward (B,T)
        self.stream_u = None                             # running common direction of the stream (the trainer copies the optimizer's U here)
        if c.fish_n:
            from .fishki import FishPool
            self.fish = FishPool(d, n=c.fish_n, hf=c.fish_hf, kinds=c.fish_kinds, pool=c.fish_pool, center=c.fish_center)
            self.heavy = nn.ModuleList()
        elif c.moe:
            self.heavy = nn.ModuleList(
                AnchorMoE(d, E=c.n_exp, k_avg=c.moe_k if c.bank else 2, k_max=max(4, c.moe_k) if c.bank else 4,
                          budget=c.moe == "budget", wave=c.wave, wave_every=c.wave_every, students=c.students,
                          hint_w=c.hint_w, frozen=c.n_frozen, bank=c.bank, act=c.moe_act if c.bank else "swiglu",
                          w_dtype=w_dtype if c.bank else torch.float32, bank_q=c.bank_q, wave_warm=c.wave_warm,
                          err_thr=c.err_thr, cap_align=c.moe_cap_align, dropless=c.moe_dropless)
                for _ in range(c.heavy))
        else:
            self.heavy = nn.ModuleList(DenseFFN(d) for _ in range(c.heavy))
        for b in self.heavy:
            b.fill = c.frac / c.cap
            if c.layer_stats and hasattr(b, "layer_stats"):
                b.layer_stats = True
        self.final = nn.ModuleList(blk() for _ in range(c.final))
        for b in list(self.light_a) + list(self.light_b) + list(self.final):
            b.attn_gain = c.attn_gain
        for b in self.light_b:
            b.tether_pcut = c.rope_pcut
        if c.prev_in:
            self.prev_g = nn.Parameter(torch.full((1,), -1.0))
        self.reread = Reread(d)
        self.norm = nn.RMSNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)
        self.register_buffer("tau", torch.tensor(5.0))
        if c.rope_mem:
            self.register_buffer("rope_tau", torch.tensor(float(c.rope_tau0)))
            if c.rope_qfrac < 1.0:
                self.register_buffer("rope_qtau", torch.tensor(float(c.rope_qtau0)))
        self._tether_mass = None
        self.want_stream_mean = False
        self._hoop = None
        if c.uroboros:
            from .fishki import Uroboros
            self.hoop = Uroboros(d)
            self.hoop_budget = c.uroboros_budget         # the training loop may step it down (`Uroboros.next_budget`)
        self.stats = {}
        self.panic = c.panic
        self.short_v = c.short_v
        if c.short_v:
            self._init_short_vocab()
        n_light = c.light_a + c.light_b
        if "ve" in c.blk:
            self.ve = nn.ModuleList(nn.Embedding(vocab, d) for _ in range(n_light))
        if "smear" in c.blk:
            self.smear = nn.Linear(d, 1, bias=False)
            nn.init.zeros_(self.smear.weight)
        if c.phrase_init:
            self._init_phrasebook(torch.load(c.phrase_init, weights_only=False))
        if c.phrase3:
            self._init_phrase_table(torch.load(c.phrase3, weights_only=False), "phr")
        if c.phrase4:
            self._init_phrase_table(torch.load(c.phrase4, weights_only=False), "phr4")
        if c.skip:
            sk = torch.load(c.skip, weights_only=False)
            g = c.skip_g / c.phrase_c
            self.skip_o = sorted(sk)
            self.skip = nn.ModuleList(nn.Embedding(vocab, d) for _ in self.skip_o)
            with torch.no_grad():
                for t, o in zip(self.skip, self.skip_o):
                    t.weight.zero_()
                    t.weight[:sk[o].shape[0]].copy_(sk[o] * g)
        if c.tongue:
            pt = torch.load(c.tongue, weights_only=False)
            for k in ("bi_idx", "bi_val", "tri_idx", "tri_val"):
                self.register_buffer("tg_" + k, pt[k], persistent=False)
            self.register_buffer("tg_keys", pt["keys"].long(), persistent=False)
            self.tg_a = nn.Parameter(torch.tensor([c.tongue_a, c.tongue_a]))
        if c.induct:
            self._init_locks()
        if c.heavy_attn:
            self.h_attn = nn.ModuleList(HeavyCtxAttn(d, c.heads) for _ in range(c.heavy))
        self.n_draft = c.n_draft
        if c.n_draft:
            self.draft = nn.ModuleList(nn.Linear(d, d, bias=False) for _ in range(c.n_draft))
            for lin in self.draft:
                nn.init.zeros_(lin.weight)
            self.draft_norm = nn.RMSNorm(d)

    # ------------------------------------------------------------------------------------------ constructors
    def _counts(self):
        c = self.cfg
        cnt = np.zeros(self.vocab, np.int64)
        if c.token_counts:
            c0 = np.load(c.token_counts).astype(np.int64)[:self.vocab]
            cnt[:len(c0)] = c0
        return cnt

    def _init_short_vocab(self):
        """Two-level output: K most frequent tokens + a "rare" bucket row (last vocab row) (full2.py:1305-1337)."""
        vocab, K = self.vocab, self.short_v
        cnt = self._counts()
        top = torch.from_numpy(np.argsort(-cnt, kind="stable")[:K].copy())
        pos = torch.full((vocab,), K, dtype=torch.long)
        pos[top] = torch.arange(K)
        self.register_buffer("sv_ids", top, persistent=False)
        self.register_buffer("sv_pos", pos, persistent=False)
        self.sv_bucket = vocab - 1
        assert cnt[self.sv_bucket] == 0 and pos[self.sv_bucket] == K, "last vocab row must be unused"
        msk = (pos < K).float() * -1e4
        msk[self.sv_bucket] = -1e4
        self.register_buffer("sv_mask", msk, persistent=False)
        rare = 1 - cnt[top.numpy()].sum() / max(cnt.sum(), 1) if cnt.sum() else 0.18
        rare = min(max(rare, 1e-3), 0.999)
        self.sv_prior0 = float(np.log(rare * K / (1 - rare)))
        self.sv_prior1 = float(np.log(rare))
        with torch.no_grad():
            self.head.weight[self.sv_bucket].zero_()
        self.rare_cap = self.cfg.rare_cap

    def _init_phrasebook(self, ph):
        """emb <- E / rms_row(E), head <- H·c, head_bias <- log p(next) (full2.py:1346-1365)."""
        c = self.cfg
        E, H = ph["emb"].float(), ph["head"].float()
        with torch.no_grad():
            rms = E.pow(2).mean(1, keepdim=True).sqrt().clamp(min=1e-6)
            n = E.shape[0]
            self.emb.weight[:n].copy_(E / rms)
            self.head.weight[:n].copy_(H * c.phrase_c)
            self.head.weight[n:].zero_()
        lp = torch.full((self.vocab,), float(ph["logp_next"].min()) - 5)
        lp[:n] = ph["logp_next"]
        self.head_bias = nn.Parameter(lp)
        if c.opaque and "ent" in ph:
            self.register_buffer("ent_t", ph["ent"].float(), persistent=False)
        if c.surp_phrase:
            self.register_buffer("sp_E", ((E / rms) * c.phrase_c).to(torch.bfloat16).contiguous(), persistent=False)
            self.register_buffer("sp_H", H.to(torch.bfloat16).contiguous(), persistent=False)
            self.register_buffer("sp_lp", ph["logp_next"].float(), persistent=False)
            self.register_buffer("sp_lse", ph["lse"].float(), persistent=False)

    def _init_phrase_table(self, tg, name):
        c = self.cfg
        K = len(tg["keys"])
        self.register_buffer(name + "_keys", tg["keys"].long(), persistent=False)
        if name == "phr" and c.phr_hash:
            hk, hv, self.phr_hmask = bucket_table(tg["keys"].long().numpy())
            self.register_buffer("phr_hkey", torch.from_numpy(hk), persistent=False)
            self.register_buffer("phr_hval", torch.from_numpy(hv), persistent=False)
        emb = nn.Embedding(K + 1, c.d)
        with torch.no_grad():
            emb.weight.zero_()
            emb.weight[:K].copy_(tg["vec"] / c.phrase_c)
        setattr(self, name, emb)
        self.phr_V = c.phr_v

    def _init_locks(self):
        c = self.cfg
        self.ind_a = nn.Parameter(torch.tensor([1.0, 1.0]))
        self.ind_in_g = nn.Parameter(torch.full((3,), -2.0))
        if c.induct == "lock":
            cnt = self._counts()
            bucket = np.clip(np.floor(np.log10(cnt + 1)), 0, 6).astype(np.int64)
            self.register_buffer("lock_bucket", torch.tensor(bucket), persistent=False)
            lw = torch.load(c.lock_trust, weights_only=False) if c.lock_trust else torch.ones(3, 7)
            self.lock_w = nn.Parameter(lw.clone().float())
            if c.induct_mix:
                pm = (lw.float().exp() * math.exp(-4.5)).clamp(0.005, 0.95)
                self.mix_w = nn.Parameter(torch.log(pm / (1 - pm)))

    # ------------------------------------------------------------------------------------------ token-only prep
    def _phr_idx(self, x):
        if hasattr(self, "phr_hkey"):
            ctx = torch.cat([torch.full_like(x[:, :1], -1), x[:, :-1]], 1) * self.phr_V + x
            row = ((ctx * _BUCKET_MUL) >> 40) & self.phr_hmask
            same = self.phr_hkey[row] == ctx[..., None]                 # at most one place of the row holds the key
            found = (self.phr_hval[row] * same).sum(-1)
            return torch.where(same.any(-1), found, torch.full_like(ctx, self.phr_keys.numel()))
        return ref.phrase_index(x, self.phr_keys, self.phr_V)

    def _lock_votes(self, x, prep=None):
        """Keys and locks: for each position the words that followed the last earlier occurrence of its 1-, 2- and
        3-word endings (`cand`), and how strongly each of them votes for the next word: the lock's trust (per key
        length and rarity bucket of the current word when a trust table is loaded, else one scalar per key length),
        zero where the lock found nothing.  Returns (cand, votes, on, bucket).  (full2.py:1540-1559)"""
        if prep and "ind_cand" in prep:
            cand, on, bk = prep["ind_cand"], prep["ind_on"], prep["ind_bk"]
        else:
            cand, on, bk, _ = self._locks_raw(x)
        n_keys = on.shape[-1]
        if hasattr(self, "lock_w"):
            # index_select: its backward is an index_add (atomics on 7 values), not the sort-based index_put of `w[bk]`
            flat = bk.reshape(-1)
            trust = torch.stack([self.lock_w[k].index_select(0, flat).view_as(bk) for k in range(n_keys)], -1)
        else:
            trust = self.ind_a[:n_keys]
        return cand, on.float() * trust, on, bk

    def _mix_gate(self, cand, on, bk):
        """Pointer mixture: the candidate of the first lock that fired (longest key first) and the learned share of the
        output distribution it takes, by key length and rarity bucket.  Returns (candidate (B,T), share (B,T))."""
        fired = on.any(-1)
        first = on.float().argmax(-1)
        pick = (cand * on).sum(-1)
        n_buckets = self.mix_w.shape[1]
        share = torch.sigmoid(self.mix_w.reshape(-1).index_select(0, (first * n_buckets + bk).reshape(-1)).view_as(bk)) * fired
        self.stats["mix_g"] = (share.sum() / fired.sum().clamp(min=1)).detach()
        return pick, share

    def _tongue_from_tables(self, x):
        """"Tongue" bias from fixed tables instead of locks: the stored top continuations of the (previous, current)
        pair where the pair is in the phrase table, else of the current word alone, scaled by the two learned
        strengths `tg_a`.  Returns (candidates (B,T,k), bias values (B,T,k)).  (full2.py:1582-1591)"""
        V0 = self.cfg.phr_v
        word = x.clamp(max=V0 - 1)
        pair = torch.cat([torch.full_like(x[:, :1], -1), x[:, :-1]], 1) * V0 + x
        K = self.tg_keys.numel()
        at = torch.searchsorted(self.tg_keys, pair).clamp(max=K - 1)
        known = (self.tg_keys[at] == pair)[..., None]
        cand = torch.where(known, self.tg_tri_idx[at], self.tg_bi_idx[word])
        val = torch.where(known, self.tg_tri_val[at].float() * self.tg_a[1], self.tg_bi_val[word].float() * self.tg_a[0])
        return cand, val

    def _phr4_idx(self, x):
        V = self.phr_V
        p1 = torch.cat([torch.full_like(x[:, :1], -1), x[:, :-1]], 1)
        p2 = torch.cat([torch.full_like(x[:, :2], -1), x[:, :-2]], 1)
        ctx = (p2 * V + p1) * V + x
        K = self.phr4_keys.numel()
        pos = torch.searchsorted(self.phr4_keys, ctx).clamp(max=K - 1)
        return torch.where(self.phr4_keys[pos] == ctx, pos, torch.full_like(pos, K))

    def _phr_surp(self, x):
        """Surprise from the phrasebook: lse[prev] - (c·Ê[prev]·H[cur] + logp[cur]) (full2.py:1479-1488)."""
        B, T = x.shape
        s_ = torch.full((B, T), 1e4, device=x.device)
        xp, xc = x[:, :-1], x[:, 1:]
        n = self.sp_lse.numel()
        ok = (xp < n) & (xc < n)
        xp, xc = xp.clamp(max=n - 1), xc.clamp(max=n - 1)
        if (ops._ext.use_cuda(self.sp_E) and self.sp_E.dtype == self.sp_H.dtype and self.sp_E.shape[1] % 4 == 0
                and self.sp_E.is_contiguous() and self.sp_H.is_contiguous()):
            ops._ext.count()                          # one gather-dot kernel instead of two row gathers, a product and a sum
            lo = ops._ext.C().table_pair_dot(self.sp_E, self.sp_H, xp.contiguous(), xc.contiguous()) + self.sp_lp[xc]
        else:
            lo = (self.sp_E[xp].float() * self.sp_H[xc].float()).sum(-1) + self.sp_lp[xc]
        s_[:, 1:] = torch.where(ok, self.sp_lse[xp] - lo, torch.full_like(lo, 1e4))
        return s_

    def _locks_raw(self, x):
        lb = self.lock_bucket if hasattr(self, "lock_w") else None
        return ops.find_locks(x, self.vocab, 3 if lb is not None else 2, lb)

    @torch.no_grad()
    def prep(self, x):
        """Everything that depends on tokens only, not on weights; computed ahead for the next batch."""
        p = {}
        if hasattr(self, "phr"):
            p["phr"] = self._phr_idx(x)
        if hasattr(self, "phr4"):
            p["phr4"] = self._phr4_idx(x)
        if hasattr(self, "ind_a"):
            p["ind_cand"], p["ind_on"], p["ind_bk"], p["ind_src"] = self._locks_raw(x)
        if hasattr(self, "sp_lse"):
            p["surp"] = self._phr_surp(x)
        return p

    def host_prep(self):
        """A stand-in that computes `prep` on the CPU (for the data loader's worker thread): copies of the token-only
        tables on the host and the same functions.  What it returns is moved to the device with the batch, so the
        step itself finds no lock, phrase index or phrase surprise left to compute (the reference's `CpuFeeder`,
        fastloop.py:108-139)."""
        return _HostPrep(self)

    @torch.no_grad()
    def table_rows(self, x):
        if self._vp is not None:                         # row-sharded tables: the rows of all ranks' tokens move
            return {}
        rows = {id(self.emb.weight): x.reshape(-1)}
        if hasattr(self, "phr"):
            rows[id(self.phr.weight)] = self._phr_idx(x).reshape(-1)
        if hasattr(self, "phr4"):
            rows[id(self.phr4.weight)] = self._phr4_idx(x).reshape(-1)
        return rows

    # ------------------------------------------------------------------------------------------ vocabulary parallel
    def vocab_shard(self, rank, world, group=None):
        """Vocabulary parallelism (the JAX port's `VocabShard`, memarch_jax/memarch_jax/dist.py:106-187): keep rows
        [rank V/W, (rank+1) V/W) of the input table, of the output head and of the light head's output table.  Every
        rank serves its rows for the tokens of all ranks (`parallel/vocab.py`); the losses are computed per token of
        the rank's own rows, so everything built on them (pointer mixture, auxiliary terms) is unchanged.  The shards
        are rank-local parameters whose gradient sums over all ranks' tokens: a hook divides it by W.
        Not combined with: the short-vocabulary head, the frequency bias, the tongue tables, the needle terms."""
        from ..parallel import vocab as vp
        if self.short_v or hasattr(self, "head_bias") or hasattr(self, "tg_a"):
            raise NotImplementedError("vocabulary parallelism: short-vocabulary head / head bias / tongue tables are not sharded")
        assert self.vocab % world == 0, "vocabulary rows must divide by the world size"
        self._vp = (rank, world, group, rank * (self.vocab // world))
        for mod in (self.emb, self.head, self.l_head[1]):
            shard = nn.Parameter(vp.shard_rows(mod.weight.detach(), rank, world)[0])
            shard._ep_local = True
            shard._vocab_table = mod.weight.shape[0] >= 10000     # stays a word table for the optimizer, whatever its slice
            shard.register_hook(lambda g, w=world: g / w)
            mod.weight = shard
        return self

    def _emb_rows(self, ids):
        if self._vp is None:
            return self.emb(ids)
        from ..parallel import vocab as vp
        return vp.take_dp(self.emb.weight, ids, self._vp[3], self._vp[2])

    def _nll_vp(self, h, w, y):
        """Per-token -log softmax(h W^T)[y] against a row-sharded table: (B,T)."""
        from ..parallel import vocab as vp
        return vp.nll_dp(h.reshape(-1, h.shape[-1]).float(), w.float(), y.reshape(-1), self._vp[3], self._vp[2]).view_as(y)

    # ------------------------------------------------------------------------------------------ forward
    def _run(self, blk, *a, heavy=False):
        k = self.cfg.ckpt
        on = k == "1" or (k == "heavy" and heavy) or (k == "light" and not heavy)
        if on and self.training and torch.is_grad_enabled():
            return checkpoint(blk, *a, use_reentrant=False)
        return blk(*a)

    def forward(self, x, prep=None):
        c = self.cfg
        B, T = x.shape
        win = self.window if T > self.window else None
        # on the GPU the token row, the gated candidate rows (INDUCT_IN) and the phrase row are summed by one kernel
        # further down; `h` stays None until then
        fuse_in = not c.resid_bf16 and ops._ext.use_cuda(self.emb.weight) and self._vp is None
        h = None if fuse_in else self._emb_rows(x)
        if c.resid_bf16 and x.is_cuda:
            h = h.to(torch.bfloat16)
        in_cand = in_sel = None
        self._tongue = self._mix = None
        if hasattr(self, "ind_a"):
            cand, votes, on, bk = self._lock_votes(x, prep)
            self._tongue = (cand, votes)
            if hasattr(self, "mix_w"):
                self._mix = self._mix_gate(cand, on, bk)
            self.stats["trust"] = (self.lock_w if hasattr(self, "lock_w") else self.ind_a).detach().float().mean()
            if c.induct_in:
                # the words the locks point at also enter the input, each through its own learned gate
                hd = torch.float32 if h is None else h.dtype
                sel = (votes != 0).to(hd) * torch.sigmoid(self.ind_in_g[:cand.shape[-1]]).to(hd)[None, None]
                if h is None:
                    in_cand, in_sel = cand, sel
                else:
                    h = h + (self._emb_rows(cand) * sel[..., None]).sum(2).type_as(h)
        if hasattr(self, "tg_a"):
            self._tongue = self._tongue_from_tables(x)
        if h is None:
            pidx = (prep["phr"] if prep and "phr" in prep else self._phr_idx(x)) if hasattr(self, "phr") else None
            h = ops.embed_sum(self.emb.weight, x, in_cand, in_sel, self.phr.weight if pidx is not None else None, pidx)
        elif hasattr(self, "phr"):
            h = h + self.phr(prep["phr"] if prep and "phr" in prep else self._phr_idx(x)).type_as(h)
        if hasattr(self, "phr4"):
            h = h + self.phr4(prep["phr4"] if prep and "phr4" in prep else self._phr4_idx(x)).type_as(h)
        if hasattr(self, "skip"):
            for t, o in zip(self.skip, self.skip_o):
                xs = torch.cat([x[:, :1].expand(-1, o - 1), x[:, :-(o - 1)]], 1)
                m = (torch.arange(T, device=x.device) >= o - 1).to(h.dtype)[None, :, None]
                h = h + t(xs).type_as(h) * m
        if c.prev_in:                                  # the word knows the word before it (as a two-word lock would)
            e0 = self._emb_rows(x).type_as(h)
            h = h + torch.sigmoid(self.prev_g).type_as(h) * torch.cat([torch.zeros_like(e0[:, :1]), e0[:, :-1]], 1)
        if hasattr(self, "smear"):
            h = torch.cat([h[:, :1], h[:, 1:] + torch.sigmoid(self.smear(h[:, 1:])) * h[:, :-1]], 1)
        lights = list(self.light_a) + list(self.light_b)
        if hasattr(self, "ent_t"):
            n = self.ent_t.numel()
            ent = self.ent_t[x.clamp(max=n - 1)]
            K = max(16, int(T * c.opaque) // 16 * 16)
            op = ent > c.opaque_thr
            keep = op & (op.cumsum(1) <= K)
            sidx = ((~keep).long() * T + torch.arange(T, device=x.device)).argsort(dim=-1, stable=True)[:, :K]
            sel = (sidx, keep.gather(1, sidx))
            for b in lights + list(self.final):
                b.cur_sel = sel
            self.stats["opaque"] = keep.float().mean()
        if "ve" in c.blk or "x0" in c.blk:
            for i, b in enumerate(lights):
                b.cur_ve = self.ve[i](x) if "ve" in c.blk else None
                b.cur_x0 = h if "x0" in c.blk else None
        h = run_blocks(self.light_a, h, win, self._run)
        h_a = h if (c.uroboros and c.uroboros_at == "light_a") else None

        seg = min(self.seg, T)
        snaps = None
        if not c.no_mem:
            reads, snaps, st = self._memory_pass(h, seg)
            self.last_mem = (snaps, st)
            h = h + reads.type_as(h)
            self.stats["mem_cards"] = st["valid"].float().sum(1).mean()

        if c.rope_mem:
            h = self._tether_pass(h, x, win)
        else:
            h = run_blocks(self.light_b, h, win, self._run)
        lh = ops.rmsnorm(h, self.l_norm.weight, self.l_norm.eps)

        if hasattr(self, "fish"):
            return self._tail(self._fish_pass(h, lh, prep), lh, x, snaps, seg, win)

        # surprise -> anchors: the light part's own prediction error decides where to think hard
        with torch.no_grad():
            if hasattr(self, "sp_lse"):
                s_ = prep["surp"] if prep and "surp" in prep else self._phr_surp(x)
            else:
                s_ = self._light_surprise(lh.detach(), x)
            self._surp = s_
            A = max(1, round(T * self.cap))
            if not c.uroboros:
                idx, valid = ops.select_anchors(s_, self.tau, A)    # this step's threshold is the one before its update
                if self.training:
                    self.tau.mul_(0.9).add_(0.1 * ref.tau_quantile(s_, self.frac))
                self.stats["anchors"] = valid.float().mean() * A / T
        self._hoop = None
        if c.uroboros:
            # the model predicts its own error before the heavy layers and hands them only the words it has not
            # "eaten" (memarch_jax/memarch_jax/model.py:364-378 of the reference's JAX port)
            feat = lh if h_a is None else ops.rmsnorm(h_a, self.l_norm.weight, self.l_norm.eps)
            pred = self.hoop.predict(feat, s_)
            with torch.no_grad():
                if c.uroboros_thr >= 0:                  # per word, no ranking over the sequence: causal
                    idx = torch.arange(T, device=x.device).expand(B, T).contiguous()
                    valid = pred > c.uroboros_thr
                    valid[:, 0] = True
                else:
                    idx, valid = self.hoop.select(pred, self.hoop_budget)
                self.stats["anchors"] = valid.float().mean() * idx.shape[1] / T
            self._hoop = (pred, idx)
            s_, A = pred.detach(), idx.shape[1]          # what the heavy layers see as the words' surprise

        h, a = self.heavy_pass(h, idx, valid, s_, self._full_layer(prep))
        if self.n_draft:
            an = self.draft_norm(a)
            self._drafts = []
            d = h.shape[-1]
            for j, lin in enumerate(self.draft, 1):
                pj = idx + j
                okj = valid & (pj < T)
                dj = lin(an)
                self._drafts.append((dj, pj.clamp(max=T - 1), okj))
                h = ops.scatter_back(h, pj.clamp(max=T - 1), dj * okj[..., None])
        if self.moe and c.layer_stats:
            self.stats["moe_fill"] = sum(b.fill_now for b in self.heavy) / len(self.heavy)
            self.stats["moe_drop_l"] = torch.stack([torch.as_tensor(b.dropped, dtype=torch.float32, device=h.device) for b in self.heavy])
            self.stats["moe_active_l"] = torch.stack([b.active_now for b in self.heavy])
        if self.moe:
            self.stats["moe_drop"] = sum(b.dropped for b in self.heavy) / len(self.heavy)
            if self.heavy[0].wave:
                L = len(self.heavy)
                self.stats["learned"] = sum(b.learned.float().mean() for b in self.heavy) / L
                self.stats["hint"] = sum(b.hint_avg[0] for b in self.heavy) / L
                self.stats["err_r"] = sum((b.err / b.err_peak.clamp(min=1e-12)).min() for b in self.heavy) / L
                if self.heavy[0].wave == "still":
                    self.stats["move_r"] = sum((b.last_move / b.move_peak.clamp(min=1e-12)).min() for b in self.heavy) / L

        return self._tail(h, lh, x, snaps, seg, win)

    def heavy_pass(self, h, idx, valid, s_, full=None):
        """The heavy layers on the anchors `idx` (B,A; `valid` marks the real ones), `s_` (B,T) the words' surprise.
        `full`: None - anchors only; k - layer k works on ALL words in this step; -1 - every layer does.  A "full" layer:
        the anchors' states are written into the stream, the layer runs over every word (all places real: fill 1),
        the anchors are read back; the order of the layers does not change (memarch_jax/memarch_jax/moe.py:298-354 of
        the reference's JAX port).  Returns (stream, anchor states)."""
        c = self.cfg
        A = idx.shape[1]
        a_in = ops.gather_tokens(h, idx)
        a = a_in
        sa = None
        if self.moe:
            sa = torch.where(valid, s_.gather(1, idx).clamp(0, 50), torch.full_like(s_[:, :A], -1.0))
        ctx = h.detach() if c.heavy_attn_detach else h
        if full is None:
            for li, b in enumerate(self.heavy):
                if hasattr(self, "h_attn"):
                    a = self.h_attn[li](a, ctx, idx)
                a = self._run(b, a, sa, heavy=True)
            return ops.scatter_back(h, idx, (a - a_in) * valid[..., None]), a
        gi = idx[..., None].expand(-1, -1, h.shape[-1])
        put = lambda hh, a_: hh.scatter(1, gi, torch.where(valid[..., None], a_.to(hh.dtype), hh.gather(1, gi)))
        s_all = s_.clamp(0, 50) if self.moe else None
        hh = h
        for li, b in enumerate(self.heavy):
            if hasattr(self, "h_attn"):
                a = self.h_attn[li](a, ctx, idx)
            if full < 0 or full == li:
                fill, b.fill = b.fill, 1.0
                hh = self._run(b, put(hh, a), s_all, heavy=True)
                b.fill = fill
                a = hh.gather(1, gi)
            else:
                a = self._run(b, a, sa, heavy=True)
        return put(hh, a), a

    def graph_key(self):
        """Host-side state that decides what a step launches (a captured step is only valid for the same values)."""
        return (self._hfull if self.cfg.heavy_rotate else None, getattr(self, "hoop_budget", None))

    def _full_layer(self, prep):
        """None: every heavy layer on the anchors.  -1: every layer on all words (`heavy_all`).  k: layer k on all
        words in this step - from `prep["hfull"]`, or by rotation over the steps (`heavy_rotate`, set by `before_step`)."""
        c = self.cfg
        if c.heavy_all:
            return -1
        if not c.heavy_rotate or not self.training:
            return None
        k = int(prep["hfull"].reshape(-1)[0]) if isinstance(prep, dict) and "hfull" in prep else self._hfull
        return k if 0 <= k < len(self.heavy) else None

    def _fish_pass(self, h, lh, prep):
        """The layer pool instead of anchors + heavy layers (memarch_jax/memarch_jax/model.py:339-363 of the reference's
        JAX port).  Training: the whole step is one kind of text (`prep["kind"]`) and every row runs through the step's
        combination of layers (`prep["fish"]`); a small router learns to tell the kind from the light state.  Finished
        model (`fish_eval`, or no combination given): the router picks each row's kind and the row runs that kind's
        whole set, or a fixed subset of `fish_eval_c` layers of it."""
        c = self.cfg
        kind = prep.get("kind") if isinstance(prep, dict) else None
        self._fish_aux = None
        if kind is not None:
            ce, acc, logits = self.fish.router_loss(lh, kind.reshape(-1).long())
            self._fish_aux = ce
            self.stats["fish_router_acc"] = acc.detach()
        else:
            logits = self.fish.router(lh.detach().float().mean(1))
        order = prep.get("fish") if isinstance(prep, dict) else None
        if c.fish_eval or order is None:
            kinds = logits.argmax(-1)
            out = torch.zeros_like(h)
            for k, pool in enumerate(self.fish.sets):
                if 0 < c.fish_eval_c < len(pool):
                    import numpy as np
                    pool = [int(v) for v in np.random.default_rng(1000 + k).permutation(pool)[:c.fish_eval_c]]
                out = out + torch.where((kinds == k)[:, None, None], self.fish(h, pool), torch.zeros_like(h))
            return out
        return self.fish(h, [int(i) for i in order.reshape(-1, order.shape[-1])[0].tolist()])

    def _tail(self, h, lh, x, snaps, seg, win):
        c = self.cfg
        h = run_blocks(self.final, h, win, self._run)

        dt = _cdt(h)
        cost = torch.zeros((), device=x.device)
        if not (c.no_mem or c.no_reread):
            o, cost = self._reread_pass(h, x, snaps, seg)
            h = h + o.type_as(h)
        if self.want_stream_mean:                     # for the optimizer's rules on the stream's common vector
            self.stats["stream_mean"] = h.detach().float().mean((0, 1))
        if c.norm_dump_proj:                          # the common vector is taken out whatever channel it sits in
            from ..ops.extras import dump_proof_norm
            hn = dump_proof_norm(h, self.norm.weight, self.stream_u, self.norm.eps or 1e-6).to(dt)
        else:
            hn = ops.rmsnorm(h, self.norm.weight, self.norm.eps, out_dtype=dt)
        if c.safe_norm_ratio > 0:
            from ..ops.extras import cap_shared
            hn = cap_shared(hn, c.safe_norm_ratio, c.safe_norm_t0)
        return (hn, lh), cost

    def _tether_pass(self, h, x, win):
        """The light blocks after the memory point with the anchor-routed read instead of plain attention
        (memarch_jax/memarch_jax/model.py:266-324 of the reference's JAX port).  Anchors are the words that surprise
        the light head after the first light blocks; the threshold follows the quantile of that surprise (updated
        first, then used, frozen in evaluation)."""
        from .rope_memory import RopeCfg, anchors_from_surprise
        c = self.cfg
        B, T = x.shape
        with torch.no_grad():
            sr = self._light_surprise(ops.rmsnorm(h, self.l_norm.weight, self.l_norm.eps).detach(), x)
            if self.training:
                self.rope_tau.mul_(0.9).add_(0.1 * ref.tau_quantile(sr, c.rope_frac or self.frac))
            A = max(1, round(T * (c.rope_cap or self.cap)))
            own, apos, avalid = anchors_from_surprise(sr.clone(), self.rope_tau, A, top=c.rope_anchor_top)
            self.stats["rope_anchors"] = avalid.float().sum(1).mean() / T
            if c.rope_key_diag:                   # needle keys among the links the search sees / among the anchors
                is_key = (x >= c.remind_tok0) & (x < c.remind_tok0 + 512)
                a_of = apos.gather(1, own.clamp(0, apos.shape[1] - 1))
                t = torch.arange(T, device=x.device)[None]
                n = is_key.float().sum().clamp(min=1.0)
                self.stats["rope_key_link"] = (is_key & (own >= 0) & (t - a_of < c.rope_links)).float().sum() / n
                self.stats["rope_key_anch"] = (is_key & (own >= 0) & (t == a_of)).float().sum() / n
            docs = (x == c.rope_doc_eos).long().cumsum(1) if c.rope_doc_eos >= 0 else None
            qmask = None
            if c.rope_qfrac < 1.0:                # only the surprised words read the tether
                if self.training:
                    self.rope_qtau.mul_(0.9).add_(0.1 * ref.tau_quantile(sr, c.rope_qfrac))
                qmask = sr >= self.rope_qtau
                self.stats["rope_qfrac_real"] = qmask.float().mean()
        rcfg = RopeCfg(K=c.rope_k, links=c.rope_links, win=c.rope_win, span_cap=c.rope_span_cap, route=c.rope_route,
                       G=c.rope_hier_g, NB=c.rope_hier_nb, BM=c.rope_hier_bm, excl_win=c.rope_excl_win, rgrad=c.rope_rgrad,
                       chunk=c.rope_chunk, mgrad=c.remind_use_w > 0, route_bf16=c.rope_route_bf16)
        pending, routed, masses = None, None, []
        for bi, b in enumerate(self.light_b):
            if c.rope_layers and bi >= c.rope_layers:
                h, pending = self._run(b, h, win, pending, True)
                continue
            # the read recomputes its own chunks, so the block is not wrapped in another checkpoint
            h, pending = b(h, win, pending, True, (own, apos, avalid, rcfg, routed, qmask, docs))
            share, route, mass = b.tether_out
            masses.append(mass)
            routed = route if c.rope_share_route else None
            if bi == 0:
                self.stats["rope_share"] = share
        self._tether_mass = sum(masses) / len(masses) if masses else None
        return h if pending is None else ops.resid_add(h, pending)

    def _light_surprise(self, lhd, x):
        """lse - logit[target] of the light head for every position but the last (full2.py:1650-1667)."""
        B, T = x.shape
        s_ = torch.full((B, T), 1e4, device=x.device)
        w0, W2 = self.l_head[0].weight, self.l_head[1].weight
        if self._vp is not None:
            s_[:, 1:] = self._nll_vp(ops.linear(lhd[:, :-1], w0), W2, x[:, 1:])
            return s_
        ch = self.cfg.ce_chunk
        for j in range(0, T - 1, 8192):
            hj = lhd[:, j:min(j + 8192, T - 1)]
            tgt = x[:, j + 1:j + 1 + hj.shape[1]]
            h128 = ops.linear(hj, w0)
            if ch:
                lse, ly = ref.chunk_lse(h128.reshape(-1, h128.shape[-1]), W2, None, tgt.reshape(-1), ch)
                s_[:, j + 1:j + 1 + hj.shape[1]] = (lse - ly).view(B, -1)
            else:
                lo = ops.linear(h128, W2).float()
                s_[:, j + 1:j + 1 + hj.shape[1]] = torch.logsumexp(lo, -1) - lo.gather(-1, tgt[..., None]).squeeze(-1)
        return s_

    # ------------------------------------------------------------------------------------------ memory / reread
    def _seg_step(self, hs, st, s0):
        r, w = self.memory.read(hs, st)
        if not self.use_memory:
            r, w = r * 0, w * 0
        snap = (st["faces"], self.memory.contents(st), st["pos"], st["valid"])
        qpos = (s0 + torch.arange(hs.shape[1], device=hs.device)).expand(hs.shape[0], -1)
        st = self.memory.write(hs + r, qpos, st, now=float(s0 + hs.shape[1]), w_read=w)
        return r, snap, st

    def _memory_pass(self, h, seg):
        """Segments of `seg` words: segment k reads the state left by segments < k, then writes
        (full2.py:1746-1767).  State is re-created empty on every call: texts of a batch are separate documents."""
        B, T, _ = h.shape
        st = self.memory.init_state(B, h.device, torch.float32)
        reads, snaps = [], []
        for s in range(0, T, seg):
            r, snap, st = self._seg_step(h[:, s:s + seg].float(), st, s)
            reads.append(r)
            snaps.append(snap)
        return torch.cat(reads, 1), snaps, st

    def _reread_pass(self, h, x, snaps, seg):
        """Re-reading for all segments as one batch (full2.py:1820-1840).  The batch is segment-major: row j * B + b
        is segment j of text b, and it reads the memory as it stood BEFORE that segment (snapshot j)."""
        B, T, d = h.shape
        n = len(snaps)
        seg_major = lambda t: t.unflatten(1, (n, seg)).transpose(0, 1).flatten(0, 1)           # (B, n*seg, ..) -> (n*B, seg, ..)
        words = seg_major(F.pad(h.float(), (0, 0, 0, n * seg - T)))
        faces, contents, pos, valid = (torch.stack(part).flatten(0, 1) for part in zip(*snaps))
        where = torch.arange(n * seg, device=h.device).view(n, 1, seg).expand(n, B, seg).flatten(0, 1)
        text = torch.arange(B, device=h.device).repeat(n)
        book = (x.contiguous(), self.book.weight, faces, contents, pos, valid)
        surp = self._surp if self.cfg.reread_anch else None
        if surp is None:
            o, cost = self.reread(words, *book, where, text)
        else:
            # only the most surprising words of every segment re-read (full2.py:1794-1808); the rest get nothing
            k = max(1, int(round(seg * self.cfg.reread_anch)))
            rank = seg_major(F.pad(surp.float(), (0, n * seg - T), value=-1e9))
            chosen = rank.topk(k, -1).indices.sort(-1).values                                     # (n*B, k) in text order
            at = chosen[..., None].expand(-1, -1, d)
            o_k, cost = self.reread(words.gather(1, at), *book, where.gather(1, chosen), text)
            o = torch.zeros(n * B, seg, d, dtype=o_k.dtype, device=h.device).scatter(1, at, o_k)
        if not self.use_memory:
            o, cost = o * 0, cost * 0
        return o.unflatten(0, (n, B)).transpose(0, 1).flatten(1, 2)[:, :T], cost

    # ------------------------------------------------------------------------------------------ loss
    def _head_w(self, hn):
        """Output table; with head_bias the word frequency rides as one extra input dimension (padded to 16)."""
        if not hasattr(self, "head_bias"):
            return hn, self.head.weight
        V = self.head.weight.shape[0]
        hn = torch.cat([hn, torch.ones_like(hn[..., :1]), torch.zeros_like(hn[..., :15])], -1)
        w = torch.cat([self.head.weight, self.head_bias[:, None].to(self.head.weight.dtype),
                       self.head.weight.new_zeros(V, 15)], 1)
        return hn, w

    def _fused_ce(self, hn, y):
        hn, w = self._head_w(hn)
        if self._mix is not None:
            c1, g = self._mix
            return ops.linear_ce(hn, w, y, gate=g, hit=(c1 == y).float())
        if self._tongue is not None:
            cand, val = self._tongue
            return ops.linear_ce(hn, w, y, cand=cand, cval=val)
        return ops.linear_ce(hn, w, y)

    def _logits(self, hn):
        if self._vp is not None:
            raise NotImplementedError("full logits are not formed under vocabulary parallelism")
        lo = ops.linear(hn, self.head.weight).float()
        if hasattr(self, "head_bias"):
            lo = lo + self.head_bias.float()
        return lo

    def _ce_tok(self, hn, y):
        lo = self._logits(hn)
        return F.cross_entropy(lo.reshape(-1, lo.shape[-1]), y.reshape(-1), reduction="none")

    def _short_rows(self):
        """Rows and biases of the first level: the `short_v` frequent words followed by one "rare" bucket row (a word of
        the vocabulary lends its output vector; its bias is the log share of rare words, or zero with a trained bias)."""
        W, b = self.head.weight, getattr(self, "head_bias", None)
        rows = torch.cat([W[self.sv_ids], W[self.sv_bucket:self.sv_bucket + 1]])
        if b is not None:
            bias = torch.cat([b[self.sv_ids].float(), b.new_full((1,), self.sv_prior1, dtype=torch.float32)])
        else:
            bias = torch.cat([W.new_zeros(self.short_v, dtype=torch.float32), W.new_full((1,), self.sv_prior0, dtype=torch.float32)])
        return rows, bias

    def _short_logp(self, h, y):
        """log P(y) of the two-level head: every position pays the small softmax over frequent words + the rare bucket;
        positions whose target is rare add the log-probability inside the bucket, computed over the full vocabulary
        with the frequent words masked out - but only for the first `rare_cap` share of positions (static shape), the
        rest of the rare targets keep the bucket's probability alone and are counted in `rare_drop`.
        (full2.py:1875-1898)"""
        N, K = h.shape[0], self.short_v
        chunk = self.cfg.ce_chunk or 16768
        rows, bias = self._short_rows()
        level1 = self.sv_pos[y]                                      # index among the frequent words, K = rare
        lse1, hit1 = ops.chunk_ce(h, rows, bias, level1, min(chunk, K + 1))
        logp = hit1 - lse1
        rare = level1 == K
        # the rare positions first (in text order), padded with frequent ones up to the static capacity
        cap = min(N, -(-int(round(self.rare_cap * N)) // 256) * 256)
        rank = rare.float() * 2 - torch.arange(N, device=h.device, dtype=torch.float32) / N
        take = rank.detach().topk(cap).indices
        served = rare[take]
        b = getattr(self, "head_bias", None)
        inside = (b.float() if b is not None else self.head.weight.new_zeros(self.head.weight.shape[0], dtype=torch.float32)) + self.sv_mask
        lse2, hit2 = ops.chunk_ce(h[take], self.head.weight, inside, y[take], chunk)
        logp = logp.index_add(0, take, torch.where(served, hit2 - lse2, torch.zeros_like(hit2)))
        self.stats["rare_drop"] = (rare.sum() - served.sum()).float() / N
        return logp

    @torch.no_grad()
    def short_top(self, h):
        """Most probable word of the short vocabulary and its probability, without gradient: h (N, d) ->
        (p_top (N,) fp32, token (N,) in the full vocabulary).  The "rare" bucket counts in the normaliser but cannot
        lead (memarch_jax/memarch_jax/ce.py:337-363)."""
        W, K = self.head.weight, self.short_v
        Ws = torch.cat([W[self.sv_ids], W[self.sv_bucket:self.sv_bucket + 1]])
        lo = ops.linear(h.detach(), Ws.detach()).float()
        lo[:, K] += self.sv_prior0
        lse = lo.logsumexp(-1)
        best, j = lo[:, :K].max(-1)
        return (best - lse).exp(), self.sv_ids[j]

    def _nll_tok(self, hn, y, j):
        """Per-token -log P(y) of positions j.. of the rows (pointer mixture and tongue included)."""
        c = self.cfg
        mix = self._mix
        tongue = self._tongue if mix is None else None
        B_, T_ = y.shape
        if self._vp is not None:
            if tongue is not None:
                raise NotImplementedError("vocabulary parallelism: lock votes added to the logits need the full row; use the pointer mixture")
            nll = self._nll_vp(hn, self.head.weight, y)
            lse, ly = nll, torch.zeros_like(nll)
        elif c.ce_chunk and tongue is None:
            if self.short_v:
                logp = self._short_logp(hn.reshape(B_ * T_, -1), y.reshape(-1)).view(B_, T_)
                lse, ly = torch.zeros_like(logp), logp
            else:
                lse, ly = ops.chunk_ce(hn.reshape(B_ * T_, -1), self.head.weight, getattr(self, "head_bias", None),
                                       y.reshape(-1), c.ce_chunk)
                lse, ly = lse.view(B_, T_), ly.view(B_, T_)
        else:
            lo = self._logits(hn)
            if tongue is not None:
                cand, val = tongue
                lo = lo.scatter_add(-1, cand[:, j:j + T_].long(), val[:, j:j + T_].float())
            lse = torch.logsumexp(lo, -1)
            ly = lo.gather(-1, y[..., None])[..., 0]
        if mix is not None:
            c1, g = mix
            c1, g = c1[:, j:j + T_], g[:, j:j + T_]
            py = (ly - lse).exp()
            return -torch.log(((1 - g) * py + g * (c1 == y).float()).clamp(min=1e-30))
        return lse - ly

    def _ce_part(self, hn, y, j):
        return self._nll_tok(hn, y, j).sum()

    # ------------------------------------------------------------------------------------------ instinct on words
    def _iw_part(self, hn, y, mult, j):
        """Sums over the positions j.. of the rows: [term, smeared, sure-but-wrong, fine, acted on] (term not yet
        divided by the number of words).  Probabilities are those of the full softmax of the head.
        (memarch_jax/memarch_jax/model.py:563-650 of the reference's JAX port)"""
        c = self.cfg
        lo = self._logits(hn)
        if self._mix is None and self._tongue is not None:
            cand, val = self._tongue
            lo = lo.scatter_add(-1, cand[:, j:j + y.shape[1]].long(), val[:, j:j + y.shape[1]].float())
        lsm = lo.log_softmax(-1)
        lp = lsm.gather(-1, y[..., None])[..., 0]
        ok = lp.detach().exp() >= c.iw_ok
        if c.iw_random:
            # the right word is known: +delta for it, -delta for ONE random other word per row; the rewritten answer
            # q = p + d (e_right - e_other) as a cross-entropy target gives the gradient d (e_other - e_right): two
            # words only, sum zero; d = min(delta, p_other), a word cannot give more than it has
            V = lo.shape[-1]
            h_ = (y.sum(1) * 2654435761 + 40503 * torch.arange(len(y), device=y.device)) % (self.short_v or V)
            other = self.sv_ids[h_] if self.short_v else h_
            lpo = lsm.gather(-1, other[:, None, None].expand(-1, y.shape[1], 1))[..., 0]
            act = ~ok & (other[:, None] != y)
            d_eff = lpo.detach().exp().clamp(max=c.iw_delta)
            term = mult * (d_eff * (lpo - lp) * act).sum()
            spread, cw = act, torch.zeros_like(act)
        elif c.iw_rewrite:
            # ... or for the top competitors of the right word, in proportion to what each of them has
            pk, ipk = lsm.detach().exp().topk(c.iw_k + 1, -1)
            rival = ipk != y[..., None]
            sel = rival & (rival.long().cumsum(-1) <= c.iw_k)
            pc = torch.where(sel, pk, torch.zeros_like(pk))
            S = pc.sum(-1)
            act = ~ok & (S > 0)
            d_eff = S.clamp(max=c.iw_delta)
            w = pc / S.clamp(min=1e-30)[..., None]
            d = (w * lsm.gather(-1, ipk)).sum(-1) - lp
            term = mult * (d_eff * d * act).sum()
            spread = ~ok & (pk[..., 0] < c.iw_spread)
            cw = ~ok & (pk[..., 0] > c.iw_cw) & (ipk[..., 0] != y)
        else:
            lpt, top = lsm.max(-1)
            p_top = lpt.detach().exp()
            spread = ~ok & (p_top < c.iw_spread)
            cw = ~ok & (p_top > c.iw_cw) & (top != y)
            act = spread | cw
            l_sp = (math.log(c.iw_target) - lp).clamp(min=0.0) * spread
            l_cw = (-torch.log1p(-lpt.exp().clamp(max=1 - 1e-6)) + math.log1p(-c.iw_cw)).clamp(min=0.0) * cw
            term = c.iw_spread_w * l_sp.sum() + c.iw_cw_w * mult * l_cw.sum()
        return torch.stack([term] + [t.float().sum() for t in (spread, cw, ok, act)])

    # ------------------------------------------------------------------------------------------ recall needles
    def _logp_rows(self, h, tok, add=None):
        """log P(tok[:, j]) under the output distribution at the states h (N,D), for every column j of tok (N,J)."""
        if self.short_v:
            return torch.stack([self._short_logp(h, tok[:, j]) for j in range(tok.shape[1])], 1)
        lo = self._logits(h[None])[0]
        if add is not None:
            lo = lo.scatter_add(-1, add[0].long(), add[1].float())
        return lo.log_softmax(-1).gather(1, tok)

    def remind_term(self, hn, y, extra):
        """Loss on the answers of recall needles (memarch_jax/memarch_jax/model.py:455-531 of the reference's JAX
        port).  `extra["rem"]` (B,T) marks the question keys, whose target is the value; the first `remind_cap`
        answers of a row are read (static shape, no host sync).  Sum of the answers' -log P over B * remind_q, or
        their mean with `remind_mean`.  `remind_cand`: the softmax runs over the 64 value tokens only, so the common
        part of their head rows gets no gradient.  `remind_strict` (with `extra["rem_vals"]`, the values of the row's
        facts): answers after the first wrong one of a row earn nothing (they could be had by elimination), and
        probability put on the row's other values is penalised.  Returns (term, statistics)."""
        c = self.cfg
        rem = extra["rem"] > 0
        B, T = y.shape
        Q = min(T, c.remind_cap or c.remind_q)
        order = rem.float() * (T - torch.arange(T, device=y.device, dtype=torch.float32))
        pos = order.topk(Q, 1).indices                                    # the first Q answers of each row, in order
        av = rem.gather(1, pos).float()
        h = hn.gather(1, pos[..., None].expand(B, Q, hn.shape[-1])).reshape(B * Q, -1)
        yq = y.gather(1, pos)
        v0 = c.remind_tok0 + 512
        vals = extra.get("rem_vals") if c.remind_strict else None
        tok = yq.reshape(-1, 1)
        if vals is not None:
            vals = vals.long()
            tok = torch.cat([tok, vals.clamp(min=0)[:, None, :].expand(B, Q, vals.shape[1]).reshape(B * Q, -1)], 1)
        add = None
        if self._mix is None and self._tongue is not None:
            add = tuple(t.gather(1, pos[..., None].expand(B, Q, t.shape[-1])).reshape(B * Q, -1) for t in self._tongue)
        rows = 2048

        def logp_of(h_, tok_, *add_):
            return self._logp_rows(h_, tok_, add_ or None)

        parts = []
        for r0 in range(0, B * Q, rows):
            a = (h[r0:r0 + rows], tok[r0:r0 + rows]) + (tuple(t[r0:r0 + rows] for t in add) if add else ())
            if B * Q > rows and torch.is_grad_enabled() and h.requires_grad:
                parts.append(checkpoint(logp_of, *a, use_reentrant=False))
            else:
                parts.append(logp_of(*a))
        logp = torch.cat(parts).float()                                   # (B*Q, 1 + n)
        if c.remind_cand:
            ids = torch.arange(v0, v0 + 64, device=y.device)
            lv = ops.linear(h[None], self.head.weight[ids])[0].float()
            if hasattr(self, "head_bias"):
                lv = lv + self.head_bias[ids].float()
            py = lv.log_softmax(-1).gather(1, (yq.reshape(-1, 1) - v0).clamp(0, 63))[:, 0].exp().view(B, Q)
        else:
            py = logp[:, 0].exp().view(B, Q)
        if self._mix is not None:
            c1, g = (t.gather(1, pos) for t in self._mix)
            py = (1 - g) * py + g * (c1 == yq).float()
        nll = -torch.log(py.clamp(min=1e-30))
        hit = (py > 0.5).float().detach()                                 # p(answer) > 0.5: the argmax is right
        den = float(B * c.remind_q)
        st = {"remind_hit": (hit * av).sum() / den, "remind_n": av.sum() / den}
        if c.remind_mean or c.remind_strict:                              # accuracy by question number within the row
            qn = av.cumsum(1) * av
            for k in range(1, 5):
                st[f"remind_hit_q{k}"] = (hit * (qn == k)).sum() / den
                st[f"remind_n_q{k}"] = (qn == k).float().sum() / den
        counted = av
        pen = None
        if vals is not None:
            wrong = av * (1.0 - hit)
            counted = av * ((wrong.cumsum(1) - wrong) < 0.5).float()
            st["remind_strict_keep"] = counted.sum() / av.sum().clamp(min=1.0)
            other = ((vals >= 0)[:, None, :] & (vals[:, None, :] != yq[..., None])).float()
            p_other = (logp[:, 1:].exp().view(B, Q, -1) * other).sum(-1)
            pen = (-torch.log((1.0 - p_other).clamp(min=1e-6)) * av).sum() / av.sum().clamp(min=1.0)
            st["remind_strict_pen"] = pen.detach()
            st["remind_strict_pother"] = ((p_other * av).sum() / av.sum().clamp(min=1.0)).detach()
        term = (nll * counted).sum() / den
        st["remind_nll"] = ((nll * av).sum() / den).detach()
        if c.remind_mean:
            term = term * (den / counted.sum().clamp(min=1.0))
        if pen is not None:
            term = term + c.remind_strict_w * pen
        return term, {k: v.detach() for k, v in st.items()}


    def train_loss(self, out, y, train=True, extra=None):
        """`extra`: what the data pipeline knows about recall needles in this batch - "rem" (B,T) marks the question
        keys, "rem_y" the true values where the text shows a blank, "rem_vals" the values of each row's facts."""
        c = self.cfg
        hn, lh = out
        rem = extra.get("rem") if isinstance(extra, dict) else None
        if rem is not None and "rem_y" in extra:          # the answer is not in the text, only in the target
            y = torch.where(rem > 0, extra["rem_y"].to(y.dtype), y)
        mask_main = rem is not None and c.remind_mask_main
        if mask_main or (train and self._hoop is not None):
            # the per-word form of the loss: the hoop's head needs the model's true error on every word as its target,
            # and the needle mask drops single words from the main loss
            parts = []
            for j in range(0, hn.shape[1], 8192):
                part = (hn[:, j:j + 8192], y[:, j:j + 8192])
                if self.training and torch.is_grad_enabled():
                    parts.append(checkpoint(self._nll_tok, *part, j, use_reentrant=False))
                else:
                    parts.append(self._nll_tok(*part, j))
            nll_tok = torch.cat(parts, 1)
            loss = nll_tok.sum()
            if mask_main:
                # in rows with needles the needle tokens (random keys, values, marker) do not teach the main loss: a
                # full softmax on them lifts the whole group of tokens everywhere in the text (model.py:437-446)
                k0 = c.remind_tok0
                keep = (~((y >= k0) & (y <= k0 + 576) & (rem > 0).any(1, keepdim=True))).float()
                self.stats["remind_main_masked"] = 1.0 - keep.mean()
                loss = (nll_tok * keep).sum()
        elif train and self.training and self.panic:
            loss = 0
            for j in range(0, hn.shape[1], 8192):
                ce = checkpoint(self._ce_tok, hn[:, j:j + 8192], y[:, j:j + 8192], use_reentrant=False)
                w = (ce / ce.mean()).detach().clamp(0.25, 4.0) ** self.panic
                loss = loss + (ce * (w / w.mean())).sum()
        elif c.fused_ce and self.training and not self.short_v and self._vp is None:
            loss = self._fused_ce(hn, y)
        else:
            loss = 0
            for j in range(0, hn.shape[1], 8192):
                part = (hn[:, j:j + 8192], y[:, j:j + 8192])
                if self.training and not c.ce_chunk and torch.is_grad_enabled():
                    loss = loss + checkpoint(self._ce_part, *part, j, use_reentrant=False)
                else:
                    loss = loss + self._ce_part(*part, j)
        loss = main = loss / y.numel()
        if train and self._hoop is not None:
            pred, hidx = self._hoop
            loss = loss + c.uroboros_w * self.hoop.loss(pred, nll_tok)
            self.stats.update(self.hoop.stats(pred, nll_tok, hidx, c.uroboros_eat))
        if rem is not None and (c.remind_w > 0 or c.remind_use_w > 0 or not train):
            term, st = self.remind_term(hn, y, extra)
            self.stats.update(st)
            if train:
                synth = bool(extra.get("synth", False)) if isinstance(extra, dict) else False
                loss = loss + (c.remind_w_synth if (synth and c.remind_w_synth >= 0) else c.remind_w) * term
                if c.remind_only:                         # stage one: the answers only (auxiliary terms stay)
                    loss = loss - main
            mass = getattr(self, "_tether_mass", None)
            if mass is not None:                          # how much of the questions' attention went down the tether
                mk, den = (rem > 0).float(), float(len(y) * c.remind_q)
                use = (mass.float() * mk).sum() / den
                self.stats["remind_rope_share"] = use.detach()
                if train and c.remind_use_w > 0:
                    loss = loss + c.remind_use_w * (mk.sum() / den - use)
        if train and c.inst_word:
            mult = extra.get("iw_mult", 1.0) if isinstance(extra, dict) else 1.0
            tot = 0
            for j in range(0, hn.shape[1], 2048):
                part = (hn[:, j:j + 2048], y[:, j:j + 2048], mult, j)
                tot = tot + (checkpoint(self._iw_part, *part, use_reentrant=False)
                             if self.training and torch.is_grad_enabled() else self._iw_part(*part))
            tot = tot / y.numel()
            loss = loss + tot[0]
            self.stats.update({"iw": tot[0].detach(), "iw_spread_frac": tot[1].detach(), "iw_cw_frac": tot[2].detach(),
                               "iw_ok_frac": tot[3].detach(), "iw_act_frac": tot[4].detach()})
        if train and c.hn_guard_w > 0:
            # hinge on the trunk after the final norm: nothing (value and gradient zero) while the row mean of hn and
            # the mean length of hn stay under their thresholds (memarch_jax/memarch_jax/model.py:539-551)
            h32 = hn.float()
            mn = (h32.mean(1).pow(2).sum(-1) + 1e-12).sqrt()
            ln = (h32.pow(2).sum(-1) + 1e-12).sqrt().mean(1)
            over = lambda v, thr: (v / thr - 1.0).clamp(min=0.0).pow(2).mean()
            self.stats["hn_mean"], self.stats["hn_len"] = mn.mean().detach(), ln.mean().detach()
            loss = loss + c.hn_guard_w * (over(mn, c.hn_guard_mean) + over(ln, c.hn_guard_len))
        if train and self._fish_aux is not None:
            loss = loss + 0.1 * self._fish_aux                   # the router's cross-entropy
        if train and self.moe:
            loss = loss + 0.01 * sum(b.aux for b in self.heavy) / len(self.heavy)
        if train and len(self.light_a) and hasattr(self.light_a[0], "moe"):
            lb = list(self.light_a) + list(self.light_b) + list(self.final)
            loss = loss + 0.01 * sum(b.moe.aux for b in lb) / len(lb)
        if train and self.n_draft and c.draft_loss:
            dl = 0
            for dj, pj, okj in self._drafts:
                tgt = y.gather(1, pj)
                lo = self._logits(ops.rmsnorm(dj, self.norm.weight, self.norm.eps))
                ce = F.cross_entropy(lo.reshape(-1, lo.shape[-1]), tgt.reshape(-1), reduction="none")
                dl = dl + (ce * okj.reshape(-1)).sum() / okj.sum().clamp(min=1)
            loss = loss + c.draft_loss * dl / len(self._drafts)
        if train and not hasattr(self, "sp_lse"):
            V = self.head.out_features
            h4, y4 = lh[:, ::4], y[:, ::4]
            h128 = ops.linear(h4, self.l_head[0].weight)
            if self._vp is not None:
                loss = loss + 0.3 * self._nll_vp(h128, self.l_head[1].weight, y4).mean()
            elif c.ce_chunk:
                lse, ly = ops.chunk_ce(h128.reshape(-1, h128.shape[-1]), self.l_head[1].weight, None, y4.reshape(-1),
                                       c.ce_chunk)
                loss = loss + 0.3 * (lse - ly).mean()
            else:
                lo = ops.linear(h128, self.l_head[1].weight).float()
                loss = loss + 0.3 * F.cross_entropy(lo.reshape(-1, V), y4.reshape(-1))
        return loss

    # ------------------------------------------------------------------------------------------ waves
    @torch.no_grad()
    def rebank(self, step, every=1000):
        """Every `every` steps move experts between banks in all layers at once; the only host read of the
        `learned` masks (full2.py:1932-1946)."""
        banks = [b for b in self.heavy if isinstance(b, AnchorMoE) and b.bank]
        if not banks or step == 0 or step % every:
            return []
        masks = torch.stack([b.learned for b in banks]).cpu().tolist()
        if not any(b.wants_rebank(mk) for b, mk in zip(banks, masks)):
            return []
        changes = []
        for b, mk in zip(banks, masks):
            changes += b.rebank(mk)
        self.stats["frozen"] = torch.tensor(sum(len(b.Fz) for b in banks) / sum(b.E for b in banks))
        return changes

    def before_step(self, step):
        c = self.cfg
        if c.heavy_rotate and len(self.heavy):
            k = max(1, c.heavy_full_every)
            self._hfull = (step // k) % len(self.heavy) if step % k == 0 else -1
        for b in self.heavy:
            if hasattr(b, "before_step"):
                b.before_step(step)


for _name in ("prep", "_phr_idx", "_phr4_idx", "_phr_surp", "_locks_raw"):
    setattr(_HostPrep, _name, getattr(MemArchLM, _name))
