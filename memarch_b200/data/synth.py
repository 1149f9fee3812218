"""Seeded synthetic token streams and the device-resident batch sampler.

Corpus: an order-1 Markov chain over the vocabulary.  Unigram marginal Zipf(alpha=1.1); every row of the transition
table has `n_succ` random successors (drawn from the marginal) with Dirichlet(0.3) weights; a share of positions
copy a token from earlier in the same text (so the keys-and-locks pointer and the anchors have something to find).
The long-context flavour plants copy *spans* of 8-64 tokens taken 1k-12k tokens back.

`TokenStore` keeps all tokens on the device and assembles batches there with a device generator, the way the
reference's `GPUData` does (fastloop.py:40-49); `HostFeeder` is the end-to-end path: batches are cut on the host into
pinned memory and copied to the device each step.
"""
from __future__ import annotations

import numpy as np
import torch


def zipf_probs(vocab, alpha=1.1):
    p = 1.0 / np.arange(1, vocab + 1, dtype=np.float64) ** alpha
    return p / p.sum()


class MarkovCorpus:
    def __init__(self, vocab=50257, n_succ=64, alpha=1.1, dirichlet=0.3, seed=0):
        rng = np.random.default_rng(seed)
        self.vocab, self.seed = vocab, seed
        self.marg = zipf_probs(vocab, alpha)
        perm = rng.permutation(vocab)                      # token id is not its frequency rank
        self.marg = self.marg[np.argsort(perm)]
        cdf = np.cumsum(self.marg)
        self.succ = np.searchsorted(cdf, rng.random((vocab, n_succ))).clip(0, vocab - 1).astype(np.int32)
        w = rng.gamma(dirichlet, 1.0, (vocab, n_succ)) + 1e-12
        self.cum = np.cumsum(w / w.sum(1, keepdims=True), 1).astype(np.float32)
        self.cum[:, -1] = 1.0
        self._cdf = cdf

    def texts(self, n_texts, length, copy_frac=0.10, seed=1, span=None, span_back=None):
        """(n_texts, length) int32.  `span=(lo, hi)` + `span_back=(lo, hi)` switch to copy spans."""
        rng = np.random.default_rng((self.seed, seed))
        out = np.empty((n_texts, length), dtype=np.int32)
        cur = np.searchsorted(self._cdf, rng.random(n_texts)).clip(0, self.vocab - 1).astype(np.int32)
        out[:, 0] = cur
        ar = np.arange(n_texts)
        for t in range(1, length):
            u = rng.random(n_texts, dtype=np.float32)
            j = (self.cum[cur] < u[:, None]).sum(1).clip(0, self.succ.shape[1] - 1)
            cur = self.succ[cur, j]
            out[:, t] = cur
        if span is None:
            m = rng.random((n_texts, length)) < copy_frac
            m[:, :2] = False
            src = (rng.random((n_texts, length)) * np.arange(length)[None]).astype(np.int64)
            # a copied position repeats the token that FOLLOWED an earlier occurrence of its predecessor's source,
            # i.e. out[t] = out[src+1] with out[t-1] forced to out[src]: the 1-gram lock fires and is right
            tt = np.nonzero(m)
            s = np.minimum(src[tt], tt[1] - 2).clip(0)
            out[tt[0], tt[1] - 1] = out[tt[0], s]
            out[tt] = out[tt[0], s + 1]
        else:
            n_spans = max(1, int(copy_frac * length / ((span[0] + span[1]) / 2)))
            for b in range(n_texts):
                for _ in range(n_spans):
                    L = int(rng.integers(span[0], span[1] + 1))
                    back = int(rng.integers(span_back[0], span_back[1] + 1))
                    dst = int(rng.integers(back + L, length - L)) if length - L > back + L else -1
                    if dst > 0:
                        out[b, dst:dst + L] = out[b, dst - back:dst - back + L]
        return out

    def stream(self, n_tokens, text_len=1024, **kw):
        n = -(-n_tokens // text_len)
        return self.texts(n, text_len, **kw).reshape(-1)[:n_tokens]


class TokenStore:
    """All tokens live on the device; `batch(B, T)` returns (B, T+1) int64 windows without host involvement."""

    def __init__(self, arr, seed, device):
        self.t = torch.from_numpy(np.asarray(arr, dtype=np.int32)).to(device)
        self.g = torch.Generator(device=device).manual_seed(seed)
        self.device = torch.device(device)

    def batch(self, B, T):
        start = torch.randint(0, len(self.t) - T - 1, (B,), device=self.device, generator=self.g)
        return self.t[start[:, None] + torch.arange(T + 1, device=self.device)].long()

    def state_dict(self):
        return {"gen": self.g.get_state()}

    def load_state_dict(self, sd):
        self.g.set_state(sd["gen"])


class HostFeeder:
    """Batches cut on the host into pinned buffers (double-buffered) and copied to the device on `stream`."""

    def __init__(self, arr, seed, device, B, T):
        self.arr = np.asarray(arr, dtype=np.int32)
        self.rng = np.random.default_rng(seed)
        self.B, self.T, self.device = B, T, torch.device(device)
        pin = self.device.type == "cuda"
        self.bufs = [torch.empty(B, T + 1, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self.i = 0
        self.bytes_per_batch = B * (T + 1) * 4

    def next(self):
        buf = self.bufs[self.i]
        self.i ^= 1
        idx = self.rng.integers(0, len(self.arr) - self.T - 1, self.B)
        view = buf.numpy()
        for r, s in enumerate(idx):
            view[r] = self.arr[s:s + self.T + 1]
        return buf.to(self.device, non_blocking=True).long()


def recall_batch(B, n_pairs=8, n_keys=64, n_vals=64, seed=None, device="cpu"):
    """Associative-recall toy task of the first prototypes (the reference's data.py:1-31): a text is `n_pairs`
    (key, value) pairs followed by a query key; the target at the last position is that key's value.
    Tokens: keys 0..n_keys-1, values n_keys..n_keys+n_vals-1, query marker = n_keys+n_vals.  Returns (x, y, mask)
    with y the next-token target and mask true only where the value must be recalled."""
    import torch
    g = torch.Generator().manual_seed(seed) if seed is not None else None
    keys = torch.stack([torch.randperm(n_keys, generator=g)[:n_pairs] for _ in range(B)])
    vals = torch.randint(0, n_vals, (B, n_pairs), generator=g) + n_keys
    which = torch.randint(0, n_pairs, (B,), generator=g)
    ar = torch.arange(B)
    pairs = torch.stack([keys, vals], -1).reshape(B, 2 * n_pairs)
    q = torch.full((B, 1), n_keys + n_vals)
    seq = torch.cat([pairs, q, keys[ar, which][:, None], vals[ar, which][:, None]], 1)
    x, y = seq[:, :-1], seq[:, 1:]
    mask = torch.zeros_like(y, dtype=torch.bool)
    mask[:, -1] = True
    return x.to(device), y.to(device), mask.to(device)
