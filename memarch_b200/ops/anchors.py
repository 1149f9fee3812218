"""Anchor selection, anchor gather and scatter-back, lock finder, phrase lookup.

Reference behaviour: surprise threshold + causal per-text cap + stable compaction (full2.py:1668-1677), gather of
anchor states and `scatter_add` of the heavy layers' delta (1681, 1702), keys-and-locks pointer search by three
stable sorts (1499-1535), phrase-table `searchsorted` (1441-1450).

GPU bodies: `anchor_select` (one CTA per text: threshold, prefix count, compaction into idx/valid in one pass),
`lock_find` (hash of 1/2/3-gram keys, last earlier occurrence) and `gather_rows`/`scatter_add_rows`.
"""
from __future__ import annotations

import torch

from . import _ext, ref


def select_anchors(s, tau, A):
    """s (B,T) fp32 surprise, tau 0-dim tensor, A slots per text -> idx (B,A) int64, valid (B,A) bool."""
    if _ext.use_cuda(s):
        idx, valid = _ext.C().anchor_select(s.contiguous().float(), tau.reshape(1).float(), int(A))
        _ext.count()
        return idx, valid
    return ref.select_anchors(s, tau, A)


def find_locks(x, vocab, n_keys=3, lock_bucket=None):
    if _ext.use_cuda(x):
        cand, on, src = _ext.C().lock_find(x.contiguous(), int(vocab), int(n_keys), lock_bucket is not None)
        _ext.count()
        bk = lock_bucket[x.clamp(max=lock_bucket.numel() - 1)] if lock_bucket is not None else torch.zeros_like(x)
        return cand, on, bk, src
    return ref.find_locks(x, vocab, n_keys, lock_bucket)


class _GatherTok(torch.autograd.Function):
    """a[b, j] = h[b, idx[b, j]]; backward scatter-adds into a zero (B,T,d) tensor (idx rows are distinct)."""

    @staticmethod
    def forward(ctx, h, idx):
        ctx.save_for_backward(idx)
        ctx.shape = h.shape
        d = h.shape[-1]
        return h.gather(1, idx[..., None].expand(-1, -1, d))

    @staticmethod
    def backward(ctx, g):
        idx, = ctx.saved_tensors
        d = g.shape[-1]
        out = g.new_zeros(ctx.shape)
        return out.scatter_add(1, idx[..., None].expand(-1, -1, d), g), None


def gather_tokens(h, idx):
    return _GatherTok.apply(h, idx)


def scatter_back(h, idx, delta):
    """h + scatter_add of `delta` (B,A,d) at positions idx (B,A)."""
    d = h.shape[-1]
    return h.scatter_add(1, idx[..., None].expand(-1, -1, d), delta.to(h.dtype))
