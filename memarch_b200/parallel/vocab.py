"""Vocabulary-parallel embedding and cross-entropy (the reference's JAX `VocabShard`, dist.py:106-187): the word
tables `emb`, `head`, `book` are row-sharded over the ranks; needed once the vocabulary is 131k and d is 2560, not for
the 50k recipe.

* `take(table_shard, ids)` — every rank looks up the ids that fall into its row range (others contribute zeros) and
  one all-reduce completes the rows; backward needs no collective: a rank's shard only receives the cotangent rows of
  its own range.
* `ce(h, head_shard, y)` — two-stage LSE: every rank computes logits against its vocabulary slice in row chunks,
  keeps the slice LSE and the correct-word logit if the target falls into the slice; one all-reduce of (max), one of
  (sum exp, correct logit) combine them.  Backward recomputes the chunk's logits and uses the *global* LSE, so the
  forward LSE and the backward probabilities see the same rounding (the consistency the reference's ce.py:23-57
  insists on).
* `take_dp` / `ce_dp` — the same with rank-local data (data parallel over the same ranks that shard the
  vocabulary, dist.py:106-151 of the reference): ids, states and targets of all ranks are gathered, every rank serves
  its rows / its vocabulary slice for all of them, and each rank keeps the rows of its own tokens; the loss returned
  is the sum over the tokens of all ranks, the same number everywhere.
Collectives are plain `torch.distributed` calls (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_rows(t, rank, world):
    n = -(-t.shape[0] // world)
    return t[rank * n:(rank + 1) * n].clone(), rank * n


class _Take(torch.autograd.Function):
    @staticmethod
    def forward(ctx, shard, ids, lo, group):
        n = shard.shape[0]
        local = ids - lo
        mine = (local >= 0) & (local < n)
        out = shard[local.clamp(0, n - 1)] * mine[..., None].to(shard.dtype)
        if dist.is_initialized():
            dist.all_reduce(out, group=group)
        ctx.save_for_backward(local, mine)
        ctx.n = n
        return out

    @staticmethod
    def backward(ctx, g):
        local, mine = ctx.saved_tensors
        gs = g.new_zeros(ctx.n, g.shape[-1])
        gs.index_add_(0, local[mine], g[mine])
        return gs, None, None, None


def take(shard, ids, lo, group=None):
    return _Take.apply(shard, ids, lo, group)


class _ShardCE(torch.autograd.Function):
    """Per row: global LSE − correct logit; h (N,d) replicated rows, head shard (Vs,d).  Returns (N,) fp32."""

    @staticmethod
    def forward(ctx, h, w, y, lo, group, chunk):
        N, Vs = h.shape[0], w.shape[0]
        m_loc = h.new_full((N,), -float("inf"), dtype=torch.float32)
        for i in range(0, N, chunk):
            m_loc[i:i + chunk] = (h[i:i + chunk] @ w.t()).float().amax(-1)
        m = m_loc.clone()
        if dist.is_initialized():
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        local = y - lo
        mine = (local >= 0) & (local < Vs)
        acc = torch.zeros(2, N, dtype=torch.float32, device=h.device)          # [sum exp, correct logit]
        for i in range(0, N, chunk):
            lo_ = (h[i:i + chunk] @ w.t()).float()
            acc[0, i:i + chunk] = (lo_ - m[i:i + chunk, None]).exp().sum(-1)
            j = local[i:i + chunk].clamp(0, Vs - 1)
            acc[1, i:i + chunk] = lo_.gather(-1, j[:, None]).squeeze(-1) * mine[i:i + chunk]
        if dist.is_initialized():
            dist.all_reduce(acc, group=group)
        lse = m + acc[0].log()
        ctx.save_for_backward(h, w, local, mine, lse)
        ctx.chunk, ctx.group = chunk, group
        return lse - acc[1]

    @staticmethod
    def backward(ctx, go):
        h, w, local, mine, lse = ctx.saved_tensors
        N, Vs = h.shape[0], w.shape[0]
        gh = torch.zeros_like(h, dtype=torch.float32)
        gw = torch.zeros_like(w, dtype=torch.float32)
        go = go.float()
        for i in range(0, N, ctx.chunk):
            hc = h[i:i + ctx.chunk]
            p = ((hc @ w.t()).float() - lse[i:i + ctx.chunk, None]).exp()
            rows = torch.arange(p.shape[0], device=h.device)[mine[i:i + ctx.chunk]]
            p[rows, local[i:i + ctx.chunk][mine[i:i + ctx.chunk]]] -= 1.0
            p = p * go[i:i + ctx.chunk, None]                                 # each row's own cotangent
            gh[i:i + ctx.chunk] = p @ w.float()
            gw += p.t() @ hc.float()
        if dist.is_initialized():
            dist.all_reduce(gh, group=ctx.group)                              # every slice contributes to dh
        return gh.to(h.dtype), gw.to(w.dtype), None, None, None, None


def nll(h, head_shard, y, lo, group=None, chunk=4096):
    """Per-token cross-entropy (N,) with the head sharded by vocabulary rows; h rows are the same on every rank."""
    return _ShardCE.apply(h.reshape(-1, h.shape[-1]), head_shard, y.reshape(-1), lo, group, chunk)


def ce(h, head_shard, y, lo, group=None, chunk=4096):
    """Summed token cross-entropy with the head sharded by vocabulary rows."""
    return nll(h, head_shard, y, lo, group, chunk).sum()


# ------------------------------------------------------------------------------------------------ rank-local data
def _world(group):
    return (dist.get_world_size(group), dist.get_rank(group)) if dist.is_initialized() else (1, 0)


def _gather(x, group):
    W, _ = _world(group)
    if W == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(W)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, 0)


class _AllRows(torch.autograd.Function):
    """Rows of this rank -> rows of all ranks (rank-major).  What consumes the result is computed identically on every
    rank and hands back a complete cotangent, so the backward only cuts out this rank's rows."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.n, ctx.rank = x.shape[0], _world(group)[1]
        return _gather(x, group)

    @staticmethod
    def backward(ctx, g):
        return g[ctx.rank * ctx.n:(ctx.rank + 1) * ctx.n], None


class _OwnRows(torch.autograd.Function):
    """Rows of all ranks -> rows of this rank; the backward gathers every rank's cotangent rows, because a table shard
    receives gradient from the tokens of all ranks."""

    @staticmethod
    def forward(ctx, x, group):
        W, r = _world(group)
        n = x.shape[0] // W
        ctx.group = group
        return x[r * n:(r + 1) * n]

    @staticmethod
    def backward(ctx, g):
        return _gather(g, ctx.group), None


def take_dp(shard, ids, lo, group=None):
    """Embedding rows for this rank's own ids (any shape) from a row-sharded table."""
    flat = _gather(ids.reshape(-1), group)
    rows = _OwnRows.apply(take(shard, flat, lo, group), group)
    return rows.view(*ids.shape, shard.shape[-1])


def nll_dp(h, head_shard, y, lo, group=None, chunk=4096):
    """Per-token cross-entropy of this rank's OWN tokens, h (N, d), y (N,), with the head sharded by vocabulary rows.
    In the backward every rank receives the cotangents of all ranks' tokens, so a head shard's gradient is the sum
    over the tokens of all ranks (divide by W for the gradient of a rank-mean loss)."""
    hg = _AllRows.apply(h.reshape(-1, h.shape[-1]), group)
    return _OwnRows.apply(nll(hg, head_shard, _gather(y.reshape(-1), group), lo, group, chunk), group)


def ce_dp(h, head_shard, y, lo, group=None, chunk=4096):
    """Summed cross-entropy over the tokens of all ranks (the same value on every rank) with the head sharded by
    vocabulary rows; h (N, d) and y (N,) are this rank's own tokens."""
    hg = _AllRows.apply(h.reshape(-1, h.shape[-1]), group)
    return ce(hg, head_shard, _gather(y.reshape(-1), group), lo, group, chunk)
