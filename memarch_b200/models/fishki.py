"""Two heavy-part variants from the reference's 12 B JAX model.

**Fishki** (fishki.py:1-78): the heavy part is a pool of many identical small relu² FFN layers without attention.  A
step holds texts of one kind; a text passes through the *combination* of layers that belongs to its kind (own layers
plus some shared with the neighbouring kind, on a ring).  A linear router on the mean light state learns to guess the
kind.  Sharded form: the pool's weights are cut along d between ranks and the chosen layer is all-gathered before use
("weights travel, not words"); the gradient returns as a reduce-scatter, which autograd derives from the gather.

**Uroboros** (uroboros.py:1-98): compute proportional to surprise, decided by the model: a small head on the light
state predicts the model's *own* loss per token; the heavy layers see only the top `budget·T` tokens by predicted
loss; the budget shrinks between steps as more tokens are predicted to be "already eaten".
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

S_MAX = 20.0


def pools(kinds, n, pool):
    """Layer numbers per kind: `n // kinds` own + (pool − own) shared with the next kind on a ring."""
    own = n // kinds
    over = max(0, pool - own)
    return [list(range(own * k, own * k + own))[:pool] + [(own * (k + 1) + j) % n for j in range(over)]
            for k in range(kinds)]


class _GatherRows(torch.autograd.Function):
    """All-gather along dim 0 whose backward is the matching reduce-scatter."""

    @staticmethod
    def forward(ctx, x, group):
        import torch.distributed as dist
        ctx.group, ctx.n = group, x.shape[0]
        W = dist.get_world_size(group)
        out = [torch.empty_like(x) for _ in range(W)]
        dist.all_gather(out, x.contiguous(), group=group)
        return torch.cat(out, 0)

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist
        W, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)            # reduce-scatter written as reduce + own slice (gloo has no RS)
        return g[r * ctx.n:(r + 1) * ctx.n].clone(), None


class FishPool(nn.Module):
    def __init__(self, d, n=16, hf=1024, kinds=4, pool=6, center=False, shard=None):
        """`shard` = (rank, world, group): keep rows [rank·d/W, …) of `up` and [rank·hf/W, …) of `down`."""
        super().__init__()
        self.kinds, self.n, self.center, self.shard = kinds, n, center, shard
        self.sets = pools(kinds, n, pool)
        up = torch.randn(n, d, hf) * d ** -0.5
        down = torch.randn(n, hf, d) * hf ** -0.5 * 0.5
        if shard is not None:
            r, W, _ = shard
            up, down = up[:, r * d // W:(r + 1) * d // W].clone(), down[:, r * hf // W:(r + 1) * hf // W].clone()
        self.norm = nn.Parameter(torch.ones(n, d))
        self.up, self.down = nn.Parameter(up), nn.Parameter(down)
        for t in (self.norm, self.up, self.down):        # the optimizer leaves the units of a step's idle kinds alone
            t._idle_rows = True
        self.router = nn.Linear(d, kinds, bias=False)

    def _weights(self, i):
        up, down = self.up[i], self.down[i]
        if self.shard is not None:
            up, down = _GatherRows.apply(up, self.shard[2]), _GatherRows.apply(down, self.shard[2])
        return up, down

    def one(self, i, h):
        x = h.float()
        xn = (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)).to(h.dtype)
        if self.center:                                  # remove the stream's common vector: causal mean over the row
            xf = xn.float()
            t = torch.arange(1, xf.shape[1] + 1, device=h.device, dtype=torch.float32)[None, :, None]
            xn = (xf - xf.cumsum(1) / t).to(h.dtype)
        up, down = self._weights(i)
        a = (xn * self.norm[i].to(h.dtype)) @ up.to(h.dtype)
        return h + F.relu(a).square() @ down.to(h.dtype)

    def forward(self, h, order):
        """h (B,T,d); order: layer numbers of this step in sequence (data of the step, not of the graph)."""
        for i in order:
            h = self.one(int(i), h)
        return h

    def router_loss(self, lh, kind):
        """lh (B,T,d) light state (detached inside), kind (B,) -> (cross-entropy, accuracy, logits)."""
        logits = self.router(lh.detach().float().mean(1))
        return F.cross_entropy(logits, kind), (logits.argmax(-1) == kind).float().mean(), logits


class Uroboros(nn.Module):
    HID = 64

    def __init__(self, d):
        super().__init__()
        self.l1 = nn.Linear(d + 1, self.HID)
        self.l2 = nn.Linear(self.HID, 1)
        nn.init.zeros_(self.l1.bias)
        nn.init.constant_(self.l2.bias, 3.0)             # typical loss at the start, in nats

    def predict(self, lh, s_cur):
        """Predicted own loss per token (B,T) >= 0 from the detached light state and the light head's surprise."""
        sc = torch.log1p(s_cur.detach().clamp(0.0, S_MAX))[..., None]
        z = torch.cat([lh.detach().float(), sc], -1)
        return F.softplus(self.l2(F.gelu(self.l1(z)))[..., 0])

    @staticmethod
    def n_slots(T, budget):
        return max(1, min(T, int(round(T * budget))))

    @staticmethod
    def select(pred, budget):
        """Hard top-k by predicted loss: idx (B,A) ascending in position, valid all true; token 0 is always taken."""
        B, T = pred.shape
        A = Uroboros.n_slots(T, budget)
        key = pred.detach().clone()
        key[:, 0] = 1e9
        idx = key.topk(A, -1).indices.sort(-1).values
        return idx, torch.ones(B, A, dtype=torch.bool, device=pred.device)

    @staticmethod
    def loss(pred, nll_tok):
        return (pred.clamp(0.0, S_MAX) - nll_tok.detach().float().clamp(0.0, S_MAX)).pow(2).mean()

    @staticmethod
    def stats(pred, nll_tok, idx, eat):
        pred, tgt = pred.detach().float(), nll_tok.detach().float()
        sel = torch.zeros_like(pred).scatter(1, idx, 1.0)
        pc, tc = pred - pred.mean(), tgt - tgt.mean()
        corr = (pc * tc).mean() / ((pc.pow(2).mean() * tc.pow(2).mean()).sqrt().clamp(min=1e-9))
        return {"uroboros_eaten": (pred < eat).float().mean(), "uroboros_corr": corr,
                "uroboros_nll_sel": (tgt * sel).sum() / sel.sum().clamp(min=1.0),
                "uroboros_nll_skip": (tgt * (1 - sel)).sum() / (1 - sel).sum().clamp(min=1.0)}

    @staticmethod
    def next_budget(cur, eaten, levels, margin=1.25, corr=None, min_corr=0.5):
        """Host side, between steps: the smallest level >= (1 − eaten)·margin, at most one level down at a time, never
        up; while the head does not yet know its errors (corr < min_corr) the budget stays."""
        if corr is not None and float(corr) < min_corr:
            return cur
        levels = sorted(levels, reverse=True)
        need = (1.0 - float(eaten)) * margin
        i = levels.index(cur) if cur in levels else 0
        if i + 1 < len(levels) and levels[i + 1] >= need:
            return levels[i + 1]
        return levels[i]
