"""One process per GPU: data parallelism for the light layers / tables, expert parallelism for the heavy layers.

Semantics (the reference's FSDP+EP torch path, fastloop.py:269-307, full2.py:1122-1156, and the JAX port's
`dist.py`): every rank routes and slots its own anchors (capacity from the local N); experts are sharded E/W per
rank and tokens travel by all-to-all; all other weights are replicated and stepped with the rank-mean gradient; the
loss fed to the optimizer, the situation vector and the anchor threshold `tau` are rank means.

Two modes share this interface:
  * `fused=False`  NCCL (or gloo on CPU) collectives only: all-to-all for the experts, asynchronous all-reduce of
                   each weight's gradient overlapped with the rest of backward.  The baseline and the CPU test path.
  * `fused=True`   the peer-memory kernels of `memarch_b200.parallel.fused`: expert rows pulled from the owners'
                   symmetric buffers, expert GEMMs whose epilogue stores result rows into the owners' buffers, and
                   the one-shot peer / NVLS all-reduce of each replicated weight's gradient on a side stream ahead
                   of that weight's Instinct step.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


class _AllToAll(torch.autograd.Function):
    """Equal-split all-to-all over dim 0 with autograd; returns a plain tensor that is complete on the current stream
    (the functional-collectives wrapper tensor must not reach a C++ kernel: its data pointer is not the data)."""

    @staticmethod
    def forward(ctx, x, gname):
        ctx.gname = gname
        n = dist.get_world_size()
        split = [x.shape[0] // n] * n
        t = torch.ops._c10d_functional.all_to_all_single(x.contiguous(), split, split, gname)
        return torch.ops._c10d_functional.wait_tensor(t)

    @staticmethod
    def backward(ctx, g):
        n = dist.get_world_size()
        split = [g.shape[0] // n] * n
        t = torch.ops._c10d_functional.all_to_all_single(g.contiguous(), split, split, ctx.gname)
        return torch.ops._c10d_functional.wait_tensor(t), None


# ---- split all-to-all: start now, wait where the data is needed.  K-chunk pipelining of the expert exchange (the
# reference's JAX port, moe.py:263-287: the exchange of chunk k+1 runs under the expert FFN of chunk k) is built from
# these two halves; in backward the halves swap roles, so the gradient exchange of a chunk overlaps the FFN backward
# of its neighbour the same way.
_IN_FLIGHT = {}          # data_ptr of the receive buffer -> (work handle, send buffer kept alive)


def _a2a_begin(x, group):
    src = x.contiguous()
    out = torch.empty_like(src)
    _IN_FLIGHT[out.data_ptr()] = (dist.all_to_all_single(out, src, group=group, async_op=True), src)
    return out


def _a2a_end(t):
    pending = _IN_FLIGHT.pop(t.data_ptr(), None)
    if pending is not None:
        pending[0].wait()
    return t


class _ExchangeStart(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _a2a_begin(x, group)

    @staticmethod
    def backward(ctx, g):
        return _a2a_end(g), None


class _ExchangeWait(torch.autograd.Function):
    @staticmethod
    def forward(ctx, t, group):
        ctx.group = group
        return _a2a_end(t).view_as(t)

    @staticmethod
    def backward(ctx, g):
        return _a2a_begin(g, ctx.group), None


def ring_exchange(x, group=None):
    """The same permutation as the equal-split all-to-all over dim 0, as W-1 point-to-point steps: in step s every
    rank sends its block for rank (r+s) and receives the block of rank (r-s).  The reference's JAX port keeps such a
    ring beside `all_to_all` (moe.py:119-152) because each step's transfer can overlap the FFN of the blocks that
    already arrived; here it is the baseline the fused exchange is compared with on meshes where all-to-all is slow."""
    W, r = dist.get_world_size(group), dist.get_rank(group)
    x = x.contiguous()
    out = torch.empty_like(x)
    n = x.shape[0] // W
    out[r * n:(r + 1) * n] = x[r * n:(r + 1) * n]
    glob = (lambda k: dist.get_global_rank(group, k)) if group is not None else (lambda k: k)
    for s_ in range(1, W):
        to, frm = (r + s_) % W, (r - s_) % W
        ops_ = [dist.P2POp(dist.isend, x[to * n:(to + 1) * n], glob(to), group),
                dist.P2POp(dist.irecv, out[frm * n:(frm + 1) * n], glob(frm), group)]
        for w in dist.batch_isend_irecv(ops_):
            w.wait()
    return out


class _Ring(torch.autograd.Function):
    """`ring_exchange` with autograd: the permutation is its own transpose."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return ring_exchange(x, group)

    @staticmethod
    def backward(ctx, g):
        return ring_exchange(g, ctx.group), None


class NcclExpertExchange:
    """Expert-parallel FFN through two autograd all-to-alls (full2.py:1137-1156), extended to a sharded frozen bank.
    `MEMARCH_EP_A2A=ring` moves the tokens by the W-1 step ring instead of one all-to-all."""

    def __init__(self, rank, world, group=None):
        import os
        self.rank, self.W, self.group = rank, world, group
        self.ring = os.environ.get("MEMARCH_EP_A2A", "a2a") == "ring"
        self.dedup = os.environ.get("EP_A2A_DEDUP") == "1"
        self.dedup_cap = float(os.environ.get("EP_DEDUP_CAP", 1.0))
        self.chunks = max(1, int(os.environ.get("MEMARCH_EP_CHUNKS", 1)))      # K-chunk pipelined exchange (all-to-all form)

    def _move(self, x, gname):
        return _Ring.apply(x, self.group) if self.ring else _AllToAll.apply(x, gname)

    def _perm(self, moe):
        """Order experts so each rank's share is contiguous: rank r gets its learning experts then its frozen ones."""
        W = self.W
        if not getattr(moe, "bank", False) or not moe.has_F:
            return None, moe.E // W, 0
        L, Fz = moe.L, moe.Fz
        El, Fl = len(L) // W, len(Fz) // W
        order = []
        for r in range(W):
            order += L[r * El:(r + 1) * El] + Fz[r * Fl:(r + 1) * Fl]
        return torch.tensor(order, device=moe.up.device), El, Fl

    def forward_dedup(self, moe, xf, table, wtab, C, cap=1.0):
        """Expert-parallel layer where a (token, rank) pair crosses the wire once, however many of the rank's experts
        the token chose (full2.py:967-1046: pays when a rank holds several experts and tokens pick more than one of
        them).  xf (N, d) normalised tokens, table (E*C,) token of every expert slot (N = empty), wtab (E*C,) routing
        weights -> (N, d) weighted sum over each token's experts.  Per destination rank the distinct tokens form a
        parcel of at most Cc = min(El*C, N, cap*El*C) rows; the owner expands a parcel row to the slots of its
        experts, runs the FFN, adds the weighted outputs per parcel row (fp32) and returns one row per pair.  Expert
        capacity and drops are those of the ordinary dispatch; with cap < 1 whole pairs beyond Cc are dropped and
        counted in `moe.dropped`.  Learning experts only (no sharded frozen bank)."""
        W, E = self.W, moe.E
        N, d = xf.shape
        El = E // W
        S = El * C
        Cc = max(1, min(S, N, int(-(-cap * S // 1))))
        gname = (self.group or dist.group.WORLD).group_name
        dev = xf.device
        with torch.no_grad():
            tb = table.view(W, S)
            hit = torch.zeros(W, N + 1, dtype=torch.bool, device=dev).scatter_(1, tb, True)[:, :N]
            pos = hit.long().cumsum(1) - 1                                   # row of token n in the parcel to rank s
            go = hit & (pos < Cc)
            pos = torch.where(go, pos, Cc)                                   # Cc = does not travel
            ctok = torch.full((W, Cc + 1), N, dtype=torch.long, device=dev)
            ctok.scatter_(1, pos, torch.arange(N, device=dev).expand(W, N))  # distinct targets except the spill column
            ctok = ctok[:, :Cc]
            row = torch.cat([pos, pos.new_full((W, 1), Cc)], 1).gather(1, tb)   # parcel row of every expert slot
            lost = ((row == Cc) & (tb < N)).sum()
            placed = (tb < N).sum().clamp(min=1)
        moe.dropped = 1 - (1 - moe.dropped) * (placed - lost) / placed
        xpad = torch.cat([xf, xf.new_zeros(1, d)])
        xr = self._move(xpad[ctok.reshape(-1)], gname).view(W, Cc, d)       # parcels from every source rank
        rr = self._move_plain(row.reshape(-1)).view(W, S)
        wr = self._move(wtab.reshape(-1).float(), gname).view(W, S)
        xrp = torch.cat([xr, xr.new_zeros(W, 1, d)], 1)
        xe = xrp.gather(1, rr[..., None].expand(-1, -1, d))                 # (W, S, d): rows expanded to the slots
        xe = xe.view(W, El, C, d).transpose(0, 1).reshape(El, W * C, d)
        y = moe._ffn(xe, moe.up, moe.down)
        y = y.view(El, W, C, d).transpose(0, 1).reshape(W, S, d)
        yw = y.float() * wr[..., None]
        yc = yw.new_zeros(W, Cc + 1, d).scatter_add(1, rr[..., None].expand(-1, -1, d), yw)[:, :Cc]
        yb = self._move(yc.to(xf.dtype).reshape(W * Cc, d), gname).view(W, Cc, d)
        ybp = torch.cat([yb, yb.new_zeros(W, 1, d)], 1)
        return ybp.gather(1, pos[..., None].expand(-1, -1, d)).float().sum(0).to(xf.dtype)

    def _move_plain(self, t):
        """Integer metadata through the same exchange, outside autograd."""
        with torch.no_grad():
            if self.ring:
                return ring_exchange(t, self.group)
            out = torch.empty_like(t)
            dist.all_to_all_single(out, t.contiguous(), group=self.group)
            return out

    def ffn(self, moe, xe):
        W = self.W
        E, C, d = xe.shape
        perm, El, Fl = self._perm(moe)
        gname = (self.group or dist.group.WORLD).group_name
        if perm is not None:
            xe = xe[perm]
        n = El + Fl

        def experts(r, c):
            """Rows received from every rank (W*n, c, d) -> outputs in the layout of the way back."""
            r = r.view(W, n, c, d).transpose(0, 1).reshape(n, W * c, d)
            y = moe._ffn(r[:El], moe.up, moe.down)
            if Fl:
                y = torch.cat([y, moe._ffn_frozen(r[El:])])
            return y.view(n, W, c, d).transpose(0, 1).reshape(E, c, d).contiguous()

        K = min(self.chunks, C)
        if K > 1 and not self.ring:
            # the places of every expert in K slices: all dispatches start at once, a slice's FFN runs as soon as its
            # rows are here, its outputs start their way back while the next slice is computed
            cuts = [C * k // K for k in range(K + 1)]
            there = [_ExchangeStart.apply(xe[:, a:b], self.group) for a, b in zip(cuts, cuts[1:])]
            back = [_ExchangeStart.apply(experts(_ExchangeWait.apply(t, self.group), t.shape[1]), self.group) for t in there]
            y = torch.cat([_ExchangeWait.apply(t, self.group) for t in back], 1)
        else:
            y = self._move(experts(self._move(xe, gname), C), gname)
        if perm is not None:
            inv = torch.empty_like(perm)
            inv[perm] = torch.arange(E, device=perm.device)
            y = y[inv]
        return y


class ParallelEngine:
    SMALL = 1 << 16          # weights below this many elements are reduced together at the end of backward

    def __init__(self, rank, world, local_rank=0, fused=True, group=None):
        self.rank, self.W, self.local = rank, world, local_rank
        self.group = group
        self.fused = bool(fused) and torch.cuda.is_available()
        self.ep = NcclExpertExchange(rank, world, group)
        self.fused_impl = None
        self.pending = []            # (param, grad, work) all-reduces in flight
        self.small = []
        self.trainer = None
        self.ctrl = None
        import os
        self.dp_mode = os.environ.get("MEMARCH_DP", "fused")           # "fused" | "nccl" (gradient mean of the replicated weights)

    def init_fused(self):
        """Create the peer-memory machinery (symmetric heap, fused EP and DP objects) if this engine is in fused mode
        and has none yet; returns it (None in NCCL mode)."""
        if self.fused and self.fused_impl is None:
            from .fused import FusedParallel
            self.fused_impl = FusedParallel(self)
        return self.fused_impl

    # ------------------------------------------------------------------------------------------ model sharding
    def shard_model(self, model):
        """Keep this rank's experts only; replicate the rest (identical init on every rank: same seed)."""
        from ..models.moe import AnchorMoE
        self.init_fused()
        for mod in model.modules():
            if isinstance(mod, AnchorMoE):
                mod.ep_shard(self.rank, self.W, self.fused_impl.ep if self.fused_impl else self.ep)
        if self.W > 1 and os.environ.get("MEMARCH_VP") == "1" and hasattr(model, "vocab_shard"):
            model.vocab_shard(self.rank, self.W, self.group)      # row-sharded word tables (large vocabularies)
        def bcast(t):
            if t.is_contiguous():
                dist.broadcast(t, 0, group=self.group)
            else:
                c = t.contiguous()
                dist.broadcast(c, 0, group=self.group)
                t.copy_(c)
        if self.W > 1:
            for p in model.parameters():
                if not getattr(p, "_ep_local", False):
                    bcast(p.data)
            for b in model.buffers():
                if b.numel() and b.dtype.is_floating_point:
                    bcast(b.data)

    def attach(self, trainer):
        self.trainer = trainer
        trainer.opt.grad_sync = self.grad_sync
        if self.fused_impl is not None:
            self.fused_impl.attach(trainer)

    def before_checkpoint(self):
        """Make every rank's copy of the row-sharded weights and their momentum whole (collective)."""
        if self.fused_impl is not None:
            self.fused_impl.dp.materialize()

    def check(self):
        """Raise if a bounded peer wait (barrier) ran out since the last check.  Host sync: call it where the loop
        already waits for the device (log interval, before a checkpoint, end of a benchmark)."""
        if self.fused_impl is not None:
            self.fused_impl.heap.check()

    # ------------------------------------------------------------------------------------------ control values
    def sync_control(self, loss, sit, model):
        """One small all-reduce: mean loss, true batch-mean situation vector and the shared anchor threshold.  NCCL in
        the baseline mode; in the fused mode the one-shot peer all-reduce on a symmetric buffer."""
        taus = [getattr(model, n) for n in ("tau", "rope_tau", "rope_qtau") if hasattr(model, n)]
        buf = torch.cat([loss.reshape(1).float()] + [t.reshape(1).float() for t in taus] + [sit.float().reshape(-1)])
        self.mean_vector(buf)
        for j, t in enumerate(taus):
            t.copy_(buf[1 + j])
        return buf[0], buf[1 + len(taus):]

    def mean_vector(self, buf):
        """Rank-mean of a small fp32 vector, in place."""
        if self.W > 1:
            if self.fused_impl is not None and buf.is_cuda:
                self.fused_impl.mean_small(buf)              # peer loads / stores between two device barriers
            else:
                dist.all_reduce(buf, group=self.group)
                buf /= self.W
        return buf

    # ------------------------------------------------------------------------------------------ gradients
    def before_backward(self, trainer):
        self.pending.clear()
        self.small.clear()

    def grad_sync(self, p, grad):
        """Called by the optimizer from the weight's grad-ready hook.  Expert weights are rank-local.  Replicated
        weights: average over ranks.  Returns the gradient to step with, or None when the step is deferred."""
        if getattr(p, "_ep_local", False):
            return grad
        if self.fused_impl is not None and self.dp_mode == "fused":   # also with one rank: the GPU's own buffers
            return self.fused_impl.dp.grad_ready(p, grad)
        if self.W == 1:
            return grad
        if grad.numel() < self.SMALL:
            self.small.append((p, grad))
            return None
        work = dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self.pending.append((p, grad, work))
        self._drain(keep=1)                      # step the weights whose reduction has had a layer's time to finish
        return None

    def _drain(self, keep=0):
        opt = self.trainer.opt
        while len(self.pending) > keep:
            p, grad, work = self.pending.pop(0)
            work.wait()
            grad.div_(self.W)
            opt.update(p, grad, synced=True)

    def after_backward(self, trainer):
        if self.fused_impl is not None and self.dp_mode == "fused":
            self.fused_impl.dp.flush()
            return
        self._drain(0)
        if self.small:
            flat = torch.cat([g.reshape(-1).float() for _, g in self.small])
            dist.all_reduce(flat, group=self.group)
            flat /= self.W
            off = 0
            for p, g in self.small:
                n = g.numel()
                trainer.opt.update(p, flat[off:off + n].view_as(g).to(g.dtype), synced=True)
                off += n
            self.small.clear()

    def reduce_grads(self, params):
        """Plain optimizers (AdamW path): average every replicated gradient after backward."""
        for p in params:
            if p.grad is not None and not getattr(p, "_ep_local", False):
                dist.all_reduce(p.grad, group=self.group)
                p.grad.div_(self.W)


def init_distributed(backend=None, timeout_s=1800):
    """torchrun-style rendezvous from RANK / WORLD_SIZE / LOCAL_RANK (fastloop.py:207-214)."""
    import datetime
    import os
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        cuda = torch.cuda.is_available()
        if cuda:
            torch.cuda.set_device(local)
        dist.init_process_group(backend or ("nccl" if cuda else "gloo"), timeout=datetime.timedelta(seconds=timeout_s))
    return rank, world, local
