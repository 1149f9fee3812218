"""Fused compute + collective paths over NVLink 5 / NVSwitch peer memory (one process per GPU).

Expert parallelism (replaces the two all-to-alls around the expert FFN, full2.py:1137-1156):
  * every rank writes its dispatched anchors `xe (E, C, d)` into a symmetric buffer;
  * the up-GEMM of the rank that owns expert e reads its A tiles straight from the owners' buffers (one TMA tensor map
    per source GPU, plain non-multicast loads) - the dispatch all-to-all happens inside the GEMM's operand fetch;
  * the down-GEMM's epilogue stores each result row into the symmetric output buffer of the GPU that owns the token -
    the combine all-to-all happens inside the GEMM's epilogue;
  * backward mirrors it: the output gradients are pulled from the owners (peer copies), the input gradient rows are
    pushed to the owners by the dgrad GEMM's epilogue.
Data parallelism (replaces reduce-scatter + all-gather of FSDP, fastloop.py:269-307):
  * a weight's gradient is staged in a symmetric buffer from its grad-ready hook; on a side stream a one-shot kernel
    reduces each rank's slice across all GPUs and broadcasts the mean (NVLS `multimem.ld_reduce` / `multimem.st` when
    the switch offers multicast, plain peer loads/stores otherwise), then the Instinct kernels step the weight while
    backward continues on the main stream.
Every device-side wait is bounded (`wait_ms`); a timeout sets a status word that `check()` turns into an exception.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import _ext
from ..ops.basic import gemm


class SymmetricHeap:
    """Symmetric allocations (same size on every rank) with peer pointers, and the bounded barrier on symmetric flags."""

    def __init__(self, rank, world, group=None, wait_ms=4000.0):
        import torch.distributed._symmetric_memory as symm_mem
        self.sm = symm_mem
        self.rank, self.W, self.wait_ms = rank, world, wait_ms
        self.group = group or dist.group.WORLD
        self.gname = self.group.group_name
        try:
            symm_mem.enable_symm_mem_for_group(self.gname)
        except Exception:     # noqa: BLE001 - newer torch enables groups implicitly
            pass
        self.flags, self.flag_hdl = self.alloc((256,), torch.int32, zero=True)
        self.flag_ptrs = [int(p) for p in self.flag_hdl.buffer_ptrs]
        dist.barrier(group=self.group)

    def alloc(self, shape, dtype, zero=False):
        t = self.sm.empty(*shape, dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))
        if zero:
            t.zero_()
        hdl = self.sm.rendezvous(t, self.gname)
        return t, hdl

    def barrier(self, channel=0):
        """Device-side barrier on the current stream: all ranks' earlier writes are visible afterwards."""
        _ext.C().peer_barrier(self.flag_ptrs, self.rank, channel, float(self.wait_ms))
        _ext.count()

    def check(self):
        st = _ext.C().peer_status_read()
        if st:
            raise RuntimeError(f"peer wait timed out (status {st}): a rank did not reach the barrier within {self.wait_ms} ms")


def _rotated(W, r):
    """Peer order of rank r: itself first, then r+1, ... — a different peer for every rank at every position."""
    return [(r + i) % W for i in range(W)]


class _FusedExpertFFN(torch.autograd.Function):
    """xe (E, C, d) on every rank -> ye (E, C, d): experts sharded over ranks, tokens moved by the GEMMs themselves."""

    @staticmethod
    def forward(ctx, xe, up, down, ep, key, act, g_off, n_local, train_w, e_lo=0, e_hi=None):
        heap, W, r = ep.heap, ep.W, ep.rank
        E, Cn, d = xe.shape
        C = _ext.C()
        X, Xh, Y, Yh = ep.layer_buffers(key, E, Cn, d)
        X.copy_(xe)
        heap.barrier(0)                                             # every rank's anchors are in place
        H = up.shape[2]
        M = W * Cn
        h = torch.empty(n_local, M, H, device=xe.device, dtype=torch.bfloat16)
        a = torch.empty_like(h) if act == "relu2" else None
        # rows of my experts land in local memory first (one bandwidth-bound gather kernel over the peer pointers),
        # the GEMM reads them locally: fetching remote tiles with the GEMM's own loads put an NVLink round trip into
        # every stage of its shared-memory ring (measured 22 ms per step slower) and was dropped
        xin = torch.empty(n_local, M, d, device=xe.device, dtype=torch.bfloat16)
        C.peer_gather([int(p) for p in Xh.buffer_ptrs], xin, r, Cn, g_off)          # one kernel over all W owners
        _ext.count()
        if act == "relu2":
            gemm(xin, up, b_mn=True, out=h, out2=a, epi=1, groups=n_local)
        else:
            a = gemm(xin, up, b_mn=True, groups=n_local)
            h = C.swiglu_fwd(a)
        # down-GEMM: A = h, cut into W row segments; segment s goes to rank s's output buffer
        hp = h.data_ptr()
        Hh = h.shape[2]
        # the GEMM walks its segments in list order: rotate the (A segment, destination) pairs by the rank, so that at
        # any moment the W ranks store to W different GPUs (own rows first) instead of all to the same one
        order = _rotated(W, r)
        a_ptrs = [hp + s * Cn * Hh * 2 for s in order]
        yptrs = [int(Yh.buffer_ptrs[s]) for s in order]
        _ext.count_flops(2 * M * Hh * d * n_local)
        C.gemm_peer(a_ptrs, Cn, Hh, n_local, Hh, M * Hh, 0, down, True, None, yptrs, d, Cn * d, g_off, None, None, 0, n_local)
        _ext.count(3)
        heap.barrier(0)                                             # every expert's rows have landed here
        # the staged rows are kept for the weight gradient: the backward then pulls only dY (E x C x d bf16 per layer)
        ctx.has_xin = train_w
        ctx.save_for_backward(up, down, a, h, *([xin] if ctx.has_xin else []))
        ctx.ep, ctx.key, ctx.act, ctx.g_off, ctx.n_local, ctx.train_w = ep, key, act, g_off, n_local, train_w
        ctx.shape = (E, Cn, d)
        ctx.e_range = (int(e_lo), int(E if e_hi is None else e_hi))        # global experts served by this call, all ranks
        return Y.view_as(Y)

    @staticmethod
    def backward(ctx, dy):
        up, down, a, h = ctx.saved_tensors[:4]
        ep, act, g_off, nl = ctx.ep, ctx.act, ctx.g_off, ctx.n_local
        heap, W, r = ep.heap, ep.W, ep.rank
        E, Cn, d = ctx.shape
        C = _ext.C()
        X, Xh, _, _ = ep.layer_buffers(ctx.key, E, Cn, d)
        DY, DYh, DX, DXh = ep.grad_buffers(E, Cn, d)
        DY.copy_(dy)
        heap.barrier(0)
        M = W * Cn
        # pull the rows of my experts from their owners once; every local GEMM reads the local copy
        dy_all = torch.empty(nl, M, d, device=dy.device, dtype=torch.bfloat16)
        xe_all = ctx.saved_tensors[4] if ctx.has_xin else None
        pull_x = ctx.train_w and xe_all is None
        if pull_x:
            xe_all = torch.empty(nl, M, d, device=dy.device, dtype=torch.bfloat16)
        C.peer_gather([int(p) for p in DYh.buffer_ptrs], dy_all, r, Cn, g_off)
        if pull_x:
            C.peer_gather([int(p) for p in Xh.buffer_ptrs], xe_all, r, Cn, g_off)
        _ext.count(2 if pull_x else 1)
        if act == "relu2":
            da = gemm(dy_all, down, epi=2, aux=a, groups=nl)
        else:
            da = C.swiglu_bwd(gemm(dy_all, down, groups=nl), a)
        dup = ddown = None
        if ctx.train_w:
            ddown = gemm(h, dy_all, a_mn=True, b_mn=True, groups=nl)
            dup = gemm(xe_all, da, a_mn=True, b_mn=True, groups=nl)
        # dxe = da . up^T, rows pushed to the owners of the tokens
        Hh = da.shape[2]
        order = _rotated(W, r)
        a_ptrs = [da.data_ptr() + s * Cn * Hh * 2 for s in order]
        dxptrs = [int(DXh.buffer_ptrs[s]) for s in order]
        _ext.count_flops(2 * M * Hh * d * nl)
        C.gemm_peer(a_ptrs, Cn, Hh, nl, Hh, M * Hh, 0, up, False, None, dxptrs, d, Cn * d, g_off, None, None, 0, nl)
        _ext.count()
        heap.barrier(0)
        # the gradient buffer is shared by every call of this shape and only the rows of this call's experts were
        # written by it (a bank layer runs one call for the learning and one for the frozen experts): hand back those
        # rows and zeros elsewhere, never what an earlier call left in the other rows
        lo, hi = ctx.e_range
        if lo == 0 and hi == E:
            dx = DX.clone()
        else:
            dx = torch.zeros_like(DX)
            dx[lo:hi].copy_(DX[lo:hi])
        return dx, dup, ddown, None, None, None, None, None, None, None, None


class FusedExpertExchange:
    """`ep_engine` of AnchorMoE in fused mode."""

    def __init__(self, heap):
        self.heap, self.W, self.rank = heap, heap.W, heap.rank
        self._layers, self._grads = {}, {}

    def layer_buffers(self, key, E, C, d):
        k = (key, E, C, d)
        if k not in self._layers:
            X, Xh = self.heap.alloc((E, C, d), torch.bfloat16)
            Y, Yh = self.heap.alloc((E, C, d), torch.bfloat16)
            self._layers[k] = (X, Xh, Y, Yh)
        return self._layers[k]

    def grad_buffers(self, E, C, d):
        k = (E, C, d)
        if k not in self._grads:
            DY, DYh = self.heap.alloc((E, C, d), torch.bfloat16)
            DX, DXh = self.heap.alloc((E, C, d), torch.bfloat16)
            self._grads[k] = (DY, DYh, DX, DXh)
        return self._grads[k]

    def ffn(self, moe, xe):
        W, r = self.W, self.rank
        if xe.dtype != torch.bfloat16:
            xe = xe.to(torch.bfloat16)
        key = id(moe)
        if getattr(moe, "bank", False) and moe.has_F:
            # learning experts L (global ids 0..nL-1 in slot order) and frozen ones: two grouped launches per GEMM
            nL, nF = len(moe.L), len(moe.Fz)
            assert moe.L == list(range(nL)) and moe.Fz == list(range(nL, nL + nF)), "fused EP expects banks in id order"
            El, Fl = nL // W, nF // W
            yL = _FusedExpertFFN.apply(xe, moe.up, moe.down, self, (key, "L"), moe.act, r * El, El, True, 0, nL)
            yF = _FusedExpertFFN.apply(xe, moe._bank_weights("up"), moe._bank_weights("down"), self, (key, "F"), moe.act,
                                       nL + r * Fl, Fl, False, nL, nL + nF)
            sel = torch.arange(moe.E, device=xe.device)[:, None, None] < nL
            return torch.where(sel, yL, yF)
        El = moe.E // W
        return _FusedExpertFFN.apply(xe, moe.up, moe.down, self, key, moe.act, r * El, El, True)


class FusedGradReduce:
    """Data-parallel gradient exchange fused with the optimizer step, on a side stream that overlaps backward.

    Two forms.  Row-sharded (`MEMARCH_DP_SHARD`, default on; the 2-D "hs" weights whose GEMMs read a bf16 matrix -
    the weight itself under BF16_W, else the bf16 shadow of the light-block linears): the reduce-scatter + update + all-gather of the reference's FSDP path (fastloop.py:269-307)
    with the cross-shard column norms of its `hsS` kind (exp_opt.py:271-280).  Rank r owns rows [r R/W, (r+1) R/W) of
    every such weight: it sums those rows of the staged gradients from all ranks into local memory (`multimem.ld_reduce`
    or peer loads), runs the Instinct statistics on them, the ranks sum the column sums in place in a symmetric
    scratch (one tiny one-shot all-reduce), the update writes momentum and fp32 weight of these rows only, and the new
    bf16 rows go to every rank's shadow (`multimem.st` or peer stores) - optimizer work and touched optimizer state
    are 1/W per rank, and the weight all-gather is the store of the update.  Replicated (everything else): one-shot
    all-reduce of the gradient, then the full Instinct step on every rank."""

    def __init__(self, heap, nvls=True):
        self.heap, self.W, self.rank = heap, heap.W, heap.rank
        # the per-weight chains (barrier, reduce, statistics, exchange, update, all-gather) are latency-bound, so
        # several run side by side: weight i takes lane i % lanes = its own stream, barrier channel, statistics
        # scratch and reduced-gradient buffer (the same assignment on every rank)
        self.lanes = max(1, min(8, int(os.environ.get("MEMARCH_DP_LANES", 4))))
        self.streams = [torch.cuda.Stream() for _ in range(self.lanes)]
        self.stream = self.streams[0]
        self.lane_of = {}
        self.nvls = nvls
        self.offsets = {}
        self.top = 0
        self.small = []
        self.trainer = None
        self.used = False
        self.cap = 0
        self.shard = os.environ.get("MEMARCH_DP_SHARD", "1") != "0"
        self.sharded = {}            # id(param) -> (byte offset of its shadow, rows per rank)

    def allocate(self, params):
        """Symmetric staging (each rank's gradient) and result (the rank mean) regions for every replicated weight."""
        heap, nvls = self.heap, self.nvls
        cap = 0
        for p in params:
            if not getattr(p, "_ep_local", False):
                cap += (p.numel() * p.element_size() + 255) // 256 * 256
        self.cap = max(cap, 256)
        self.gin, self.gin_h = heap.alloc((self.cap,), torch.uint8)
        self.gout, self.gout_h = heap.alloc((self.cap,), torch.uint8)
        self.in_ptrs = [int(p) for p in self.gin_h.buffer_ptrs]
        self.out_ptrs = [int(p) for p in self.gout_h.buffer_ptrs]
        mc_ok = nvls and os.environ.get("MEMARCH_NVLS", "1") == "1"
        try:
            self.mc_in = int(self.gin_h.multicast_ptr) if mc_ok else 0
            self.mc_out = int(self.gout_h.multicast_ptr) if mc_ok else 0
        except Exception:     # noqa: BLE001
            self.mc_in = self.mc_out = 0
        self._allocate_shards(params, mc_ok)

    def _allocate_shards(self, params, mc_ok):
        """The bf16 matrices the GEMMs read (the weight itself when it lives in bf16 with an fp32 copy in the optimizer,
        else its bf16 shadow) move into one symmetric buffer, because peers write their rows into them; plus the
        symmetric statistics scratch and a local buffer for this rank's reduced gradient rows."""
        opt, W = self.trainer.opt, self.W
        if not self.shard:
            return
        todo = [p for p in params if not getattr(p, "_ep_local", False) and opt.can_shard(p)
                and (p.dtype == torch.bfloat16 or getattr(p, "_shard_ok", False))
                and p.numel() >= 4096 and p.shape[0] % W == 0 and (p.shape[0] // W * p.shape[1]) % 8 == 0]
        if not todo:
            return
        tot = sum((p.numel() * 2 + 255) // 256 * 256 for p in todo)
        self.wsh, self.wsh_h = self.heap.alloc((tot,), torch.uint8)
        self.wsh_ptrs = [int(x) for x in self.wsh_h.buffer_ptrs]
        try:
            self.mc_wsh = int(self.wsh_h.multicast_ptr) if mc_ok else 0
        except Exception:     # noqa: BLE001
            self.mc_wsh = 0
        need = max(3 * ((p.shape[0] // W + 3) // 4 * 4) + 2 * ((p.shape[1] + 3) // 4 * 4) + 4 for p in todo)
        self.scr, self.scr_ptrs, self.gred = [], [], []
        for _ in range(self.lanes):
            t, h = self.heap.alloc(((need + 63) // 64 * 64,), torch.float32)
            self.scr.append(t)
            self.scr_ptrs.append([int(x) for x in h.buffer_ptrs])
            self.gred.append(torch.empty(max(p.numel() // W for p in todo), device=self.wsh.device, dtype=torch.bfloat16))
        off = 0
        with torch.no_grad():
            for p in todo:
                sh = self.wsh[off:off + p.numel() * 2].view(torch.bfloat16).view(p.shape)
                sh.copy_(p.detach())
                if p.dtype == torch.bfloat16:
                    p.data = sh                                   # the parameter itself now lives where peers can write
                else:
                    p._bf16_shadow, p._shadow_ver = sh, p._version
                self.sharded[id(p)] = (off, p.shape[0] // W)
                off += (p.numel() * 2 + 255) // 256 * 256
        self.heap.barrier(0)

    def _exchange(self, offset, count, lane=0):
        """Sum `count` floats at `offset` of a lane's symmetric statistics scratch over the ranks, in place (every rank
        reduces its own 1/W of the range from all peers and writes it back to all of them)."""
        if self.W == 1:
            return
        self.heap.barrier(4 + lane)
        _ext.C().peer_allreduce(self.scr_ptrs[lane], self.scr_ptrs[lane], 0, 0, offset, count, False, self.rank, 1.0)
        _ext.count()
        self.heap.barrier(4 + lane)

    def materialize(self):
        """fp32 weights and momentum of the row-sharded weights are current only in the owner's rows; before anything
        reads them whole (a checkpoint in the single-file layout, an evaluation that bypasses the shadows) the ranks
        exchange their rows.  Collective; not on the training path."""
        if not self.sharded or self.W == 1:
            return
        opt = self.trainer.opt
        for p in self.trainer.params:
            if id(p) in self.sharded:
                i = opt.idx[id(p)]
                whole = [opt.m[i]] + ([opt.w[i]] if opt.w[i] is not None else [p.data])
                for t in whole:
                    parts = list(t.chunk(self.W, 0))
                    dist.all_gather(parts, parts[self.rank].clone(), group=self.heap.group)

    def _region(self, p, grad):
        k = id(p)
        if k not in self.offsets:
            n = grad.numel() * grad.element_size()
            n = (n + 255) // 256 * 256
            if self.top + n > self.cap:
                raise RuntimeError("gradient staging buffer too small for this weight")
            self.offsets[k] = self.top
            self.top += n
        return self.offsets[k]

    def grad_ready(self, p, grad):
        """From the weight's grad-ready hook (main stream).  Returns None: the step is made on the side stream."""
        if grad.numel() % 8 or grad.numel() < 4096 or grad.dtype not in (torch.bfloat16, torch.float32):
            self.small.append((p, grad))
            return None
        off = self._region(p, grad)
        es = grad.element_size()
        n = grad.numel()
        stage = self.gin[off:off + n * es].view(grad.dtype).view(grad.shape)
        stage.copy_(grad)                                            # main stream: gradient into symmetric staging
        ev = torch.cuda.Event()
        ev.record()
        C = _ext.C()
        heap = self.heap
        lane = self.lane_of.setdefault(id(p), len(self.lane_of) % self.lanes)      # first-use order: backward's order, the same on every rank
        stream = self.streams[lane]
        sh = self.sharded.get(id(p)) if grad.dtype == torch.bfloat16 else None
        if sh is not None:
            woff, rows = sh
            r0, r1 = self.rank * rows, (self.rank + 1) * rows
            cols = p.shape[1]
            with torch.cuda.stream(stream):
                stream.wait_event(ev)
                heap.barrier(4 + lane)                               # every rank has staged this weight's gradient
                g_rows = self.gred[lane][:rows * cols].view(rows, cols)
                C.peer_reduce_to_local(self.in_ptrs, self.mc_in, g_rows, off // es + r0 * cols, 1.0 / self.W)
                self.trainer.opt.update_sharded(p, g_rows, r0, r1, self.scr[lane],
                                                None if p.dtype == torch.bfloat16 else p._bf16_shadow[r0:r1],
                                                lambda o_, n_, lane=lane: self._exchange(o_, n_, lane))
                C.peer_broadcast_from_local(self.wsh_ptrs, self.mc_wsh, woff + r0 * cols * 2, rows * cols * 2, self.rank)
                _ext.count(2)
            self.used = self.pushed = True
            return None
        with torch.cuda.stream(stream):
            stream.wait_event(ev)
            heap.barrier(4 + lane)                                   # every rank has staged this weight's gradient
            C.peer_allreduce(self.in_ptrs, self.out_ptrs, self.mc_in, self.mc_out, off // es, n, grad.dtype == torch.bfloat16,
                             self.rank, 1.0 / self.W)
            _ext.count()
            heap.barrier(4 + lane)                                   # every slice of the mean has landed here
            red = self.gout[off:off + n * es].view(grad.dtype).view(grad.shape)
            self.trainer.opt.update(p, red, synced=True)
        self.used = True
        return None

    def flush(self):
        if self.small:
            flat = torch.cat([g.reshape(-1).float() for _, g in self.small])
            dist.all_reduce(flat, group=self.heap.group)
            flat /= self.W
            off = 0
            for p, g in self.small:
                n = g.numel()
                self.trainer.opt.update(p, flat[off:off + n].view_as(g).to(g.dtype), synced=True)
                off += n
            self.small.clear()
        if self.used:
            for st in self.streams:
                torch.cuda.current_stream().wait_stream(st)
            self.used = False
        if getattr(self, "pushed", False):
            self.heap.barrier(0)             # every rank's rows of the updated shadows have landed before the next forward
            self.pushed = False


class FusedParallel:
    def __init__(self, engine, wait_ms=None):
        wait_ms = wait_ms or float(os.environ.get("MEMARCH_PEER_WAIT_MS", 4000))
        self.heap = SymmetricHeap(engine.rank, engine.W, engine.group, wait_ms)
        self.ep = FusedExpertExchange(self.heap)
        self.dp = FusedGradReduce(self.heap)
        self.ctrl, ch = self.heap.alloc((4096,), torch.float32, zero=True)      # the per-step control vector
        self.ctrl_ptrs = [int(p) for p in ch.buffer_ptrs]
        self.heap.barrier(0)

    def mean_small(self, buf):
        """Mean over the ranks of a small fp32 vector, in place, on the current stream: copy into the symmetric
        control buffer, one-shot all-reduce by peer loads and stores between two device barriers, copy back (no NCCL
        kernel, no host synchronisation).  Every rank must call it at the same point of its main stream."""
        n = buf.numel()
        if n > self.ctrl.numel():
            raise ValueError(f"control vector of {n} floats exceeds the {self.ctrl.numel()}-float buffer")
        W = self.heap.W
        pad = (n + 4 * W - 1) // (4 * W) * (4 * W)                  # every rank reduces a 16-byte multiple
        self.ctrl[:n].copy_(buf)
        if pad > n:
            self.ctrl[n:pad].zero_()
        self.heap.barrier(2)
        _ext.C().peer_allreduce(self.ctrl_ptrs, self.ctrl_ptrs, 0, 0, 0, pad, False, self.heap.rank, 1.0 / W)
        _ext.count()
        self.heap.barrier(2)
        buf.copy_(self.ctrl[:n])
        return buf

    def attach(self, trainer):
        self.dp.trainer = trainer
        if os.environ.get("MEMARCH_DP", "fused") == "fused":
            self.dp.allocate(trainer.params)

    def selftest(self, tol=1e-2):
        """Small end-to-end check of the peer paths on this set of GPUs: barrier, the one-shot all-reduce (NVLS and plain
        peer loads) against NCCL, and the fused expert exchange (forward and backward) against a local computation
        from all-gathered inputs.  Returns (ok, message); every rank gets the same answer.  Costs a few host syncs,
        so it belongs before a run, not inside it."""
        heap, W, r = self.heap, self.heap.W, self.heap.rank
        dev = torch.device("cuda", torch.cuda.current_device())
        C = _ext.C()
        msg = "ok"
        self.selftest_errors = errs = {}
        try:
            heap.barrier(0)
            torch.cuda.synchronize()
            heap.check()
            # ---- all-reduce
            n = 1 << 16
            buf, bh = heap.alloc((n,), torch.float32)
            out, oh = heap.alloc((n,), torch.float32)
            g = torch.Generator(device=dev).manual_seed(100 + r)
            x = torch.randn(n, device=dev, generator=g)
            want = x.clone()
            dist.all_reduce(want, group=heap.group)
            want /= W
            ip, op = [int(p) for p in bh.buffer_ptrs], [int(p) for p in oh.buffer_ptrs]
            modes = [(0, 0)]
            try:
                if os.environ.get("MEMARCH_NVLS", "1") == "1" and int(bh.multicast_ptr) and int(oh.multicast_ptr):
                    modes.append((int(bh.multicast_ptr), int(oh.multicast_ptr)))
            except Exception:     # noqa: BLE001 - no multicast object on this system
                pass
            for mi, mo in modes:
                buf.copy_(x)
                out.zero_()
                heap.barrier(1)
                C.peer_allreduce(ip, op, mi, mo, 0, n, False, r, 1.0 / W)
                heap.barrier(1)
                torch.cuda.synchronize()
                heap.check()
                err = (out - want).abs().max().item()
                errs["allreduce_" + ("nvls" if mi else "p2p")] = err
                if not err < 1e-4:
                    raise RuntimeError(f"peer all-reduce ({'NVLS' if mi else 'P2P'}) differs from NCCL by {err:.3e}")
            # ---- fused expert exchange
            E, Cn, d, H = W, 300, 256, 512
            torch.manual_seed(7)
            up_all = (torch.randn(E, d, H, device=dev) * d ** -0.5).bfloat16()
            down_all = (torch.randn(E, H, d, device=dev) * H ** -0.5).bfloat16()
            up, down = up_all[r:r + 1].clone().requires_grad_(), down_all[r:r + 1].clone().requires_grad_()
            xe = torch.randn(E, Cn, d, device=dev, generator=g).bfloat16().requires_grad_()
            y = _FusedExpertFFN.apply(xe, up, down, self.ep, "selftest", "relu2", r, 1, True)
            go = torch.randn(E, Cn, d, device=dev, generator=g).bfloat16()
            y.backward(go)
            torch.cuda.synchronize()
            heap.check()
            xr = xe.detach().float().requires_grad_()
            yr = torch.bmm(torch.relu(torch.bmm(xr, up_all.float())) ** 2, down_all.float())
            yr.backward(go.float())
            rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-9)).item()
            e1, e2 = rel(y, yr), rel(xe.grad, xr.grad)
            errs["ep_fwd"], errs["ep_dx"] = e1, e2
            if not (e1 < tol and e2 < tol):
                raise RuntimeError(f"fused expert exchange differs from the local computation: fwd {e1:.3e}, bwd {e2:.3e}")
            # weight gradients of this rank's expert: it saw the rows that every rank routed to it
            xs, gs = [torch.empty_like(go) for _ in range(W)], [torch.empty_like(go) for _ in range(W)]
            dist.all_gather(xs, xe.detach().contiguous(), group=heap.group)
            dist.all_gather(gs, go.contiguous(), group=heap.group)
            xa, ga = torch.cat([t[r] for t in xs]).float(), torch.cat([t[r] for t in gs]).float()
            ur, dr = up_all[r].float().requires_grad_(), down_all[r].float().requires_grad_()
            ((torch.relu(xa @ ur) ** 2) @ dr).backward(ga)
            e3, e4 = rel(up.grad[0], ur.grad), rel(down.grad[0], dr.grad)
            errs["ep_dup"], errs["ep_ddown"] = e3, e4
            if not (e3 < tol and e4 < tol):
                raise RuntimeError(f"fused expert exchange: weight gradients differ: up {e3:.3e}, down {e4:.3e}")
        except Exception as e:   # noqa: BLE001 - the reason travels in the message
            msg = f"{type(e).__name__}: {e}"
        flag = torch.tensor([1.0 if msg == "ok" else 0.0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=heap.group)
        ok = bool(flag.item() > 0.5)
        return ok, (msg if msg != "ok" or ok else "another rank failed")
