"""Run guards: non-finite loss, loss-spike log, loss-spike rollback, hang watchdog.

* `NanGuard` - a non-finite loss stops the run *without* saving (train_tpu.py:1433-1436 of the reference's JAX
  trainer).  The flag accumulates on the device; the host looks at it every `every` steps, so the step loop keeps
  running ahead of the GPU.
* `SpikeLog` - `loss > spike x EMA` is logged (train_tpu.py:1437-1439).
* `RollbackGuard` - if the loss of a step exceeds `ratio` x its running mean after `warm` steps, weights, momentum and
  optimizer cards go back to the snapshot taken before the *previous* step, this step's update is discarded, and the
  next step learns again from the previous step's batch (kept on the device) with the step size x `lr_mul`; a kind of
  step that was just rejected is not rejected twice in a row (instinct.py:158-174, step.py:64-124 of the JAX port).
  Everything is a device-side select (`torch.where` on a 0-dim flag): there is no host synchronisation, hence no
  bubble in the launch queue; the price is one extra pass over weights and momentum per step, which is why the guard
  is off unless asked for.
* `Watchdog` - when no heartbeat arrives for `timeout` seconds, dump the stack of every thread plus host and device
  memory figures, and again every `repeat` seconds (diag.py:58-68).  Nothing is killed: the dump is the product.
"""
from __future__ import annotations

import faulthandler
import os
import sys
import threading
import time

import torch


class NonFiniteLoss(RuntimeError):
    pass


class NanGuard:
    def __init__(self, every=10):
        self.every, self.flag, self.n = max(1, every), None, 0

    def check(self, loss):
        bad = ~torch.isfinite(loss.detach()).all()
        self.flag = bad if self.flag is None else (self.flag | bad)
        self.n += 1
        if self.n % self.every == 0:
            self.flush()

    def flush(self):
        if self.flag is not None and bool(self.flag):
            raise NonFiniteLoss(f"loss became non-finite within the last {self.every} steps; not saving")
        self.flag = None


class SpikeLog:
    def __init__(self, spike=2.0, beta=0.98, out=None):
        self.spike, self.beta, self.ema, self.out, self.events = spike, beta, None, out or sys.stderr, []

    def check(self, step, loss):
        """Host-side (call it where the loss is read anyway, e.g. at evaluation points)."""
        loss = float(loss)
        if self.ema is not None and loss > self.spike * self.ema:
            self.events.append((step, loss, self.ema))
            print(f"[spike] step {step}: loss {loss:.4f} > {self.spike} x running mean {self.ema:.4f}", file=self.out, flush=True)
        self.ema = loss if self.ema is None else self.beta * self.ema + (1 - self.beta) * min(loss, self.spike * self.ema)


def _tensors_of(opt):
    """Every device tensor of an Instinct-like optimizer as a flat list of (owner, key, index) handles."""
    out = []
    skip = getattr(opt, "_SKIP", set())
    for k, v in vars(opt).items():
        if k in skip:
            continue
        if torch.is_tensor(v):
            out.append((k, None))
        elif isinstance(v, list) and v and all(t is None or torch.is_tensor(t) for t in v):
            out.extend((k, j) for j, t in enumerate(v) if t is not None)
    return out


def _get(opt, h):
    k, j = h
    return getattr(opt, k) if j is None else getattr(opt, k)[j]


class RollbackGuard:
    def __init__(self, trainer, ratio=1.5, beta=0.98, lr_mul=0.5, warm=50, kinds=1):
        """`kinds` > 1: one running mean of the loss and one "just rejected" flag per kind of step (`step(..., kind=k)`):
        kinds of text differ in their loss level, and a kind whose step was rejected learns at its next step, or a kind
        with a raised loss would never learn again (memarch_jax/memarch_jax/step.py:64-124 of the reference's JAX port)."""
        self.tr, self.ratio, self.beta, self.lr_mul, self.warm = trainer, ratio, beta, lr_mul, warm
        if getattr(trainer.opt, "offload", False):
            raise ValueError("the device-side rollback keeps a copy of the optimizer state on the device: "
                             "it cannot be combined with the host offload of the momentum (offload_m)")
        dev = trainer.device
        self.lema = torch.zeros(kinds, device=dev)         # running mean of the loss per kind (0 = not started)
        self.rep = torch.zeros((), dtype=torch.bool, device=dev)     # next step replays the kept batch
        self.cool = torch.zeros(kinds, dtype=torch.bool, device=dev)  # the kind's last step was rejected: not again
        self.n_hit = torch.zeros((), dtype=torch.long, device=dev)
        self.n = 0
        self.prev_xy = None
        self.snap_p = self.snap_o = None
        self.handles = None
        self.one = torch.ones((), device=dev)

    def _state(self):
        tr = self.tr
        if self.handles is None:
            self.handles = _tensors_of(tr.opt) if hasattr(tr.opt, "plist") else []
        return [p.data for p in tr.params], [_get(tr.opt, h) for h in self.handles]

    @torch.no_grad()
    def step(self, xy, step, kind=0, **kw):
        tr = self.tr
        k = min(max(int(kind), 0), self.lema.numel() - 1)
        if self.prev_xy is not None and self.prev_xy.shape != xy.shape:
            # a step of another shape (a batch of short synthetic rows): it is neither judged nor kept for a replay,
            # but the state before it becomes the snapshot, so the next ordinary step can still undo its update
            ps, os_ = self._state()
            before_p, before_o = [t.clone() for t in ps], [t.clone() for t in os_]
            with torch.enable_grad():
                loss = tr.step(xy, step, **kw)
            self.snap_p, self.snap_o = before_p, before_o
            self.n += 1
            return loss
        if self.prev_xy is None:
            self.prev_xy = xy.clone()
        xy_eff = torch.where(self.rep, self.prev_xy, xy)
        if hasattr(tr.opt, "lr_mul_dev"):
            tr.opt.lr_mul_dev = torch.where(self.rep, self.one * self.lr_mul, self.one)
        ps, os_ = self._state()
        before_p, before_o = [t.clone() for t in ps], [t.clone() for t in os_]
        with torch.enable_grad():
            loss = tr.step(xy_eff, step, **kw)
        l = loss.detach().float()
        par = getattr(tr, "parallel", None)
        if par is not None and hasattr(par, "mean_vector"):
            l = par.mean_vector(l.reshape(1).clone())[0]     # one verdict for all ranks: weights must stay equal
        lema = self.lema[k]
        hit = (l > self.ratio * lema) & (lema > 0) & ~self.cool[k] & ~self.rep
        if self.n < self.warm or self.snap_p is None:
            hit = torch.zeros_like(hit)
        if self.snap_p is not None:
            ps2, os2 = self._state()                        # the optimizer may have re-bound tensors (rebank)
            if len(ps2) == len(self.snap_p) and all(a.shape == b.shape for a, b in zip(ps2, self.snap_p)):
                for t, s in zip(ps2, self.snap_p):
                    t.copy_(torch.where(hit, s, t))
                for t, s in zip(os2, self.snap_o):
                    if t.shape == s.shape:
                        t.copy_(torch.where(hit, s, t))
        # new snapshot: the state before this step; kept batch: this step's batch unless a replay is pending
        self.snap_p, self.snap_o = before_p, before_o
        self.prev_xy = torch.where(hit, self.prev_xy, xy_eff)
        new_l = torch.where(lema > 0, self.beta * lema + (1 - self.beta) * torch.minimum(l, lema * self.ratio), l)
        self.lema[k] = torch.where(self.rep, lema, new_l)
        self.cool[k] = torch.where(self.rep, self.cool[k], hit)          # a replayed batch leaves the kind's flag alone
        self.rep = hit
        self.n_hit += hit.long()
        self.n += 1
        return loss


class Watchdog:
    def __init__(self, timeout=180.0, repeat=120.0, out=None, on_fire=None):
        self.timeout, self.repeat, self.out, self.on_fire = timeout, repeat, out, on_fire
        self.last = time.monotonic()
        self.fired = 0
        self._stop = threading.Event()
        self.t = threading.Thread(target=self._run, daemon=True)
        self.t.start()

    def beat(self):
        self.last = time.monotonic()

    def _dump(self):
        f = self.out or sys.stderr
        idle = time.monotonic() - self.last
        print(f"[watchdog] no progress for {idle:.0f}s; thread stacks follow", file=f, flush=True)
        try:
            faulthandler.dump_traceback(file=f, all_threads=True)
        except Exception:   # noqa: BLE001 - file objects without a descriptor
            import traceback
            for tid, fr in sys._current_frames().items():
                print(f"--- thread {tid}", file=f)
                traceback.print_stack(fr, file=f)
        try:
            import psutil
            vm = psutil.virtual_memory()
            print(f"[watchdog] host rss {psutil.Process(os.getpid()).memory_info().rss / 2**30:.2f} GiB, "
                  f"available {vm.available / 2**30:.1f} GiB", file=f, flush=True)
        except Exception:   # noqa: BLE001
            pass
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            print(f"[watchdog] device allocated {torch.cuda.memory_allocated() / 2**30:.2f} GiB, "
                  f"reserved {torch.cuda.memory_reserved() / 2**30:.2f} GiB", file=f, flush=True)

    def _run(self):
        next_at = self.timeout
        while not self._stop.wait(min(1.0, self.timeout / 4)):
            idle = time.monotonic() - self.last
            if idle < self.timeout:
                next_at = self.timeout
                continue
            if idle >= next_at:
                self.fired += 1
                self._dump()
                if self.on_fire:
                    self.on_fire(self.fired)
                next_at = idle + self.repeat

    def close(self):
        self._stop.set()
        self.t.join(timeout=2)
