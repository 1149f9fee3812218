"""Trainer: one training step with no host synchronisation, weights updated inside backward.

Stage letters follow the reference (fastloop.py:1-13, 217-497): `A` tokens resident on the device and no per-step
host sync; `B` each weight is stepped from its grad-ready hook on the last micro-batch; `X` the Instinct optimizer
(with `B`: device-only `prepare -> update -> finish`); `S` SurpriseAdamW; `C` micro-batches forward on separate
CUDA streams with one backward; `G` the step is replayed as a CUDA graph.  Without `B` gradients are clipped to 1.0.
"""
from __future__ import annotations

import math

import torch

from ..config import OptConfig, TrainConfig
from ..optim.instinct import Instinct, SurpriseAdamW


def lr_at(step, cfg: TrainConfig):
    """Warm-up then cosine to 0.1·lr, or WSD: flat, then linear to `lr_floor` over the last `wsd_frac` of steps
    (fastloop.py:52-60)."""
    up = min(1, (step + 1) / max(cfg.warmup, 1))
    if cfg.lr_sched == "wsd":
        d0 = (1 - cfg.wsd_frac) * cfg.steps
        if step < d0:
            return cfg.lr * up
        return cfg.lr * up * (1 - (1 - cfg.lr_floor) * min(1, (step - d0) / max(cfg.steps - d0, 1e-9)))
    return cfg.lr * up * (0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * min(1, step / max(cfg.steps, 1)))))


def cast_linear_weights(model, dtype=torch.bfloat16):
    """Linear weights (outside memory / reread, which stay fp32 on purpose) live in `dtype`; the optimizer keeps the
    exact fp32 copy (the reference's BF16_W, fastloop.py:223-228)."""
    for nm, mod in model.named_modules():
        if isinstance(mod, torch.nn.Linear) and not nm.startswith(("memory", "reread")):
            mod.weight = torch.nn.Parameter(mod.weight.detach().to(dtype))
    return model


class Trainer:
    def __init__(self, model, tcfg: TrainConfig, ocfg: OptConfig = None, stage=None, parallel=None, graph=None):
        self.model, self.cfg = model, tcfg
        self.stage = stage or tcfg.stage
        import os
        self.graph = ("G" in self.stage or os.environ.get("MEMARCH_GRAPH") == "1") if graph is None else bool(graph)
        self._graphs, self._graph_pool, self._eager_steps, self._graph_failed = {}, None, 0, False
        self.ocfg = ocfg or OptConfig(lr=tcfg.lr)
        self.parallel = parallel
        dev = next(model.parameters()).device
        self.device = dev
        if dev.type == "cuda" and self.ocfg.bf16_weights and "X" in self.stage:
            cast_linear_weights(model)
        if parallel is not None:
            parallel.shard_model(model)
        self.params = [p for p in model.parameters() if p.requires_grad]
        st = self.stage
        self.apply_now = False
        self.card = None                 # kind of the coming step (a number), for `OptConfig.card_by_kind`
        self.acc = {}
        if "X" in st and self.ocfg.kind == "instinct":
            import dataclasses
            by_id = {id(p): n for n, p in model.named_parameters()}
            self.opt = Instinct(self.params, dataclasses.replace(self.ocfg, lr=tcfg.lr),
                                names=[by_id.get(id(p), "") for p in self.params])
            self.in_backward = "B" in st and self.ocfg.in_backward
            if (self.ocfg.stream_proj or self.ocfg.m_rate) and hasattr(model, "want_stream_mean"):
                model.want_stream_mean = True
            if parallel is not None:
                parallel.attach(self)
            # Graph mode runs the whole step on one private stream: the per-parameter AccumulateGrad nodes (kept alive
            # by the hooks) remember the stream they were created on, and capture needs it to be the capturing stream.
            self._gstream = torch.cuda.Stream() if (self.graph and dev.type == "cuda") else None
            if self.in_backward:
                import contextlib
                with (torch.cuda.stream(self._gstream) if self._gstream is not None else contextlib.nullcontext()):
                    for p in self.params:
                        p.register_post_accumulate_grad_hook(self._hook)
        elif "X" in st and self.ocfg.kind == "experience":
            from ..optim.experience import ExperienceOpt
            self.opt = ExperienceOpt(self.params, lr=tcfg.lr, weight_decay=0.1, cards=self.ocfg.cards, beta=self.ocfg.beta,
                                     new_card=self.ocfg.new_card, ema=self.ocfg.ema, norm=self.ocfg.norm,
                                     scale=self.ocfg.scale, m_dtype="bf16" if self.ocfg.m_bf16 else "fp32")
            self.in_backward = False
        elif self.ocfg.kind == "muon":
            from ..optim.muon import MuonAdamW
            self.opt = MuonAdamW(self.params, lr=tcfg.lr, weight_decay=0.1, betas=(0.9, 0.95), mul=self.ocfg.muon_mul)
            self.in_backward = False
        elif "S" in st:
            self.opt = SurpriseAdamW(self.params, lr=tcfg.lr, betas=(0.9, 0.95), weight_decay=0.1)
            self.in_backward = False
        else:
            self.opt = torch.optim.AdamW(self.params, lr=tcfg.lr, betas=(0.9, 0.95), weight_decay=0.1,
                                         fused=dev.type == "cuda")
            self.in_backward = False
        self.streams = None
        self.last_loss = None
        if not hasattr(self, "_gstream"):
            self._gstream = None

    # ------------------------------------------------------------------------------------------ hooks
    def _direct_grad(self, p, g):
        """bf16 weight gradient handed over by `ops.basic._WeightBf16`: step the weight now (last micro-batch, nothing
        accumulated yet, the weight is one of this trainer's) or decline."""
        if not (self.in_backward and self.apply_now) or p.grad is not None or id(p) not in self.opt.idx:
            return False
        self.opt.update(p, g.contiguous())
        return True

    def _hook(self, p):
        """Grad-ready hook: accumulate until the last micro-batch, then step this weight and drop its grad."""
        if p.grad is None:
            return
        if not self.apply_now:
            return                                   # autograd keeps accumulating into p.grad
        self.opt.update(p)
        p.grad = None

    def register_new_param(self, p):
        if self.in_backward:
            import contextlib
            with (torch.cuda.stream(self._gstream) if self._gstream is not None else contextlib.nullcontext()):
                p.register_post_accumulate_grad_hook(self._hook)

    # ------------------------------------------------------------------------------------------ loss
    def loss_fn(self, xy, prep=None):
        m = self.model
        x_in, y_t = xy[:, :-1], xy[:, 1:]
        out, cost = m(x_in, prep) if prep is not None else m(x_in)
        needles = prep.get("remind") if isinstance(prep, dict) else None
        loss = m.train_loss(out, y_t, True, extra=needles) if needles is not None else m.train_loss(out, y_t, True)
        return loss + self.cfg.read_cost * cost.float()

    def set_lr(self, step, mul=1.0):
        lr = lr_at(step, self.cfg) * mul
        for g in self.opt.param_groups:
            g["lr"] = lr

    def _stream_to_opt(self):
        sm = getattr(self.model, "stats", {}).get("stream_mean") if (self.ocfg.stream_proj or self.ocfg.m_rate) else None
        if sm is not None:
            if self.parallel is not None and hasattr(self.parallel, "mean_vector"):
                sm = self.parallel.mean_vector(sm.clone())
            self.opt.observe_stream(sm)
            if hasattr(self.model, "stream_u"):
                self.model.stream_u = self.opt.U         # the final norm's `norm_dump_proj` uses the same direction

    def situation(self, xy):
        with torch.no_grad():
            return self.model.emb(xy[:, :-1]).float().mean((0, 1))

    # ------------------------------------------------------------------------------------------ step
    def step(self, xy, step, preps=None, lr_mul=1.0):
        """One training step; returns the loss as a device tensor (no host sync).

        With stage `G` (or `graph=True`) the device work of the step - forward, backward with the weight updates in
        its hooks, gradient exchange, optimizer bookkeeping - is captured once per (shape, |g|/|w|-step or not) as a
        CUDA graph after three eager steps and replayed afterwards: one launch per step instead of ~2000."""
        if self._gstream is not None and xy.is_cuda:
            cur = torch.cuda.current_stream()
            self._gstream.wait_stream(cur)
            with torch.cuda.stream(self._gstream):
                total = self._step(xy, step, preps, lr_mul)
            cur.wait_stream(self._gstream)
            return total
        return self._step(xy, step, preps, lr_mul)

    def _step(self, xy, step, preps, lr_mul):
        self.set_lr(step, lr_mul)
        m = self.model
        if hasattr(m, "before_step"):
            m.before_step(step)
        inst = isinstance(self.opt, Instinct)
        if inst:
            self.opt._sync_lr()
        host_rules = self.ocfg.m_rate or self.ocfg.culprit == "ema"      # their step counters live on the host
        if self.graph and xy.is_cuda and preps is None and inst and "C" not in self.stage and not host_rules:
            total = self._step_graphed(xy)
        else:
            total = self._core(xy, preps)
        if inst and hasattr(m, "rebank"):
            self._apply_rebank(m.rebank(step))
        self.last_loss = total
        return total

    def _step_graphed(self, xy):
        # host-side choices that shape the captured program (which heavy layer is full, the hoop's budget) are part of the key
        key = (tuple(xy.shape), self.opt.n_step % self.opt.rel_every == 0, getattr(self.model, "graph_key", tuple)())
        if self._eager_steps < 3 or self._graph_failed:
            self._eager_steps += 1
            return self._core(xy, None)
        ent = self._graphs.get(key)
        if ent is None:
            from ..ops import _ext
            static_xy = xy.clone()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            n0, f0, step0 = _ext.launch_count, _ext.gemm_flops, self.opt.n_step
            try:
                with torch.cuda.graph(g, pool=self._graph_pool, stream=self._gstream):
                    out = self._core(static_xy, None)
            except Exception as e:   # noqa: BLE001 - capture is an optimisation; the eager path is always there
                import warnings
                warnings.warn(f"CUDA graph capture of the training step failed ({type(e).__name__}: {e}); running eagerly")
                self._graph_failed = True
                torch.cuda.synchronize()
                return self._core(xy, None)
            if self._graph_pool is None:
                self._graph_pool = g.pool()
            ent = self._graphs[key] = (g, static_xy, out, _ext.launch_count - n0, _ext.gemm_flops - f0)
            self.opt.n_step = step0              # capture ran the host bookkeeping once; the replay below is the real step
        g, static_xy, out, launches, flops = ent
        static_xy.copy_(xy)
        g.replay()
        self.opt.n_step += 1
        from ..ops import _ext
        _ext.count(launches)
        _ext.count_flops(flops)
        return out

    def _core(self, xy, preps=None):
        """Device work of one step: micro-batches forward/backward (weights stepped in the grad hooks), exchange, finish."""
        m = self.model
        from ..ops import basic
        basic.WEIGHT_GRAD_SINK = self._direct_grad if (getattr(self, "in_backward", False) and isinstance(self.opt, Instinct)) else None
        micro = self.cfg.micro or len(xy)
        mbs = xy.split(micro)
        inst = isinstance(self.opt, Instinct)
        if inst and self.ocfg.sparse_rows and hasattr(m, "table_rows"):
            self.opt.rows = m.table_rows(xy[:, :-1])
        if "C" in self.stage and xy.is_cuda and len(mbs) > 1:
            return self._step_interleaved(mbs, len(xy), xy)
        total = torch.zeros((), device=xy.device)
        for i, mb in enumerate(mbs):
            last = i == len(mbs) - 1
            self.apply_now = last
            loss = self.loss_fn(mb, preps[i] if preps is not None else None)
            w = len(mb) / len(xy)
            if inst and last:
                tl = total + loss.detach() * w
                sit = self.situation(xy)
                if self.parallel is not None:
                    tl, sit = self.parallel.sync_control(tl, sit, m)
                self._stream_to_opt()
                self.opt.prepare(tl, sit, card=self.card)
            if self.parallel is not None:
                self.parallel.before_backward(self)
            (loss * w).backward()
            total = total + loss.detach() * w
        self._after_backward(total, xy)
        return total

    def _after_backward(self, total, xy):
        inst = isinstance(self.opt, Instinct)
        if inst:
            if self.parallel is not None:
                self.parallel.after_backward(self)
            if not self.in_backward:
                self.opt.update_all()
            self.opt.finish()
        else:
            if self.parallel is not None:
                self.parallel.reduce_grads(self.params)
            torch.nn.utils.clip_grad_norm_(self.params, 1.0)
            if isinstance(self.opt, SurpriseAdamW):
                self.opt.step(total)
            elif hasattr(self.opt, "pick"):                       # experience cards: loss (host read) and situation
                self.opt.step(total, self.situation(xy))
            else:
                self.opt.step()
            self.opt.zero_grad(set_to_none=True)

    def _apply_rebank(self, changes):
        """Experts moved between banks: the optimizer follows the new tensors (momentum by position)."""
        for old, new, slot_map in changes:
            self.opt.swap(old, new, slot_map)
            self.register_new_param(new)
        if changes:
            self.params = [p for p in self.model.parameters() if p.requires_grad]

    def _step_interleaved(self, mbs, n, xy):
        """Stage C: independent micro-batches run forward on their own streams, one backward for all."""
        if self.streams is None or len(self.streams) != len(mbs):
            self.streams = [torch.cuda.Stream() for _ in mbs]
        cur = torch.cuda.current_stream()
        losses = []
        for s, mb in zip(self.streams, mbs):
            s.wait_stream(cur)
            mb.record_stream(s)
            with torch.cuda.stream(s):
                losses.append(self.loss_fn(mb) * len(mb) / n)
        for s in self.streams:
            cur.wait_stream(s)
        total = torch.stack(losses).sum()
        self.apply_now = True
        if isinstance(self.opt, Instinct):
            self._stream_to_opt()
            self.opt.prepare(total.detach(), self.situation(xy), card=self.card)
        total.backward()
        self._after_backward(total.detach(), xy)
        return total.detach()


@torch.no_grad()
def val_loss(model, store, seq, n=20, batch=8):
    """Fixed validation windows (generator seed 0), mean token CE (fastloop.py:500-515)."""
    was = model.training
    model.eval()
    g = torch.Generator(device=store.device).manual_seed(0)
    t = store.t
    total = torch.zeros((), device=store.device)
    for _ in range(n):
        start = torch.randint(0, len(t) - seq - 1, (batch,), device=store.device, generator=g)
        xy = t[start[:, None] + torch.arange(seq + 1, device=store.device)].long()
        out, _ = model(xy[:, :-1])
        total += model.train_loss(out, xy[:, 1:], False)
    model.train(was)
    return total / n
