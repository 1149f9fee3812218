"""Instinct: a one-momentum optimizer whose step is scaled by loss surprise per "situation card", with
homeostasis normalisation (row -> column -> row) of the update, applied to each weight the moment its gradient is
ready inside backward.  No value ever travels to the host.

API and state names follow the reference's `InstinctOptB` (exp_opt.py:428-729) so its checkpoints load:
`prepare(loss, situation)` -> `update(p)` per parameter (from the grad-ready hook) or `update_all()` ->
`finish()`; `swap(old, new, slot_map)` after a re-bank.  State: `m` (per-parameter momentum, fp32 or bf16), `w` (exact
fp32 copy of bf16 weights), `gain (K,P)`, `keys (K,d)`, `used`, `expect`, `seen`, `rel (P,)`, `k, s, stake, g, oh`,
`cs` (lagged second-axis mean squares), `n_step`.

Step kinds by shape (exp_opt.py:653-665): 2-D tables with >= 10 000 rows -> "vocab" (row-rms, only rows with a
non-zero gradient move, no weight decay); 2-D -> "hs"; 3-D experts (E, in, out) -> "hs3" (norm over in, out, in);
everything else -> "tensor".  With norm="row"/"tensor"/"hs<n>" the reference's other kinds apply.

GPU body: `instinct_stat` / `instinct_apply` kernels (csrc/instinct.cu): fp32 math, weight decay, optional
counter-hash stochastic rounding of bf16 stores, |g|/|w| every `rel_every` steps.  CPU body: `ops.ref`.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..config import OptConfig
from ..ops import _ext, ref


def _kind_code(kind):
    """Kernel form of a normalisation kind, -1 = PyTorch statement (hsn<n> with two or more "columns, rows" rounds;
    one round, `norm="hs1"`, is `hs` itself and takes its kernels - see `Instinct.spec`)."""
    return {"tensor": 0, "row": 1, "row3": 2, "vocab": 3, "hs": 4, "hs3": 5}.get(kind, -1)


class Instinct:
    def __init__(self, params, cfg: OptConfig = None, d_sit=None, names=None, **kw):
        cfg = cfg or OptConfig()
        if kw:
            import dataclasses
            cfg = dataclasses.replace(cfg, **{k: v for k, v in kw.items() if k in OptConfig.__dataclass_fields__})
        self.cfg = cfg
        self.m_dtype = torch.bfloat16 if cfg.m_bf16 else torch.float32
        self.rel_every, self.n_step = cfg.rel_every, 0
        self.plist = list(params)
        self.idx = {id(p): i for i, p in enumerate(self.plist)}
        # parameter names (optional): the switches that address weights by name need them (wd_norm, norm_anchor, lr_mul)
        self.names = list(names) if names is not None else [""] * len(self.plist)
        is_norm = lambda n: n in ("norm.weight", "l_norm.weight") or n.endswith((".n1.weight", ".n2.weight"))
        self._norm_w = [p.dim() == 1 and is_norm(n) for p, n in zip(self.plist, self.names)]
        self._anchor = [nw and n.startswith(("light_a.", "light_b.", "final.")) for nw, n in zip(self._norm_w, self.names)]
        # safe16: the light blocks and the two output norms take their step direction from a momentum that never
        # moves against the fresh gradient (PyTorch statement of the update; the stored momentum stays the plain EMA)
        self._safe = [bool(cfg.safe16) and (n.startswith(tuple(cfg.safe16_prefix)) or n in ("norm.weight", "l_norm.weight"))
                      for n in self.names]
        self._snr_on = [not n.startswith(tuple(cfg.snr_skip)) and (not cfg.snr_only or n.startswith(tuple(cfg.snr_only)))
                        if (cfg.snr_skip or cfg.snr_only) else True for n in self.names]
        self._mul = [next((float(m) for pref, m in cfg.lr_mul if n.startswith(pref)), 1.0) for n in self.names]
        self.param_groups = [dict(lr=cfg.lr, weight_decay=cfg.weight_decay)]
        self.K, self.beta, self.new_card, self.ema = cfg.cards, cfg.beta, cfg.new_card, cfg.ema
        self.good, self.bad, self.top, self.relax = cfg.good, cfg.bad, cfg.top, cfg.relax
        self.scale, self.norm = cfg.scale, cfg.norm
        self.lr_peak = cfg.lr_peak or cfg.lr
        self.hs_lag, self.sr = cfg.hs_lag, cfg.sr
        dev = self.plist[0].device
        P = len(self.plist)
        self.gain = torch.ones(cfg.cards, P, device=dev)
        self.keys = None
        self.used = torch.zeros(cfg.cards, dtype=torch.bool, device=dev)
        self.expect = torch.zeros(cfg.cards, device=dev)
        self.seen = torch.zeros(cfg.cards, device=dev)
        self.rel = torch.zeros(P, device=dev)
        # culprit="ema": a tensor is to blame for a bad step when its |g|/|w| is high against ITS OWN running mean,
        # not against the other tensors (whose ranking hardly changes, so the same few were blamed at every step)
        self.culprit, self.g_max, self.card_by_kind = cfg.culprit, cfg.g_max, cfg.card_by_kind
        if self.culprit not in ("abs", "ema"):
            raise ValueError(f"culprit must be 'abs' or 'ema', not {cfg.culprit!r}")
        if self.culprit == "ema":
            self.rel_avg = torch.zeros(P, device=dev)
        # rules on the stream's common vector (stream_proj, m_rate): the matrices of the light blocks that write into or
        # read from the residual stream, and along which of their axes the stream runs.  The JAX port addresses "the
        # first axis of size d" of its (in, out) layout; weights here are (out, in), hence the axes in reverse order
        self.U = None
        self._stream_ax = [None] * P
        if cfg.stream_proj or cfg.m_rate:
            hit = lambda n: n.startswith(("light_a.", "light_b.", "final.")) and n.endswith((".o.weight", ".down.weight", ".qkv.weight"))
            d = cfg.stream_d or min((p.shape[-1] for p, n in zip(self.plist, self.names) if p.dim() >= 2 and hit(n)), default=0)
            for j, (p, n) in enumerate(zip(self.plist, self.names)):
                if p.dim() >= 2 and hit(n):
                    self._stream_ax[j] = next((ax for ax in reversed(range(p.dim())) if p.shape[ax] == d), None)
            if cfg.m_rate:
                self.mrl_n = 0
                shape = lambda p, ax: p.shape[:ax] + p.shape[ax + 1:]
                self.mrl_bank = [None if ax is None else torch.zeros(shape(p, ax), device=dev) for p, ax in zip(self.plist, self._stream_ax)]
                self.mrl_v = [None if b is None else torch.zeros_like(b) for b in self.mrl_bank]
                self.mrl_base = [None if b is None else torch.zeros((), device=dev) for b in self.mrl_bank]
                self.mrl_cut = torch.zeros((), device=dev)
        self.m = [torch.zeros_like(p, dtype=self.m_dtype) for p in self.plist]
        # optimizer-state offload (memarch_jax/memarch_jax/dist.py:311-322, step.py:154-155): the momentum of every weight
        # rests in pinned host memory and visits the device only for its own update, on the stream of that update
        self.offload = bool(cfg.offload_m)
        if self.offload:
            self.m = [self._to_host(t) for t in self.m]
        self.w = [p.detach().float().clone() if (p.dtype == torch.bfloat16 and not cfg.no_master) else None
                  for p in self.plist]
        self.cs = [None] * P
        self.cs_ok = [None] * P        # lagged form on the GPU: device flag "every entry of cs is positive"
        self.k = torch.zeros((), dtype=torch.long, device=dev)
        self.s = torch.zeros((), device=dev)
        self.stake = torch.zeros((), device=dev)
        self.g = torch.ones(P, device=dev)
        self.oh = torch.zeros(cfg.cards, device=dev)
        self._lr_t = torch.zeros((), device=dev)
        self._lr_v = torch.zeros((), device=dev)
        self._lr_ratio = torch.zeros((), device=dev)
        self._seed_t = torch.zeros((), dtype=torch.int64, device=dev)
        self._lr_last = None
        self.lr_mul_dev = None         # optional 0-dim device tensor multiplying the step (set by the rollback guard)
        self.dv = torch.zeros(cfg.cards, P, device=dev) if cfg.damp > 0 else None   # usual |g|^2 per (card, weight)
        self.df = torch.ones(P, device=dev) if cfg.damp > 0 else None               # last damping factor (for the log)
        geared = cfg.damp > 0 and cfg.gearbox
        self.gear = torch.full((P,), 2, dtype=torch.long, device=dev) if geared else None   # index into the gear table
        self.speed = torch.ones(P, device=dev) if geared else None                          # current step multiplier
        self.snr_v = torch.zeros(P, device=dev) if cfg.snr else None                # EMA of |g|^2 (or of c^2, dead-zone form)
        self.snr_f = torch.ones(P, device=dev) if cfg.snr else None                 # last factor (for the log)
        self.rows = {}
        self._scratch = {}
        self.grad_sync = None          # set by the data-parallel engine: called as grad_sync(p, grad) -> grad

    @staticmethod
    def _to_host(t):
        h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=torch.cuda.is_available())
        h.copy_(t)
        return h

    # ------------------------------------------------------------------------------------------ card logic
    @torch.no_grad()
    def observe_stream(self, stream_mean, update=True, beta=0.9):
        """U <- unit(beta U + (1 - beta) unit(mean state of the stream before the final norm)); the first time just the
        unit mean (memarch_jax/memarch_jax/instinct.py:370-383)."""
        mv = F.normalize(stream_mean.detach().float().flatten(), dim=0, eps=1e-8)
        if self.U is None:
            self.U = mv.clone()
        elif update:
            self.U.copy_(F.normalize(beta * self.U + (1 - beta) * mv, dim=0, eps=1e-8))

    def prepare(self, loss, situation, card=None):
        """Pick the situation card, its expectation and the surprise of this step's loss (exp_opt.py:349-372).
        With `card_by_kind` and a `card` number the kind of the step names the card instead of the similarity of the
        input (memarch_jax/memarch_jax/instinct.py:486-495)."""
        sit = F.normalize(situation.float().flatten(), dim=0)
        if self.keys is None:
            self.keys = torch.zeros(self.K, sit.numel(), device=sit.device)
        self._sync_lr()
        used = self.used
        if self.card_by_kind and card is not None:
            k = torch.as_tensor(card, device=sit.device).long().reshape(()).clamp(0, self.K - 1)
        else:
            best_sim, best = (self.keys @ sit).masked_fill(~used, -2).max(0)
            free = ~used
            first_free = free.int().argmax()
            newer = (best_sim < self.new_card) & free.any()
            k = torch.where(~used.any(), torch.zeros_like(best), torch.where(newer, first_free, best))
        oh = F.one_hot(k, self.K).float()
        was = (oh * used).sum() > 0
        key_k = oh @ self.keys
        new_key = torch.where(was, F.normalize(0.95 * key_k + 0.05 * sit, dim=0), sit)
        self.keys.add_(oh[:, None] * (new_key - key_k)[None])
        self.used.copy_(used | oh.bool())
        loss = loss.detach().float()
        e = torch.where((oh * self.seen).sum() > 0, (oh * self.expect).sum(), loss)
        self.s = (e - loss) / e.clamp(min=1e-6)
        self.expect.add_(oh * (self.ema * e + (1 - self.ema) * loss - self.expect))
        self.seen.add_(oh * (1 - self.seen))
        self.stake = (4 * self.s.abs() + 0.5 * self._lr_ratio).clamp(max=1.0)
        self.k, self.oh = k, oh
        self.g = oh @ self.gain

    @torch.no_grad()
    def finish(self):
        """The instinct learns: gains of the card move by the outcome of the step (exp_opt.py:375-383)."""
        s, gk = self.s, self.g.clone()
        if self.culprit == "ema":
            avg = torch.where(self.rel_avg > 0, self.rel_avg, self.rel)      # the first time: no surprise
            ratio = self.rel / (avg + 1e-12)
            culprit = (ratio >= ratio.quantile(1 - self.top)).float()
            fresh = self.n_step % self.rel_every == 0                         # |g|/|w| was measured at this very step
            self.rel_avg.copy_(0.9 * avg + 0.1 * self.rel if fresh else avg)
        else:
            culprit = (self.rel >= self.rel.quantile(1 - self.top)).float()
        self.n_step += 1
        if self.cfg.m_rate and self.U is not None:
            self.mrl_n += 1
        gk += torch.where(s < 0, culprit * self.bad * (-s * 10).clamp(max=1), torch.zeros_like(gk))
        gk += torch.where(s > 0, self.good * (s * 10).clamp(max=1) * (1 - gk), torch.zeros_like(gk))
        gk += self.relax * (1 - gk)
        gk = gk.clamp(0.5, self.g_max)
        self.gain.add_(self.oh[:, None] * (gk / gk.mean() - self.gain))

    def _sync_lr(self):
        lr = self.param_groups[0]["lr"]
        if self.lr_mul_dev is not None:                       # device-side multiplier: no host sync, rewritten every step
            self._lr_t.copy_(self.lr_mul_dev * (lr * self.scale))
            self._lr_v.copy_(self.lr_mul_dev * (lr * self.scale * self.cfg.vocab_lr_mul))
            self._lr_ratio.fill_(lr / self.lr_peak)
            self._lr_last = None
        elif self._lr_last != lr:
            self._lr_t.fill_(lr * self.scale)
            self._lr_v.fill_(lr * self.scale * self.cfg.vocab_lr_mul)
            self._lr_ratio.fill_(lr / self.lr_peak)
            self._lr_last = lr

    # ------------------------------------------------------------------------------------------ per-weight step
    def spec(self, p):
        """(kind, has weight decay, is a word table) from the weight's shape (exp_opt.py:653-665)."""
        vocab_table = p.dim() == 2 and (p.shape[0] >= 10000 or getattr(p, "_vocab_table", False))
        n = "hs" if self.norm == "hs1" else self.norm          # one homeostasis round is the plain form
        if vocab_table:
            kind = "vocab"
        elif n == "row" and p.dim() == 3:
            kind = "row3"
        elif n.startswith("hs") and n != "hs" and p.dim() == 3:
            kind = n.replace("hs", "hsn") + "e"
        elif n.startswith("hs") and n != "hs" and p.dim() == 2:
            kind = n.replace("hs", "hsn")
        elif n == "hs" and p.dim() == 3:
            kind = "hs3"
        elif n == "hs" and p.dim() == 2:
            kind = "hs"
        elif (n in ("row", "row_old") or n.startswith("hs")) and p.dim() >= 2:
            kind = "row"
        else:
            kind = "tensor"
        wd = bool(self.param_groups[0]["weight_decay"]) and p.dim() >= 2 and not vocab_table
        return kind, wd, vocab_table

    @torch.no_grad()
    def update(self, p, grad=None, synced=False):
        """One Instinct step of one weight; called from the weight's grad-ready hook.  With a data-parallel engine
        attached the gradient first goes through `grad_sync`, which may defer the step (returns None) and call back
        with `synced=True` once the rank-mean gradient is there."""
        i = self.idx[id(p)]
        grad = p.grad if grad is None else grad
        if grad is None:
            return
        if self.grad_sync is not None and not synced:
            grad = self.grad_sync(p, grad)
            if grad is None:
                return
        if not self.offload:
            return self._step_one(i, p, grad)
        home = self.m[i]
        self.m[i] = home.to(p.device, non_blocking=True)
        try:
            self._step_one(i, p, grad)
            home.copy_(self.m[i], non_blocking=True)
        finally:
            self.m[i] = home

    def _step_one(self, i, p, grad):
        """A weight stacked over units of which only a few work in a step (`p._idle_rows`, the layer pool of
        `models.fishki`): a unit whose gradient is all zero stays exactly as it was - no weight decay, no coasting on
        momentum - as an unused parameter does under an optimizer that skips `grad is None`.  Otherwise weight decay
        would wipe a unit that idles 97 % of the steps (the JAX Instinct's `_freeze_idle`, instinct.py:1165-1195)."""
        if not getattr(p, "_idle_rows", False):
            return self._step_stream(i, p, grad)
        n = p.shape[0]
        act = (grad.reshape(n, -1).abs().sum(1) > 0)
        pick = lambda new, old: torch.where(act.view(-1, *([1] * (new.dim() - 1))), new, old.to(new.dtype))
        old_p, old_m = p.detach().clone(), self.m[i].clone()
        old_w = self.w[i].clone() if self.w[i] is not None else None
        old_cs = self.cs[i].clone() if torch.is_tensor(self.cs[i]) else None
        self._step_stream(i, p, grad)
        p.data.copy_(pick(p.data, old_p))
        self.m[i].copy_(pick(self.m[i], old_m))
        if old_w is not None:
            self.w[i].copy_(pick(self.w[i], old_w))
        cs = self.cs[i]
        if old_cs is not None and torch.is_tensor(cs) and cs.shape == old_cs.shape and cs.shape[:1] == (n,):
            cs.copy_(pick(cs, old_cs))                  # only statistics that run over the units

    def _step_stream(self, i, p, grad):
        """The two rules on the stream's common vector U (the running mean direction of the state before the final
        norm), for the matrices of the light blocks.  `stream_proj`: the component along U is taken out of the gradient
        and of the momentum, so the optimizer itself never pulls on the common vector.  `m_rate`: after the step the
        U-component of the weight's move, c = dW.U, is limited by its coherent speed v = EMA(c) <= kappa x its usual
        size; the excess waits in a bank and is released by later steps, nothing is thrown away (with `m_rate_gate`
        only where the fresh gradient still agrees).  (instinct.py:370-484 of the reference's JAX port)"""
        ax = self._stream_ax[i]
        if ax is None or self.U is None:
            return self._step_body(i, p, grad)
        c = self.cfg
        U = self.U

        def off(x):
            xf = x.float().movedim(ax, -1)
            return (xf - (xf @ U)[..., None] * U).movedim(-1, ax).to(x.dtype)
        if c.stream_proj:
            grad = off(grad)
            self.m[i].copy_(off(self.m[i]))
        if not c.m_rate:
            return self._step_body(i, p, grad)
        t = self.w[i] if self.w[i] is not None else p.data
        old = t.detach().float().clone()
        self._step_body(i, p, grad)
        new = t.float().movedim(ax, -1)
        moved = (new - old.movedim(ax, -1)) @ U
        bank, v, base = self.mrl_bank[i], self.mrl_v[i], self.mrl_base[i]
        if c.m_rate_gate:                                # what waits is released only where the model still wants it
            bank = torch.where(bank * (grad.float().movedim(ax, -1) @ U) < 0, bank, torch.zeros_like(bank))
        want = moved + bank
        bv = 0.9
        v_new = bv * v + (1 - bv) * want
        size = v_new.norm()
        warm = self.mrl_n < c.m_rate_warm                # first steps: only learn the usual size
        scale = torch.ones_like(size) if warm else (c.m_rate_kappa * base / size.clamp(min=1e-30)).clamp(max=1.0)
        v_cut = v_new * scale
        out = torch.where(scale < 1.0, (v_cut - bv * v) / (1 - bv), want)
        self.mrl_bank[i] = want - out
        self.mrl_v[i] = v_cut
        sz = v_cut.norm()
        if warm:
            base.copy_(sz if self.mrl_n == 0 else 0.95 * base + 0.05 * sz)
        else:
            base.copy_(0.998 * base + 0.002 * torch.minimum(sz, base))          # no ratchet: pressure does not lift the limit
        self.mrl_cut += (scale < 1.0).float()
        t.copy_((new + (out - moved)[..., None] * U).movedim(-1, ax).to(t.dtype))
        if self.w[i] is not None:
            p.data.copy_(t)

    def _step_body(self, i, p, grad):
        self._sync_lr()
        kind, wd, vocab = self.spec(p)
        want_rel = self.n_step % self.rel_every == 0
        lr_t = self._lr_v if vocab else self._lr_t
        if self.cfg.surge_thr > 0:                       # surprise brake (device scalars only)
            bad = (-self.s).clamp(min=self.cfg.surge_thr)
            lr_t = lr_t * (self.cfg.surge_thr / bad) ** 2
        raw = grad if (self.cfg.gnorm and self.cfg.gnorm_rawrel) else None
        if self.cfg.gnorm:                               # a step with a large gradient does not drown the small ones in the momentum
            g32 = grad.float()
            grad = (g32 * torch.rsqrt(g32.pow(2).mean() + 1e-30)).to(grad.dtype if grad.dtype == torch.float32 else torch.float32)
        if self._mul[i] != 1.0:
            lr_t = lr_t * self._mul[i]
        if self.dv is not None and (self.cfg.gearbox or self.cfg.err_step):
            lr_t = self._pace(i, grad, lr_t)
        elif self.dv is not None and not vocab:
            grad, lr_t = self._damp(i, grad, lr_t)
        if self.snr_v is not None and not vocab and self.m[i].shape == grad.shape and self._snr_on[i]:
            lr_t = self._snr(i, grad, lr_t)
        wd_v = self.param_groups[0]["weight_decay"] / self.scale if wd else 0.0
        if not wd and self.cfg.wd_norm > 0 and self._norm_w[i]:
            wd_v = self.cfg.wd_norm / self.scale             # norm weights otherwise take constant-length steps with no pull back
        if self.cfg.norm_anchor and self._anchor[i]:
            self._anchor_norm(i, p)
        rows = self.rows.get(id(p)) if vocab else None
        if rows is not None:
            self._update_rows(i, p, grad, rows, lr_t)
            if want_rel:
                self.rel[i] = 0.0
            return
        if (_ext.use_cuda(p) and _kind_code(kind) >= 0 and p.is_contiguous() and grad.is_contiguous()
                and getattr(p, "_row_shard", None) is None and not self._safe[i]
                and not (self.hs_lag and kind in ("hs", "hs3") and not self._lag_on_gpu(p, kind))):
            self._update_cuda(i, p, grad, kind, wd_v, lr_t, want_rel)
        else:
            self._update_ref(i, p, grad, kind, wd_v, lr_t, want_rel)
        if raw is not None and want_rel:
            # the normalised gradient has the same length for every tensor, so |g|/|w| would only say whose |w| shrinks:
            # who is to blame is measured on the raw gradient
            t = self.w[i] if self.w[i] is not None else p
            self.rel[i] = raw.float().norm() / (t.float().norm() + 1e-8)

    def _anchor_norm(self, i, p):
        """w <- w - lr wd (w - 1) on a 1-D norm weight (and its exact copy): what weight decay is for matrices, with 1
        as the resting point (the JAX Instinct's `norm_anchor`, instinct.py:393-401)."""
        pull = self._lr_t / self.scale * self.param_groups[0]["weight_decay"]
        t = self.w[i] if self.w[i] is not None else p.data
        t.sub_((t - 1.0) * pull.to(t.dtype))
        if self.w[i] is not None:
            p.data.copy_(t)

    def _damp(self, i, grad, lr_t):
        """Per-tensor gradient-surge damping (the reference's JAX Instinct, instinct.py:132-150): the optimizer
        normalises the step by the momentum and does not see the gradient's scale, so when |g| of a tensor surges
        the step stays full.  While |g| <= damp x usual nothing changes; above it the gradient enters the momentum
        clipped to damp x usual and the step shrinks by (damp x usual / |g|)^damp_p.  Device-side, no host sync."""
        c = self.cfg
        gg = grad.float().pow(2).sum()
        dv = (self.oh @ self.dv)[i]                                        # usual |g|^2 on the current card
        started = dv > 0
        ratio = torch.where(started & (gg > 0), (gg / dv.clamp(min=1e-38)).sqrt(), torch.ones_like(gg))
        f = torch.where(ratio > c.damp, c.damp / ratio, torch.ones_like(ratio))
        into = torch.minimum(gg, (c.damp_cap ** 2) * dv)
        new = torch.where(started, c.damp_beta * dv + (1 - c.damp_beta) * into, gg)
        self.dv[:, i] += self.oh * (torch.where(gg > 0, new, dv) - dv)
        self.df[i] = f
        return (grad * f.to(grad.dtype), lr_t * f ** c.damp_p)

    def _pace(self, i, grad, lr_t):
        """Two step-length rules of the reference's JAX Instinct that read |g| against its usual value on the current
        card and leave the gradient itself alone (instinct.py:150-172, 753-772, 918-937).
        err_step: step x clip(usual |g| / |g|, 0, err_cap) - a tensor whose sensitivity surges 28x takes a 28x shorter
        step.  gearbox: the multiplier follows a gear (0.25, 0.5, 1, gb_top), shifted one gear per step - down on a
        surge above gb_down x usual, or when driving above 1.0 while the step's loss is worse than expected; up when
        calm (below gb_up x usual) and the speed has caught up with the current gear - and the speed itself changes by
        at most gb_acc per step.  Device-side, no host sync."""
        c = self.cfg
        gg = grad.float().pow(2).sum()
        dv = (self.oh @ self.dv)[i]
        live, started = gg > 0, dv > 0
        into = torch.minimum(gg, (c.damp_cap ** 2) * dv)
        usual = torch.where(started, c.damp_beta * dv + (1 - c.damp_beta) * into, gg)
        self.dv[:, i] += self.oh * (torch.where(live, usual, dv) - dv)
        if c.gearbox:
            gears = torch.tensor([0.25, 0.5, 1.0, c.gb_top], device=gg.device)
            ratio = torch.where(started & live, (gg / dv.clamp(min=1e-38)).sqrt(), torch.ones_like(gg))
            v, gi = self.speed[i], self.gear[i]
            fined = (v > 1.0) & (self.s < 0)
            down = (ratio > c.gb_down) | fined
            up = (ratio < c.gb_up) & ~fined & (v >= gears[gi] - 1e-3)
            shift = torch.where(down, -1, torch.where(up, 1, 0))
            gi_new = torch.where(live, (gi + shift).clamp(0, 3), gi)
            v_new = torch.where(live, v + (gears[gi_new] - v).clamp(-c.gb_acc, c.gb_acc), v)
            self.gear[i], self.speed[i] = gi_new, v_new
            f = v_new
        else:
            f = torch.where(started & live, (dv / gg.clamp(min=1e-38)).sqrt().clamp(0, c.err_cap), torch.ones_like(gg))
        self.df[i] = f
        return lr_t * f

    def _snr(self, i, grad, lr_t):
        """Confidence of a tensor's direction (the reference's JAX Instinct, instinct.py:76-84, 100-104, 953-975):
        c = |beta m + (1-beta) g| / sqrt(EMA |g|^2).  Gradients that agree from step to step give c near 1, noise
        gives c near sqrt((1-beta)/(1+beta)); the step is scaled by clip(c / snr_ref, snr_floor, 1).  The dead-zone
        form keeps an EMA of c^2 instead and brakes only what is indistinguishable from a random walk:
        k = (1-beta)/(1+beta), r = max(c2 - k, 0) / (1 - c2), factor = clip(sqrt(r horizon / k), floor, 1).
        A tensor without gradient keeps its state.  Three scalar reductions, device-side, no host sync."""
        c = self.cfg
        g32, m32 = grad.float(), self.m[i].float()
        gg, mg, m2 = (g32 * g32).sum(), (m32 * g32).sum(), (m32 * m32).sum()
        b = self.beta
        mn2 = (b * b * m2 + 2 * b * (1 - b) * mg + (1 - b) * (1 - b) * gg).clamp(min=0.0)
        v_old = self.snr_v[i]
        if c.snr_dz:
            c2 = mn2 / (gg + 1e-30)
            ok = (v_old > 0) & (v_old <= 1.0)
            v_new = torch.where(ok, c.snr_beta * v_old + (1 - c.snr_beta) * c2, c2)
            k = (1 - b) / (1 + b)
            r = (v_new - k).clamp(min=0.0) / (1 - v_new).clamp(min=1e-6)
            f = (r * c.snr_horizon / k).sqrt().clamp(c.snr_floor, 1.0)
        else:
            v_new = torch.where(v_old > 0, c.snr_beta * v_old + (1 - c.snr_beta) * gg, gg)
            f = (mn2.sqrt() / (v_new.sqrt() + 1e-30) / c.snr_ref).clamp(c.snr_floor, 1.0)
        live = gg > 0
        self.snr_v[i] = torch.where(live, v_new, v_old)
        f = torch.where(live, f, torch.ones_like(f))
        self.snr_f[i] = f
        return lr_t * f

    def _frozen_mask(self, p):
        fr = getattr(p, "_frozen_rows", None)
        return fr

    def _update_ref(self, i, p, grad, kind, wd, lr_t, want_rel):
        m, w = self.m[i], self.w[i]
        grad = grad.float()
        m_old = m.float().clone() if self._safe[i] else None
        mf = m.float() * self.beta + grad * (1 - self.beta)
        if self.sr and m.dtype == torch.bfloat16:
            self._seed_t.add_(1)
            r_m, r_w = ref.sr_counter(mf.numel(), int(self._seed_t) * 1000003 + i, mf.device)
            m.copy_(ref.sr_bf16(mf.reshape(-1), r_m).view_as(m))
        else:
            m.copy_(mf)
            r_w = None
        cs = None
        if self.hs_lag and kind in ("hs", "hs3"):
            if self.cs[i] is None:
                shp = (1, p.shape[1]) if kind == "hs" else (p.shape[0], p.shape[1], 1)
                self.cs[i] = torch.zeros(shp, device=p.device, dtype=torch.float32)
            cs = self.cs[i]
        shard = getattr(p, "_row_shard", None)
        if self._safe[i]:
            # (1) the part of the old momentum that points against the fresh gradient is projected out (per input
            # column of a matrix - the first axis of the JAX port's (in, out) layout - or for a whole 1-D tensor),
            # (2) coordinates of the step that still go against the gradient are masked ("cautious"), (3) 1-D norm
            # weights step relative to |w| (at most 2x), so near-zero sink channels are not kicked out
            # (memarch_jax/memarch_jax/instinct.py:1033-1043)
            dims = tuple(range(grad.dim() - 1)) if grad.dim() >= 2 else None
            tot = (lambda t: t.sum(dims, keepdim=True)) if dims is not None else (lambda t: t.sum())
            mg, gg = tot(m_old * grad), tot(grad * grad) + 1e-30
            mstep = (m_old - mg.clamp(max=0.0) / gg * grad) * self.beta + grad * (1 - self.beta)
            mstep = torch.where(mstep * grad >= 0, mstep, torch.zeros_like(mstep))
            upd, new_cs = ref.instinct_direction(mstep, grad, kind, cs)
            if p.dim() == 1:
                w0 = (p if w is None else w).float()
                lr_t = lr_t * (w0.abs() / (w0.pow(2).mean().sqrt() + 1e-8)).clamp(max=2.0)
        elif shard is not None and kind == "hs":
            upd, new_cs = self._direction_row_sharded(mf, shard), None
        else:
            upd, new_cs = ref.instinct_direction(mf, grad, kind, cs)
        if new_cs is not None:
            self.cs[i].copy_(new_cs)
        t = p if w is None else w
        if want_rel:
            self.rel[i] = grad.norm() / (t.norm().float() + 1e-8)
        eff = 1 + (self.g[i] - 1) * self.stake
        fr = self._frozen_mask(p)
        keep = t.detach().clone() if fr is not None else None
        if self.sr and w is None and t.dtype == torch.bfloat16:
            new = t.float()
            if wd:
                new = new * (1 - lr_t * wd)
            new = new - upd * (lr_t * eff)
            if r_w is None:
                self._seed_t.add_(1)
                _, r_w = ref.sr_counter(new.numel(), int(self._seed_t) * 1000003 + i, new.device)
            t.copy_(ref.sr_bf16(new.reshape(-1), r_w).view_as(t))
        else:
            if wd:
                t.mul_(1 - lr_t * wd)
            t.sub_((upd * (lr_t * eff)).to(t.dtype))
        if keep is not None:
            t.copy_(torch.where(fr.view(-1, *[1] * (t.dim() - 1)), keep, t))
        if w is not None:
            p.copy_(w)

    @staticmethod
    def _direction_row_sharded(mf, shard):
        """Homeostasis of a weight cut by rows between ranks (the reference's kind `hsS<W>,<rows>`, exp_opt.py:271-280):
        rows are local, the per-column norm is a sum over all ranks - one small all-reduce of a (1, C) vector."""
        import torch.distributed as dist
        _, total_rows, group = shard
        upd = mf / (mf.pow(2).mean(1, keepdim=True).sqrt() + 1e-8)
        col = upd.pow(2).sum(0, keepdim=True)
        if dist.is_initialized():
            dist.all_reduce(col, group=group)
        upd = upd / ((col / total_rows).sqrt() + 1e-8)
        return upd / (upd.pow(2).mean(1, keepdim=True).sqrt() + 1e-8)

    def _arena(self, p, kind):
        """One fp32 scratch arena per (device, stream) for the row / column statistics, sized for the largest weight
        seen there.  Per stream, because the data-parallel engine steps replicated weights on a side stream while the
        expert weights are stepped on the main one: two steps in flight must not share their statistics."""
        if kind in ("hs", "vocab"):
            E, R, Cn = 1, p.shape[0], p.shape[1]
        elif kind in ("hs3", "row3"):
            E, R, Cn = p.shape
        elif kind == "row":
            E, R, Cn = 1, p.shape[0], p.numel() // p.shape[0]
        else:
            E, R, Cn = 1, 1, p.numel()
        need = 3 * ((E * R + 3) // 4 * 4) + 2 * ((E * Cn + 3) // 4 * 4) + 4
        key = ("arena", p.device, torch.cuda.current_stream(p.device).cuda_stream)
        cur = self._scratch.get(key)
        if cur is None or cur.numel() < need:
            cur = self._scratch[key] = torch.empty(max(need, 1 << 16), device=p.device, dtype=torch.float32)
        return cur

    def _lag_on_gpu(self, p, kind):
        """The lagged form runs on the kernels for hs3 always and for hs when three rows fit in shared memory."""
        return kind == "hs3" or (kind == "hs" and 3 * 4 * p.shape[1] <= 200 * 1024)

    def _update_cuda(self, i, p, grad, kind, wd, lr_t, want_rel):
        C = _ext.C()
        m, w = self.m[i], self.w[i]
        lag = self.hs_lag and kind in ("hs", "hs3")
        if lag and self.cs[i] is None:
            shp = (1, p.shape[1]) if kind == "hs" else (p.shape[0], p.shape[1], 1)
            self.cs[i] = torch.zeros(shp, device=p.device, dtype=torch.float32)
        if lag and self.cs_ok[i] is None:
            self.cs_ok[i] = torch.zeros((), device=p.device, dtype=torch.int32)    # 0: look for non-positive entries
        if self.sr:
            self._seed_t.add_(1)
        fr = self._frozen_mask(p)
        n = C.instinct_step(p, grad, m, w, self.cs[i] if lag else None, self.g, int(i), self.stake, lr_t,
                            self.rel if want_rel else None, float(self.beta), float(wd), _kind_code(kind),
                            bool(self.sr), self._seed_t, fr, self._arena(p, kind), self.cs_ok[i] if lag else None,
                            getattr(p, "_bf16_shadow", None))
        _ext.count(int(n) + 1)

    def can_shard(self, p):
        """True when `update_sharded` can step this weight: a 2-D weight of kind "hs" - bf16 with its exact fp32 copy
        here, or fp32 (the caller provides the bf16 shadow the GEMMs read) - none of the per-tensor brakes (they need
        whole-tensor sums) and no lag / offload / stochastic rounding."""
        c = self.cfg
        i = self.idx[id(p)]
        layout = (p.dtype == torch.bfloat16 and self.w[i] is not None) or (p.dtype == torch.float32 and self.w[i] is None)
        return (p.dim() == 2 and layout and self.spec(p)[0] == "hs" and not self.hs_lag and not self.offload
                and not self.sr and self.dv is None and self.snr_v is None and c.surge_thr <= 0)

    @torch.no_grad()
    def update_sharded(self, p, g_rows, r0, r1, scratch, shadow_rows, exchange):
        """Step rows [r0, r1) of a weight whose rows are split between the ranks (the reference's kind `hsS`,
        exp_opt.py:271-280: rows are local, a column's norm is a sum over all ranks).  `g_rows` is the rank-mean
        gradient of these rows, `scratch` an fp32 arena every rank can reach (the statistics are summed in place),
        `shadow_rows` the rows of the bf16 copy the GEMMs read (None for a bf16 weight: it is its own), `exchange(offset, count)` sums `scratch[offset:
        offset + count]` over the ranks (device-side, on the current stream).  Momentum and the fp32 weight are touched
        in these rows only: every other row of `p` and of the momentum is another rank's to keep."""
        region = self.shard_stats(p, g_rows, r0, r1, scratch, shadow_rows)
        exchange(*region)                                       # column sums (and the |g|, |w| sums behind them)
        self.shard_apply(p, g_rows, r0, r1, scratch, shadow_rows)

    def _shard_call(self, p, g_rows, r0, r1, scratch, shadow_rows, phase):
        i = self.idx[id(p)]
        self._sync_lr()
        _, wd, _ = self.spec(p)
        want_rel = self.n_step % self.rel_every == 0
        wd_v = self.param_groups[0]["weight_decay"] / self.scale if wd else 0.0
        pr, mr = p[r0:r1], self.m[i][r0:r1]
        wr = self.w[i][r0:r1] if self.w[i] is not None else None
        n = _ext.C().instinct_step(pr, g_rows, mr, wr, None, self.g, int(i), self.stake, self._lr_t,
                                   self.rel if want_rel else None, float(self.beta), float(wd_v), _kind_code("hs"), False,
                                   self._seed_t, None, scratch, None, shadow_rows, phase, int(p.shape[0]))
        _ext.count(int(n))

    def shard_stats(self, p, g_rows, r0, r1, scratch, shadow_rows=None):
        """First half of `update_sharded`: the statistics of rows [r0, r1) into `scratch`.  Returns (offset, count) of
        the part of `scratch` that must be summed over the ranks before `shard_apply`."""
        self._shard_call(p, g_rows, r0, r1, scratch, shadow_rows, 1)
        pad4 = lambda v: (v + 3) // 4 * 4
        return 3 * pad4(r1 - r0), 2 * pad4(p.shape[1]) + 4

    def shard_apply(self, p, g_rows, r0, r1, scratch, shadow_rows=None):
        """Second half: the update of rows [r0, r1) from the summed statistics."""
        self._shard_call(p, g_rows, r0, r1, scratch, shadow_rows, 2)

    def _update_rows(self, i, p, grad, rows, lr_t):
        """Word / phrase tables: only rows used in this step move (exp_opt.py:306-318)."""
        m, w = self.m[i], self.w[i]
        g = grad[rows].float()
        mr = m[rows].float() * self.beta + g * (1 - self.beta)
        m[rows] = mr.to(m.dtype)
        upd = mr / (mr.pow(2).mean(1, keepdim=True).sqrt() + 1e-8)
        t = p if w is None else w
        t[rows] = t[rows] - (upd * (lr_t * (1 + (self.g[i] - 1) * self.stake))).to(t.dtype)
        if w is not None:
            p[rows] = w[rows].to(p.dtype)

    @torch.no_grad()
    def update_all(self):
        """Step every weight that holds a gradient (after backward; used with sharded gradients)."""
        for p in self.plist:
            if p.grad is not None:
                self.update(p)
                p.grad = None

    @torch.no_grad()
    def swap(self, old, new, slot_map):
        """Experts moved between banks: the new parameter takes the old one's slot; momentum (and the exact fp32
        copy) of experts that keep learning is carried by position (exp_opt.py:711-725)."""
        i = self.idx.pop(id(old))
        self.plist[i] = new
        self.idx[id(new)] = i
        m = torch.zeros_like(new, dtype=self.m_dtype)
        w = new.detach().float().clone() if (new.dtype == torch.bfloat16 and not self.cfg.no_master) else None
        for j, s in enumerate(slot_map):
            if s is not None:
                m[j] = self.m[i][s]
                if w is not None and self.w[i] is not None:
                    w[j] = self.w[i][s]
        self.m[i], self.w[i] = (self._to_host(m) if self.offload else m), w
        self.cs[i] = None
        self.cs_ok[i] = None

    @property
    def last(self):
        return dict(card=self.k, s=self.s, stake=self.stake)

    # ------------------------------------------------------------------------------------------ checkpoint blob
    _SKIP = {"plist", "idx", "param_groups", "rows", "cfg", "grad_sync", "_scratch", "lr_mul_dev", "offload", "cs_ok"}

    def state_dict(self):
        out = {}
        for k, v in vars(self).items():
            if k in self._SKIP:
                continue
            if torch.is_tensor(v):
                out[k] = v.detach().cpu()
            elif isinstance(v, list) and all(torch.is_tensor(t) or t is None for t in v):
                own = self.offload and k == "m"             # already on the host: the blob must not alias the live state
                out[k] = [None if t is None else (t.detach().clone() if own else t.detach().cpu()) for t in v]
            elif isinstance(v, (int, float, bool, str)) or v is None:
                out[k] = v
        out["_lr"] = [g["lr"] for g in self.param_groups]   # a list, one per group (the reference's layout, fastloop.py:668-677)
        return out

    def load_state_dict(self, sd):
        dev = self.plist[0].device
        for k, v in sd.items():
            if k == "_lr":                                     # a list per group (reference layout) or a scalar (older files)
                lrs = list(v) if isinstance(v, (list, tuple)) else [v] * len(self.param_groups)
                for g, lr in zip(self.param_groups, lrs):
                    g["lr"] = float(lr)
            elif torch.is_tensor(v):
                cur = getattr(self, k, None)
                if torch.is_tensor(cur) and cur.shape == v.shape:
                    cur.copy_(v.to(cur.device))
                else:
                    setattr(self, k, v.to(dev))
            elif isinstance(v, list):
                cur = getattr(self, k, None)
                new = []
                for j, t in enumerate(v):
                    if t is None:
                        new.append(None)
                    elif cur is not None and j < len(cur) and torch.is_tensor(cur[j]) and cur[j].shape == t.shape:
                        cur[j].copy_(t.to(cur[j].device))
                        new.append(cur[j])
                    else:
                        new.append(t.to(self.plist[j].device if j < len(self.plist) else dev))
                setattr(self, k, new)
            elif k in ("n_step", "rel_every"):
                setattr(self, k, v)
        self._lr_last = None


class SurpriseAdamW(torch.optim.AdamW):
    """AdamW whose step is rescaled by the loss surprise (surprise_opt.py:1-47): the update of a step whose loss
    beats its running expectation is amplified, a worse-than-expected step is damped."""

    def __init__(self, params, lr=1e-3, ema=0.98, strength=1.0, lo=0.5, hi=2.0, **kw):
        super().__init__(params, lr=lr, **kw)
        self.ema, self.strength, self.lo, self.hi = ema, strength, lo, hi
        self.expect = None

    @torch.no_grad()
    def step(self, loss=None):
        if loss is None:
            return super().step()
        loss = float(loss)
        e = loss if self.expect is None else self.expect
        s = (e - loss) / max(e, 1e-6)
        self.expect = self.ema * e + (1 - self.ema) * loss
        mul = min(self.hi, max(self.lo, 1 + self.strength * s))
        before = [[p.detach().clone() for p in g["params"]] for g in self.param_groups]
        super().step()
        for g, bs in zip(self.param_groups, before):
            for p, b in zip(g["params"], bs):
                p.copy_(b + (p - b) * mul)
