"""Heavy MoE layer that runs on anchor tokens only: shared-budget routing, fixed-capacity slots, SwiGLU/relu²
experts, wave training and a real frozen bank, expert parallelism.

One class covers the reference's `BudgetMoE` (full2.py:384-643) and `BankMoE` (full2.py:870-1242):
  * router softmax -> top-k_max, per-token expert budget from surprise (budget mode) or a fixed k;
  * capacity C = int(cf·fill·N·k/E)+1 places per expert filled in arrival order, overflow dropped and reported;
  * Switch-style balance loss in `.aux`, dropped share in `.dropped`;
  * waves: `learned` experts stop training ("err" = error below a share of its peak, "still" = weights stopped
    moving); bank mode moves learned experts into a frozen bf16 (or int8/int4) bank without grads or optimizer
    state and thaws those that start erring again (`rebank`);
  * expert parallelism: `ep_shard(rank, W)` keeps E/W experts per rank; tokens travel by all-to-all through the
    attached `ep_engine` (NCCL baseline or the fused peer-memory kernels in `memarch_b200.parallel.ep`).
State-dict names match the reference: `norm.weight, router.weight, up, down`, buffers `s_mean, err, err_peak,
err_freeze, move_peak, last_move, hint_avg, learned, up_snap, L_idx, F_idx, up_f, down_f, up_fs, down_fs`.
"""
from __future__ import annotations

import os

import torch
import torch.nn as nn

from .. import ops
from .blocks import _cdt


class _ErrProbe(torch.autograd.Function):
    """Identity forward; backward folds the mean output-gradient norm of every expert into an EMA buffer
    (the expert's "error": how much the loss wants its output changed).  (full2.py:331-344)"""

    @staticmethod
    def forward(ctx, y, buf):
        ctx.buf = buf
        return y.view_as(y)

    @staticmethod
    def backward(ctx, g):
        with torch.no_grad():
            # fp32 accumulation straight from the bf16 gradient: no fp32 copy of the (E, C, d) tensor
            ctx.buf.mul_(0.9).add_(0.1 * torch.linalg.vector_norm(g, dim=-1, dtype=torch.float32).mean(1))
        return g, None


class _ErrProbeWords(torch.autograd.Function):
    """The same probe read off the gradient of the combined word outputs (N, d), for the exchange that sums a word's
    experts on the owning rank so that no per-place output exists here: the gradient of place (e, c) is its combine
    weight times its word's gradient, hence its norm |w| * |g_word|; empty places (table == N) count as zero.
    (full2.py:347-364)"""

    @staticmethod
    def forward(ctx, out, buf, table, wtab, E):
        ctx.buf, ctx.E = buf, E
        ctx.save_for_backward(table, wtab)
        return out.view_as(out)

    @staticmethod
    def backward(ctx, g):
        table, wtab = ctx.saved_tensors
        with torch.no_grad():
            N = g.shape[0]
            word = torch.linalg.vector_norm(g, dim=-1, dtype=torch.float32)
            place = torch.where(table < N, word[table.clamp(max=N - 1)], word.new_zeros(())) * wtab.float().abs()
            ctx.buf.mul_(0.9).add_(0.1 * place.view(ctx.E, -1).mean(1))
        return g, None, None, None, None


class _FrozenBankI8(torch.autograd.Function):
    """Forward of the frozen int8 bank on the int8 tensor cores: rows of the input and of the hidden activation are
    quantised (absmax / 127 per row), both products run as `tcgen05.mma.kind::i8` GEMMs against the stored int8 weights
    with the per-output-column scales applied in the epilogue (the reference's int8 bank: full2.py:919-958 with the
    matmul of int8mm.py:35-88).  Only the input gets a gradient (the bank is frozen); it is computed in bf16 from the
    dequantised weights, like the bf16 bank."""

    @staticmethod
    def forward(ctx, xe, up_t, up_s, down_t, down_s, moe):
        from ..ops import _ext, int8
        C = _ext.C()
        a = int8.quant_mm_stored(xe, up_t, up_s)                               # (F, C, width_in) bf16 pre-activations
        h = C.relu2_fwd(a) if moe.act == "relu2" else C.swiglu_fwd(a)
        y = int8.quant_mm_stored(h, down_t, down_s)
        _ext.count(1)
        ctx.save_for_backward(a)
        ctx.moe = moe
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops import _ext
        a, = ctx.saved_tensors
        moe, C = ctx.moe, _ext.C()
        up, down = moe._bank_weights("up"), moe._bank_weights("down")          # (F, d, width_in), (F, width_out, d) bf16
        F_ = up.shape[0]
        dh = ops.gemm(dy.contiguous(), down, groups=F_)                        # dy (F,C,d) · down (F,width_out,d)ᵀ
        da = C.relu2_bwd(dh, a) if moe.act == "relu2" else C.swiglu_bwd(dh, a)
        dx = ops.gemm(da, up, groups=F_)                                       # da (F,C,width_in) · up (F,d,width_in)ᵀ
        _ext.count(1)
        return dx, None, None, None, None, None


class AnchorMoE(nn.Module):
    def __init__(self, d, E=8, k_avg=2, k_max=4, budget=True, wave="", wave_every=50, students=5, hint_w=1.0,
                 frozen=0, bank=False, act="swiglu", w_dtype=torch.float32, bank_q="", wave_warm=500,
                 err_thr=0.3, cap_align=0, local_experts=None, dropless=False):
        super().__init__()
        self.dropless = dropless
        self.E, self.k_avg, self.k_max, self.budget = E, k_avg, k_max, budget
        self.bank, self.act, self.bank_q, self.cap_align = bank, act, bank_q, cap_align
        self.fill = 1.0
        self.norm = nn.RMSNorm(d)
        self.router = nn.Linear(d, E, bias=False)
        if bank:
            hid = 2 * d * 2 // k_avg
            self.width_in = 3 * hid // 2 if act == "relu2" else 2 * hid        # columns of `up`
            self.width_out = 3 * hid // 2 if act == "relu2" else hid           # rows of `down`
            wave, hint_w, budget = "still", 0.0, False
            self.budget = False
        else:
            hid = 2 * d
            self.width_in, self.width_out = 2 * hid, hid
            act = self.act = "swiglu"
        Ea = (E - frozen) if local_experts is None else local_experts
        self.n_frozen = frozen
        self.up = nn.Parameter((torch.randn(Ea, d, self.width_in) * d ** -0.5).to(w_dtype))
        self.down = nn.Parameter((torch.randn(Ea, self.width_out, d) * self.width_out ** -0.5 * 0.5).to(w_dtype))
        self.w_dtype = w_dtype
        self.aux = torch.zeros(())
        self.dropped = torch.zeros(())
        self.layer_stats = False
        self.fill_now = self.active_now = torch.zeros(())
        self.register_buffer("s_mean", torch.tensor(5.0))
        self.wave, self.wave_every, self.students, self.hint_w = wave, wave_every, students, hint_w
        self.warm, self.err_thr = wave_warm, err_thr
        self.hint_now = False
        self.hint = torch.zeros(())
        if wave:
            for nm in ("err", "err_peak", "err_freeze", "move_peak", "last_move", "hint_avg"):
                self.register_buffer(nm, torch.zeros(E))
            self.register_buffer("learned", torch.zeros(E, dtype=torch.bool))
            if wave == "still":
                self.register_buffer("up_snap", self.up.detach().clone())
        if frozen and not bank:
            self.register_buffer("up_f", (torch.randn(frozen, d, self.width_in) * d ** -0.5).bfloat16())
            self.register_buffer("down_f", (torch.randn(frozen, self.width_out, d) * self.width_out ** -0.5 * 0.5)
                                 .bfloat16())
        if bank:
            self.L, self.Fz = list(range(E)), []
            self.has_L, self.has_F = True, False
            self.register_buffer("L_idx", torch.arange(E))
            self.register_buffer("F_idx", torch.zeros(0, dtype=torch.long))
            self.register_buffer("up_f", torch.zeros(0, d, self.width_in, dtype=torch.bfloat16))
            self.register_buffer("down_f", torch.zeros(0, self.width_out, d, dtype=torch.bfloat16))
            self.register_buffer("up_fs", torch.zeros(0, 1, self.width_in, dtype=torch.bfloat16))
            self.register_buffer("down_fs", torch.zeros(0, 1, d, dtype=torch.bfloat16))
        self.ep_W, self.ep_rank, self.ep_engine = 1, 0, None

    # ------------------------------------------------------------------------------------------ routing
    def capacity(self, N):
        if self.dropless:
            # a token picks an expert at most once, so N places per expert hold everything; the places past an
            # expert's fill count are padding that the grouped GEMMs neither load nor multiply
            return -(-N // 8) * 8
        cf = 1.6 if self.budget else 1.25
        C = int(cf * self.fill * N * self.k_avg / self.E) + 1
        if self.cap_align:
            C = max(self.cap_align, round(C / self.cap_align) * self.cap_align)
        return C

    def _route(self, x, surprise):
        N, d = x.shape[0] * x.shape[1], x.shape[-1]
        xf = ops.rmsnorm(x, self.norm.weight, self.norm.eps, out_dtype=_cdt(x)).reshape(N, d)
        real = (surprise.reshape(N) >= 0) if surprise is not None else torch.ones(N, dtype=torch.bool, device=x.device)
        if self.budget and surprise is not None:
            s = surprise.reshape(N).float().clamp(min=0)
            k_tok = (self.k_avg * s / self.s_mean.clamp(min=1e-6)).round().clamp(1, self.k_max).long()
            if self.training:
                with torch.no_grad():
                    self.s_mean.mul_(0.99).add_(0.01 * (s * real).sum() / real.sum().clamp(min=1))
        else:
            k_tok = torch.full((N,), self.k_avg, device=x.device, dtype=torch.long)
        k_tok = k_tok * real
        C = self.capacity(N)
        w, table, wtab, flat_idx, aux, dropped, _, counts = ops.route_and_slot(
            xf, self.router.weight.float() if not x.is_cuda else self.router.weight, real, k_tok, self.k_max, self.E, C,
            want_counts=True)
        self.aux, self.dropped = aux, dropped
        self._counts = counts                # filled places per expert (GPU): the expert GEMMs skip the padding
        if self.layer_stats:                 # share of the capacity in use, experts with at least one place (collapse watch)
            with torch.no_grad():
                used = (flat_idx < self.E * C)
                per_expert = torch.zeros(self.E + 1, device=x.device).index_add_(
                    0, torch.where(used, flat_idx // C, torch.full_like(flat_idx, self.E)).reshape(-1),
                    torch.ones(flat_idx.numel(), device=x.device))[:-1]
                self.fill_now, self.active_now = used.float().sum() / float(self.E * C), (per_expert > 0).float().sum()
        return xf, table, wtab, flat_idx, C

    def forward(self, x, surprise=None):
        xf, table, wtab, flat_idx, C = self._route(x, surprise)
        N, d = xf.shape
        eng = self.ep_engine if self.ep_W > 1 else None
        if eng is not None and getattr(eng, "dedup", False) and not (self.bank and self.has_F) and not (self.wave and not self.bank):
            out = eng.forward_dedup(self, xf, table, wtab, C, eng.dedup_cap)
            if self.wave and self.training:
                out = _ErrProbeWords.apply(out, self.err, table, wtab, self.E)
            return ops.resid_add(x, out.view_as(x))
        xe = ops.slot_gather(xf, table, flat_idx).view(self.E, C, d)
        ye = self._experts(xe, wtab, C)
        out = ops.combine(ye.reshape(self.E * C, d), wtab.to(ye.dtype), flat_idx, table, N)
        return ops.resid_add(x, out.view_as(x))

    # ------------------------------------------------------------------------------------------ experts
    def _ffn(self, xe, up, down, train_w=True, counts=None):
        return ops.expert_ffn(xe, up.to(xe.dtype) if up.dtype != xe.dtype else up,
                              down.to(xe.dtype) if down.dtype != xe.dtype else down, self.act, train_w, counts)

    # ------------------------------------------------------------------------------------------ frozen bank storage
    # Stored form of a frozen table (F, in, out): bf16 as is; int8 with one scale per output column; int4 with one
    # scale per output column and block of 128 inputs, two values per byte (even input in the low nibble).
    # (full2.py:919-958)
    def _bank_weights(self, which):
        """The frozen `up` / `down` table expanded to bf16."""
        stored, scale = getattr(self, which + "_f"), getattr(self, which + "_fs")
        if not self.bank_q:
            return stored
        if self.bank_q == "int8":
            return stored.to(torch.bfloat16) * scale
        n_f, half, n_out = stored.shape
        low, high = (stored << 4) >> 4, stored >> 4                       # sign-extending nibble extraction
        vals = torch.stack([low, high], 2).reshape(n_f, 2 * half // 128, 128, n_out)
        return (vals.to(torch.bfloat16) * scale[:, :, None]).reshape(n_f, 2 * half, n_out)

    def _quantise(self, w):
        """float (F, in, out) -> (stored table, scales) in the layout above."""
        if not self.bank_q:
            return w.bfloat16().contiguous(), w.new_zeros(w.shape[0], 1, w.shape[2]).bfloat16()
        if self.bank_q == "int8":
            scale = (w.abs().amax(1, keepdim=True) / 127).clamp(min=1e-8)
            return (w / scale).round().clamp(-127, 127).to(torch.int8).contiguous(), scale.bfloat16()
        n_f, n_in, n_out = w.shape
        blocks = w.view(n_f, n_in // 128, 128, n_out)
        scale = (blocks.abs().amax(2, keepdim=True) / 7).clamp(min=1e-8)
        vals = (blocks / scale).round().clamp(-7, 7).to(torch.int8).view(n_f, n_in, n_out)
        packed = ((vals[:, 0::2] & 0x0F) | (vals[:, 1::2] << 4)).to(torch.int8)
        return packed.contiguous(), scale[:, :, 0].bfloat16().contiguous()

    def _bank_i8(self):
        """The int8 bank in the layout the int8 GEMM reads (contraction contiguous): (F, out, in) copies of the stored
        (F, in, out) tables and their fp32 column scales, rebuilt when the bank's tensors change."""
        key = (self.up_f.data_ptr(), self.down_f.data_ptr(), tuple(self.up_f.shape))
        if getattr(self, "_i8_key", None) != key:
            self._i8_cache = (self.up_f.transpose(1, 2).contiguous(), self.up_fs.float().reshape(self.up_f.shape[0], -1).contiguous(),
                              self.down_f.transpose(1, 2).contiguous(), self.down_fs.float().reshape(self.down_f.shape[0], -1).contiguous())
            self._i8_key = key
        return self._i8_cache

    def _ffn_frozen(self, xe, counts=None):
        from ..ops import _ext, int8
        if (self.bank_q == "int8" and _ext.use_cuda(xe) and xe.dtype == torch.bfloat16 and self.up_f.dtype == torch.int8
                and int8.i8_ok(xe.shape[1], self.up_f.shape[2], xe.shape[2]) and self.down_f.shape[1] % 16 == 0
                and os.environ.get("MEMARCH_BANK_I8", "1") != "0"):
            return _FrozenBankI8.apply(xe.contiguous(), *self._bank_i8(), self)
        return self._ffn(xe, self._bank_weights("up"), self._bank_weights("down"), train_w=False, counts=counts)

    def _experts(self, xe, wtab, C):
        cnt = getattr(self, "_counts", None)
        sub = (lambda idx: cnt.index_select(0, idx)) if cnt is not None else (lambda idx: None)
        if self.ep_W > 1:
            ye = self.ep_engine.ffn(self, xe)
        elif self.bank:
            if not self.has_F:
                ye = self._ffn(xe, self.up, self.down, counts=cnt)
            else:
                ye = xe.new_zeros(xe.shape)
                if self.has_L:
                    ye = ye.index_copy(0, self.L_idx, self._ffn(xe[self.L_idx], self.up, self.down,
                                                                counts=sub(self.L_idx)).to(ye.dtype))
                ye = ye.index_copy(0, self.F_idx, self._ffn_frozen(xe[self.F_idx], sub(self.F_idx)).to(ye.dtype))
        else:
            up, down = self.up, self.down
            if self.wave:
                fr = self.learned[:, None, None]
                up, down = torch.where(fr, up.detach(), up), torch.where(fr, down.detach(), down)
            if self.n_frozen:
                Ea = self.E - self.n_frozen
                ye = torch.cat([self._ffn(xe[:Ea], up, down, counts=cnt[:Ea].contiguous() if cnt is not None else None),
                                self._ffn(xe[Ea:], self.up_f, self.down_f, train_w=False,
                                          counts=cnt[Ea:].contiguous() if cnt is not None else None)])
            else:
                ye = self._ffn(xe, up, down, counts=cnt)
        if self.wave and self.training:
            ye = _ErrProbe.apply(ye, self.err)
            if not self.bank:
                if self.hint_now:
                    self.hint = self._hint(xe, ye, wtab.view(self.E, C))
                    with torch.no_grad():
                        self.hint_avg[0].mul_(0.9).add_(0.1 * self.hint.detach())
                else:
                    self.hint = torch.zeros((), device=xe.device)
                self.aux = self.aux + self.hint_w * self.hint
        return ye

    def _teachers(self):
        """For every expert the learned expert that teaches it: the students, in order, are dealt out `students` to a
        teacher, the teachers taken in order and round again.  (index per expert, who is a student at all)"""
        student = ~self.learned
        n_teachers = self.learned.sum()
        ranked = student.long().argsort(stable=True)              # learned experts first, in order
        seat = student.long().cumsum(0) - 1                       # a student's number among the students
        return ranked[(seat // self.students) % n_teachers.clamp(min=1)], student & (n_teachers > 0)

    def _hint(self, xe, ye, wt):
        """A learned expert (teacher) briefly pulls its students' outputs towards its own on the students' worst
        10 % of places (full2.py:604-619)."""
        teacher, student = self._teachers()
        with torch.no_grad():
            target = self._ffn(xe, self.up[teacher], self.down[teacher], train_w=False)
        gap = (ye.float() - target.float()).pow(2).mean(-1) * (wt > 0)          # per place, filled places only
        tenth = max(1, gap.shape[1] // 10)
        return (gap.topk(tenth, dim=1).values.mean(1) * student).sum() / student.sum().clamp(min=1)

    # ------------------------------------------------------------------------------------------ waves
    def _relative_move(self):
        """How far every expert's `up` moved since the last look, relative to its size; the look is renewed.  With a
        bank only the learning experts have weights here: the others count as not moved."""
        now, then = self.up.float(), self.up_snap.float()
        moved = (now - then).flatten(1).norm(dim=1) / (then.flatten(1).norm(dim=1) + 1e-8) if now.shape[0] else now.new_zeros(0)
        self.up_snap.copy_(self.up)
        if not self.bank:
            return moved.to(self.err.dtype)
        return torch.zeros(self.E, device=self.err.device).index_copy(0, self.L_idx, moved) if self.L else \
            torch.zeros(self.E, device=self.err.device)

    def _settled(self):
        """Experts that look finished at this check: by their error against its peak (`err`), or by how little they
        still move against their largest move (`still`; only experts that are learning here can be judged)."""
        if self.wave == "err":
            return self.err < self.err_thr * self.err_peak
        move = self._relative_move()
        self.move_peak.copy_(torch.maximum(self.move_peak, move.masked_fill(self.learned, 0.0)))
        self.last_move.copy_(move)
        quiet = (move < 0.3 * self.move_peak) & ~self.learned
        if self.bank:
            here = torch.zeros(self.E, dtype=torch.bool, device=move.device).index_fill(0, self.L_idx, True)
            quiet = quiet & here
        return quiet

    @torch.no_grad()
    def before_step(self, step):
        """Once per step, device-only: who has learned / who is a student again (full2.py:621-643, 1176-1196)."""
        if not self.wave:
            return
        check = step % self.wave_every == 0
        self.hint_now = (not self.bank) and step > 0 and check and bool(self.training)
        if not self.bank:
            self.up._frozen_rows = self.down._frozen_rows = self.learned        # the optimizer leaves these rows alone
        if not check or step < self.warm:
            return
        self.err_peak.copy_(torch.maximum(self.err_peak, self.err))
        settled = self._settled()
        fresh = settled & ~self.learned
        slipped = self.learned & (self.err > 1.5 * self.err_freeze)             # error grew since it froze: learn again
        self.err_freeze.copy_(torch.where(fresh, self.err, self.err_freeze))
        self.learned.copy_((self.learned | fresh) & ~slipped)

    def _moves(self, learned_cpu):
        """(experts that leave the learning bank, experts that come back from the frozen one) for a `learned` mask."""
        return [e for e in self.L if learned_cpu[e]], [e for e in self.Fz if not learned_cpu[e]]

    @torch.no_grad()
    def wants_rebank(self, learned_cpu):
        """Moving experts costs a re-layout of both tables: do it when anyone must thaw, when at least a quarter of the
        experts is ready to freeze, or when all remaining learners are."""
        freeze, thaw = self._moves(learned_cpu)
        return bool(thaw) or len(freeze) >= max(1, self.E // 4) or (bool(freeze) and len(freeze) == len(self.L))

    def _whole_table(self, which):
        """All E experts of `up` / `down` in fp32, learners and (expanded) frozen ones at their expert index."""
        live = getattr(self, which)
        table = torch.empty(self.E, *live.shape[1:], device=live.device, dtype=torch.float32)
        if self.L:
            table[self.L_idx] = live.detach().float()
        if self.Fz:
            table[self.F_idx] = self._bank_weights(which).float()
        return table

    @torch.no_grad()
    def rebank(self, learned_cpu):
        """Move experts between the learning and the frozen bank.  Returns [(old param, new param, slot map)] so
        the optimizer can carry momentum of the experts that keep learning (full2.py:1206-1242)."""
        freeze, thaw = self._moves(learned_cpu)
        learners = sorted((set(self.L) - set(freeze)) | set(thaw))
        bank = sorted((set(self.Fz) - set(thaw)) | set(freeze))
        came_from = [self.L.index(e) if e in self.L else None for e in learners]      # old row of every new learner
        dev = self.up.device
        changes = []
        for which in ("up", "down"):
            old = getattr(self, which)
            table = self._whole_table(which)
            rows = table[torch.tensor(learners, device=dev, dtype=torch.long)] if learners else table[:0]
            new = nn.Parameter(rows.to(self.w_dtype).contiguous())
            setattr(self, which, new)
            if bank:
                stored, scale = self._quantise(table[torch.tensor(bank, device=dev, dtype=torch.long)])
            else:
                stored, scale = getattr(self, which + "_f")[:0], getattr(self, which + "_fs")[:0]
            setattr(self, which + "_f", stored)
            setattr(self, which + "_fs", scale)
            changes.append((old, new, came_from))
        self.set_banks(learners, bank)
        return changes

    def set_banks(self, L, Fz):
        dv = self.up.device
        self.L, self.Fz = list(L), list(Fz)
        self.has_L, self.has_F = bool(L), bool(Fz)
        self.L_idx = torch.tensor(self.L, device=dv, dtype=torch.long)
        self.F_idx = torch.tensor(self.Fz, device=dv, dtype=torch.long)
        self.up_snap = self.up.detach().clone()

    def grow_bank(self, n_frozen, seed=0):
        """Wave-trained layout used by the 48-expert benchmark config: append `n_frozen` random-init frozen bf16
        experts to the bank; the router grows to E + n_frozen outputs."""
        assert self.bank and not self.Fz
        d = self.up.shape[1]
        g = torch.Generator().manual_seed(seed)
        E0, E1 = self.E, self.E + n_frozen
        dv = self.up.device
        self.up_f = (torch.randn(n_frozen, d, self.width_in, generator=g, device="cpu") * d ** -0.5).bfloat16().to(dv)
        self.down_f = (torch.randn(n_frozen, self.width_out, d, generator=g, device="cpu") * self.width_out ** -0.5 * 0.5
                       ).bfloat16().to(dv)
        self.up_fs = torch.zeros(n_frozen, 1, self.width_in, dtype=torch.bfloat16, device=dv)
        self.down_fs = torch.zeros(n_frozen, 1, d, dtype=torch.bfloat16, device=dv)
        r = torch.cat([self.router.weight.detach(),
                       (torch.randn(n_frozen, d, generator=g, device="cpu") * d ** -0.5).to(self.router.weight)])
        self.router = nn.Linear(d, E1, bias=False).to(r.device)
        with torch.no_grad():
            self.router.weight.copy_(r)
        for nm in ("err", "err_peak", "err_freeze", "move_peak", "last_move", "hint_avg"):
            setattr(self, nm, torch.cat([getattr(self, nm), torch.zeros(n_frozen, device=dv)]))
        self.learned = torch.cat([self.learned, torch.ones(n_frozen, dtype=torch.bool, device=dv)])
        self.E = E1
        self.set_banks(list(range(E0)), list(range(E0, E1)))

    # ------------------------------------------------------------------------------------------ EP
    def ep_shard(self, rank, W, engine):
        """Keep only this rank's E/W learning experts; expert grads are sums over ranks, so the hook divides by W
        (full2.py:1122-1135).  With a frozen bank the bank is sharded the same way (new capability: the
        reference asserts `not has_F` here)."""
        nL = len(self.L) if self.bank else self.up.shape[0]
        assert nL % W == 0, "EP: learning experts must divide by the world size"
        El = nL // W
        sl = slice(rank * El, (rank + 1) * El) if self.up.shape[0] == nL else slice(0, El)
        self.up = nn.Parameter(self.up.detach()[sl].to(self.w_dtype).clone())
        self.down = nn.Parameter(self.down.detach()[sl].to(self.w_dtype).clone())
        if self.bank and self.has_F:
            nF = len(self.Fz)
            assert nF % W == 0, "EP: frozen experts must divide by the world size"
            Fl = nF // W
            fs = slice(rank * Fl, (rank + 1) * Fl)
            for nm in ("up_f", "down_f", "up_fs", "down_fs"):
                setattr(self, nm, getattr(self, nm)[fs].clone())
        if hasattr(self, "up_snap"):
            self.up_snap = self.up.detach().clone()
        self.ep_W, self.ep_rank, self.ep_engine = W, rank, engine
        for p in (self.up, self.down):
            p.register_hook(lambda g, W=W: g / W)
            p._ep_local = True
