"""Light (sliding-window) transformer blocks, dense FFN heavy layer and the plain transformer baseline.

Parameter names follow the reference so checkpoints interchange: `n1, qkv, o, n2, up, down` per block
(baseline.py:35-52), FFN `norm, up, down` (lm.py:45-50).  Block variants are the reference's `BLK` set
(full.py:113-182): zero, ve, x0, relu2, relu2c, qk, qkv3; `LIGHT_FFN`, `LIGHT_MOE`; opaque-token FFN skipping.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


def _cdt(x):
    """Compute dtype of matmul operands: bf16 on the GPU (tcgen05), the tensor's own dtype on CPU."""
    return torch.bfloat16 if x.is_cuda else x.dtype


class FineMoE(nn.Module):
    """Light-layer MoE: E small SwiGLU experts, k active per token, fixed capacity (full.py:51-91)."""

    def __init__(self, d, E=32, k=4, hid=None):
        super().__init__()
        self.E, self.k = E, k
        h = hid or 4 * d // k
        self.router = nn.Linear(d, E, bias=False)
        self.up = nn.Parameter(torch.randn(E, d, 2 * h) * d ** -0.5)
        self.down = nn.Parameter(torch.randn(E, h, d) * h ** -0.5)
        self.aux = torch.zeros(())

    def forward(self, x):
        """Dispatch without a sort and combine without atomics: a (token, choice) pair's place inside its expert is
        the running count of earlier pairs of that expert (token order, so the first to ask are served when an expert
        is over capacity, as the reference's stable sort by expert does); every token then sums its own k results."""
        E, k, d = self.E, self.k, x.shape[-1]
        tokens = x.reshape(-1, d)
        N = tokens.shape[0]
        scores = F.linear(tokens.float(), self.router.weight.float())
        top, chosen = scores.topk(k, -1)
        share = top.softmax(-1)                                             # (N,k) weights of the chosen experts
        asked = F.one_hot(chosen, E)                                        # (N,k,E)
        self.aux = E * ((asked.float().sum(1).mean(0) / k) * scores.softmax(-1).mean(0)).sum()   # load x importance
        cap = int(1.25 * N * k / E) + 1
        place = (asked.view(N * k, E).cumsum(0) - 1).gather(1, chosen.view(-1, 1)).view(N, k)
        served = place < cap
        spill = E * cap                                                      # one extra row takes what does not fit
        cell = torch.where(served, chosen * cap + place, torch.full_like(place, spill))
        rows = tokens.new_zeros(spill + 1, d).index_copy(0, cell.view(-1), tokens.repeat_interleave(k, 0))
        out = ops.expert_ffn(rows[:-1].view(E, cap, d).to(_cdt(x)), self.up, self.down, "swiglu").reshape(spill, d)
        out = torch.cat([out, out.new_zeros(1, d)])
        mine = out[cell] * (share * served)[..., None].to(out.dtype)         # (N,k,d), zero where dropped
        return mine.to(tokens.dtype).sum(1).view(x.shape)


class LightBlock(nn.Module):
    """RMSNorm -> qkv -> RoPE + causal/window attention -> o ; RMSNorm -> FFN (SwiGLU 4d or relu² 6d)."""

    def __init__(self, d, heads, blk=(), light_ffn=0.0, light_moe="", vocab_heads=None, rope_half=False):
        super().__init__()
        self.heads, self.blk, self.rope_half = heads, set(blk), rope_half
        self.attn_gain, self.tether_pcut = 1.0, 0.0      # sharper attention scores; p-RoPE of a tethered layer
        self.n1 = nn.RMSNorm(d)
        self.qkv = nn.Linear(d, 3 * d, bias=False)
        self.o = nn.Linear(d, d, bias=False)
        self.n2 = nn.RMSNorm(d)
        self.relu2 = "relu2" in self.blk or "relu2c" in self.blk
        if self.relu2:
            self.up = nn.Linear(d, 6 * d, bias=False)
            self.down = nn.Linear(6 * d, d, bias=False)
        else:
            self.up = nn.Linear(d, 8 * d, bias=False)
            self.down = nn.Linear(4 * d, d, bias=False)
        if light_ffn:
            hid = max(256, int(round(light_ffn * d / 256)) * 256)
            self.up = nn.Linear(d, hid if self.relu2 else 2 * hid, bias=False)
            self.down = nn.Linear(hid, d, bias=False)
        if "zero" in self.blk:
            nn.init.zeros_(self.o.weight)
            nn.init.zeros_(self.down.weight)
        if "ve" in self.blk:
            self.ve_gate = nn.Linear(d, heads, bias=False)
            nn.init.zeros_(self.ve_gate.weight)
        if "x0" in self.blk:
            self.x0_l = nn.Parameter(torch.zeros(()))
        if light_moe:
            E, k = map(int, light_moe.split(":"))
            self.moe = FineMoE(d, E, k)
            del self.up, self.down
        self.cur_ve = self.cur_x0 = self.cur_sel = None
        for nm in ("qkv", "o", "up", "down"):
            if hasattr(self, nm):
                # used once per step through a bf16 shadow: the data-parallel engine may keep its optimizer state
                # and update row-sharded across the ranks
                getattr(self, nm).weight._shard_ok = True

    def _act(self, h):
        return ops.relu2(h) if self.relu2 else ops.swiglu(h)

    def forward(self, x, window=None, pending=None, defer=False, tether=None):
        """`pending`: the previous block's FFN output not yet added to the stream (added here, fused with n1).
        `defer=True` returns (x, ffn_out) and leaves the last residual add to the next block.
        `tether` = (own, apos, avalid, RopeCfg, routed, qmask, docs): the attention becomes the anchor-routed read of
        `models.rope_memory` (local window + the spans of the anchors each query opens); what it chose and how much
        of the softmax mass went there is left in `self.tether_out` = (share, route, mass per position)."""
        B, T, D = x.shape
        hd = D // self.heads
        dt = _cdt(x)
        if self.cur_x0 is not None:
            if pending is not None:
                x, pending = ops.resid_add(x, pending), None
            x = x + self.x0_l * self.cur_x0
        if pending is not None:
            x, n1 = ops.add_rmsnorm(x, pending, self.n1.weight, self.n1.eps)
        else:
            n1 = ops.rmsnorm(x, self.n1.weight, self.n1.eps, out_dtype=dt)
        qkv = ops.linear(n1, self.qkv.weight, direct=True).view(B, T, 3, self.heads, hd)
        if self.attn_gain != 1.0:
            qkv = torch.stack([qkv[:, :, 0] * self.attn_gain, qkv[:, :, 1], qkv[:, :, 2]], 2)
        if self.cur_ve is not None:
            g = 2 * torch.sigmoid(F.linear(x, self.ve_gate.weight.to(x.dtype)))[..., None]        # (B,T,H,1)
            v = qkv[:, :, 2] + (g * self.cur_ve.view(B, T, self.heads, hd)).to(qkv.dtype)
            qkv = torch.stack([qkv[:, :, 0], qkv[:, :, 1], v], 2)
        if tether is not None:
            from ..ops import ref
            from .rope_memory import rope_attention
            q, k, v = qkv.permute(2, 0, 3, 1, 4)
            if "qk" in self.blk:
                q, k = F.rms_norm(q, (hd,)), F.rms_norm(k, (hd,))
            cos, sin = ref.rope_angles(T, hd, x.device, pcut=self.tether_pcut)
            q, k = ref.apply_rope(q, cos, sin, self.rope_half), ref.apply_rope(k, cos, sin, self.rope_half)
            own, apos, avalid, rcfg, routed, qmask, docs = tether
            a, share, route, mass = rope_attention(q, k, v, own, apos, avalid, rcfg, routed, qmask, docs, want_mass=True)
            self.tether_out = (share, route, mass)
            a = a.transpose(1, 2).reshape(B, T, D).to(dt)
        else:
            a = ops.attention(qkv, window, self.rope_half, qk_norm="qk" in self.blk)
        fin = (lambda t: (t, None)) if defer else (lambda t: t)
        if hasattr(self, "moe") or self.cur_sel is not None:
            x = ops.resid_add(x, ops.linear(a, self.o.weight))
        if hasattr(self, "moe"):
            return fin(x + self.moe(ops.rmsnorm(x, self.n2.weight, self.n2.eps)))
        if self.cur_sel is not None:                      # opaque tokens only: FFN skipped where the talker is sure
            idx, ok = self.cur_sel
            xs = ops.rmsnorm(x, self.n2.weight, self.n2.eps, out_dtype=dt).gather(1, idx[..., None].expand(-1, -1, D))
            y = ops.linear(self._act(ops.linear(xs, self.up.weight)), self.down.weight) * ok[..., None].to(dt)
            return fin(x.scatter_add(1, idx[..., None].expand(-1, -1, D), y.to(x.dtype)))
        x, n2 = ops.add_rmsnorm(x, ops.linear(a, self.o.weight, direct=True), self.n2.weight, self.n2.eps)
        y = ops.ffn(n2, self.up.weight, self.down.weight, "relu2" if self.relu2 else "swiglu", direct=True)
        if defer:
            return x, y
        return ops.resid_add(x, y)


def run_blocks(blocks, x, window, run=None):
    """A stack of light blocks with the residual add at each block boundary fused into the next block's norm."""
    pending = None
    for b in blocks:
        if run is not None:
            x, pending = run(b, x, window, pending, True)
        else:
            x, pending = b(x, window, pending, True)
    return x if pending is None else ops.resid_add(x, pending)


class DenseFFN(nn.Module):
    """Attention-free heavy layer on anchors: x + down(SwiGLU(up(norm(x)))) (lm.py:45-60)."""

    def __init__(self, d):
        super().__init__()
        self.norm = nn.RMSNorm(d)
        self.up = nn.Linear(d, 8 * d, bias=False)
        self.down = nn.Linear(4 * d, d, bias=False)

    def forward(self, x, surprise=None):
        n = ops.rmsnorm(x, self.norm.weight, self.norm.eps, out_dtype=_cdt(x))
        return x + ops.linear(ops.swiglu(ops.linear(n, self.up.weight)), self.down.weight).to(x.dtype)


class TransformerLM(nn.Module):
    """Llama-style baseline (`T300`, `Td<d>L<L>`, lm.py:128-140): the control the reference races against."""

    def __init__(self, vocab, d=512, layers=8, heads=8, fused_ce=True):
        super().__init__()
        self.vocab, self.fused_ce = vocab, fused_ce
        self.emb = nn.Embedding(vocab, d)
        self.blocks = nn.ModuleList(LightBlock(d, heads) for _ in range(layers))
        self.norm = nn.RMSNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)
        self.stats = {}

    def vocab_shard(self, rank, world, group=None):
        """Vocabulary parallelism: keep rows [rank V/W, (rank+1) V/W) of the input table and of the output head.  Every
        rank then serves its rows for the tokens of all ranks (`parallel/vocab.py`: ids and states are gathered, the
        cross-entropy is a two-stage log-sum-exp), so a 131k-word vocabulary costs each GPU 1/W of both tables, of
        their optimizer state and of the head's FLOPs.  The shards are rank-local parameters: their gradient already
        holds the contribution of every rank's tokens, W times the scale of a rank-mean gradient (see `train_loss`), and
        is divided by W in a hook."""
        from ..parallel import vocab as vp
        assert self.vocab % world == 0, "vocabulary rows must divide by the world size"
        self._vp = (rank, world, group, rank * (self.vocab // world))
        for mod in (self.emb, self.head):
            shard = nn.Parameter(vp.shard_rows(mod.weight.detach(), rank, world)[0])
            shard._ep_local = True                       # no data-parallel averaging: see above
            shard.register_hook(lambda g, w=world: g / w)
            mod.weight = shard
        return self

    def forward(self, x, prep=None):
        vpar = getattr(self, "_vp", None)
        if vpar is not None:
            from ..parallel import vocab as vp
            h = vp.take_dp(self.emb.weight, x, vpar[3], vpar[2])
        else:
            h = self.emb(x)
        h = run_blocks(self.blocks, h, None)
        return ops.rmsnorm(h, self.norm.weight, self.norm.eps, out_dtype=_cdt(h)), torch.zeros((), device=x.device)

    def train_loss(self, out, y, train=True):
        vpar = getattr(self, "_vp", None)
        if vpar is not None:
            # S = summed loss of ALL ranks' tokens (the same number on every rank); this rank's backward reaches the
            # replicated weights only through its own tokens.  Gradient of S / (own token count): its mean over the
            # ranks is the gradient of the mean loss per token, which is what data-parallel averaging assumes.
            # Value: the mean loss per token of the whole batch.
            from ..parallel import vocab as vp
            per_own = vp.ce_dp(out.reshape(-1, out.shape[-1]).float(), self.head.weight.float(), y.reshape(-1), vpar[3], vpar[2]) / y.numel()
            return per_own.detach() / vpar[1] + (per_own - per_own.detach())
        if self.fused_ce and self.training:
            return ops.linear_ce(out, self.head.weight, y) / y.numel()
        lo = ops.linear(out, self.head.weight).float()
        return F.cross_entropy(lo.reshape(-1, lo.shape[-1]), y.reshape(-1))
