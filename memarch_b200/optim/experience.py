"""The first optimizer of the family: experience cards with a momentum per card.

`ExperienceOpt` (exp_opt.py:21-108 of the reference; what its stage `X` without `B` builds unless OPT_KW asks for the
instinct kind).  K situation cards, each with a key in "what the model reads" space, an expected loss and ITS OWN
momentum for every weight: a batch is recognised by its input before the loss is known, the most similar card's
momentum takes the gradient, and the step comes from that momentum normalised over the tensor (per row for word
tables).  Surprise s = (expected - loss) / expected widens the whole step when the batch went better than the card
expected and strengthens only the weights with the largest gradients when it went worse.  It reads the loss on the
host every step and keeps K momenta per weight - the later `Instinct` (one momentum, device-only) replaced it; it is
here because the registry of training stages still offers it (`OptConfig(kind="experience")`).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


class ExperienceOpt:
    def __init__(self, params, lr=1e-3, weight_decay=0.1, cards=4, beta=0.9, new_card=0.5, good=4.0, bad=6.0,
                 max_good=2.0, max_bad=3.0, top=0.1, ema=0.98, m_dtype="bf16", surprise=True, norm="tensor", scale=0.2, **_):
        self.plist = list(params)
        self.param_groups = [dict(lr=lr, weight_decay=weight_decay)]
        self.K, self.beta, self.new_card, self.ema = cards, beta, new_card, ema
        self.good, self.bad, self.max_good, self.max_bad, self.top = good, bad, max_good, max_bad, top
        self.m_dtype = torch.float32 if m_dtype == "fp32" else torch.bfloat16
        self.surprise, self.norm, self.scale = surprise, norm, scale
        self.keys = None                                   # (K, d_sit), unit rows
        self.used = [False] * cards
        self.expect = [None] * cards
        self.m = [None] * len(self.plist)                  # per weight: (K, *shape) momenta, made on first use
        self.seen = [[False] * cards for _ in self.plist]
        self.last = dict(card=0, s=0.0)

    # ------------------------------------------------------------------------------------------ cards
    @torch.no_grad()
    def pick(self, situation):
        """The card of this batch: the most similar used card, or a free one when nothing is similar enough."""
        sit = F.normalize(situation.float().flatten(), dim=0)
        if self.keys is None:
            self.keys = torch.zeros(self.K, sit.numel(), device=sit.device)
        k = 0
        if any(self.used):
            sim = (self.keys @ sit).tolist()
            best = max((i for i in range(self.K) if self.used[i]), key=lambda i: (sim[i], -i))
            free = [i for i in range(self.K) if not self.used[i]]
            k = free[0] if (sim[best] < self.new_card and free) else best
        if self.used[k]:
            self.keys[k] = F.normalize(0.95 * self.keys[k] + 0.05 * sit, dim=0)      # the key follows its situations
        else:
            self.keys[k], self.used[k] = sit, True
        return k

    def _surprise(self, k, loss):
        if self.expect[k] is None:
            self.expect[k] = loss
        s = (self.expect[k] - loss) / max(self.expect[k], 1e-6)
        self.expect[k] = self.ema * self.expect[k] + (1 - self.ema) * loss
        return s

    # ------------------------------------------------------------------------------------------ step
    def _direction(self, p, m, grad):
        if p.dim() == 2 and p.shape[0] >= 10000:           # word tables: a scale per word, rows without a lesson stay
            rms = m.pow(2).mean(1, keepdim=True).sqrt()
            return torch.where(grad.abs().sum(1, keepdim=True) > 0, m / (rms + 1e-8), torch.zeros_like(m))
        if self.norm == "row" and p.dim() >= 2:
            rms = m.pow(2).flatten(1).mean(1).sqrt().view(-1, *[1] * (p.dim() - 1))
            return m / (rms + 1e-8)
        return m / (m.pow(2).mean().sqrt() + 1e-8)

    @torch.no_grad()
    def step(self, loss, situation):
        k = self.pick(situation)
        s = self._surprise(k, float(loss))
        self.last = dict(card=k, s=s)
        lr, wd = self.param_groups[0]["lr"], self.param_groups[0]["weight_decay"]
        for i, p in enumerate(self.plist):
            if p.grad is None:
                continue
            if self.m[i] is None:
                self.m[i] = torch.zeros(self.K, *p.shape, device=p.device, dtype=self.m_dtype)
            grad = p.grad.float()
            if not self.seen[i][k]:                         # a new card starts from the experience of an existing one
                if any(self.seen[i]):
                    self.m[i][k] = self.m[i][self.seen[i].index(True)]
                self.seen[i][k] = True
            m = self.m[i][k].float().mul_(self.beta).add_(grad, alpha=1 - self.beta)
            self.m[i][k] = m.to(self.m_dtype)
            upd = self._direction(p, m, grad)
            if self.surprise and s > 0:
                upd = upd * min(self.max_good, 1 + self.good * s)
            elif self.surprise and s < 0:
                mag = grad.abs().flatten()
                if mag.numel() > 65536:
                    mag = mag[torch.randint(0, mag.numel(), (65536,), device=mag.device)]
                guilty = (grad.abs() >= mag.quantile(1 - self.top)).float()
                upd = upd * (1 + guilty * (min(self.max_bad, 1 + self.bad * -s) - 1))
            word_table = p.dim() == 2 and p.shape[0] >= 10000
            if wd and p.dim() >= 2 and not word_table:
                p.mul_(1 - lr * wd)
            p.add_(upd.to(p.dtype), alpha=-lr * self.scale)

    def zero_grad(self, set_to_none=True):
        for p in self.plist:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()

    def state_dict(self):
        return {"m": self.m, "seen": self.seen, "keys": self.keys, "used": self.used, "expect": self.expect,
                "lr": self.param_groups[0]["lr"]}

    def load_state_dict(self, sd):
        self.m, self.seen, self.keys, self.used, self.expect = sd["m"], sd["seen"], sd["keys"], sd["used"], sd["expect"]
        self.param_groups[0]["lr"] = sd.get("lr", self.param_groups[0]["lr"])
