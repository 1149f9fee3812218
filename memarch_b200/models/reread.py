"""Re-reading at a bookmark with recognition.

A word picks cards by face, jumps to each card's bookmark, re-reads up to R raw tokens from the shelf table
(`book`) with an ACT-style halting cost per token read, and the card checks that what was read matches it.
Semantics of the reference `Reread` (full2.py:184-280); parameter names identical (`offset, norm, query, halt_v,
halt_h, recog_r, recog_c, out`).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class Reread(nn.Module):
    def __init__(self, d, d_face=64, d_book=128, top_k=4, max_read=4):
        super().__init__()
        self.k, self.R, self.df = top_k, max_read, d_face
        self.norm = nn.RMSNorm(d)
        self.query = nn.Linear(d, d_face, bias=False)
        self.offset = nn.Parameter(torch.randn(max_read, d_book) * 0.02)
        self.halt_v = nn.Linear(d_book, 1)
        self.halt_h = nn.Linear(d, 1, bias=False)
        self.recog_r = nn.Linear(d_book, d_face, bias=False)
        self.recog_c = nn.Linear(d, d_face, bias=False)
        self.out = nn.Linear(d_book, d, bias=False)

    def forward(self, h, ids, table, faces, contents, pos, valid, qpos, rows=None):
        """h (B,S,d) words of a segment; ids (Bt,T) token ids of the texts and `table` (V,Db) the shelf;
        cards: faces (B,C,L,f), contents (B,C,d), pos/valid (B,C); qpos (B,S) text positions of the words;
        rows (B,) text of every batch row.  Returns (addition to h, expected tokens read per word)."""
        B, S = h.shape[:2]
        n = self.norm(h)
        q = F.normalize(self.query(n), dim=-1)
        sc = torch.einsum("bsf,bclf->bscl", q, F.normalize(faces, dim=-1)).amax(-1) * math.sqrt(self.df)
        sc = sc.masked_fill(~valid[:, None], -1e4)
        k = min(self.k, sc.shape[-1])
        top_s, top_j = sc.topk(k, -1)
        w = F.softmax(top_s.float(), -1).type_as(h) * (top_s > -1e3)
        mark = pos.gather(1, top_j.reshape(B, -1)).view(B, S, k)
        rpos = mark[..., None] + torch.arange(self.R, device=h.device)
        readable = rpos < qpos[:, :, None, None]
        Tb, Db = ids.shape[1], table.shape[1]
        rpos = rpos.clamp(0, Tb - 1)
        if rows is None:
            rows = torch.arange(B, device=h.device)
        flat = (rows[:, None, None, None] * Tb + rpos).reshape(-1)
        v = F.embedding(ids.reshape(-1)[flat], table).float().view(B, S, k, self.R, Db) + self.offset
        halt = torch.sigmoid(self.halt_v(v).squeeze(-1) + self.halt_h(n)[:, :, None])
        halt = torch.where(readable, halt, torch.ones_like(halt))
        halt = torch.cat([halt[..., :-1], torch.ones_like(halt[..., -1:])], -1)
        stay = 1 - halt[..., :-1]
        surv = [torch.ones_like(halt[..., 0])]
        for i in range(stay.shape[-1]):
            surv.append(surv[-1] * stay[..., i])
        survive = torch.stack(surv, -1)
        read = ((survive * halt * readable)[..., None] * v).sum(-2)
        cp = self.recog_c(contents)
        card_p = cp.gather(1, top_j.reshape(B, -1, 1).expand(-1, -1, cp.shape[-1])).view(B, S, k, -1)
        recog = torch.sigmoid((F.normalize(self.recog_r(read), dim=-1) * F.normalize(card_p, dim=-1))
                              .sum(-1, keepdim=True) * 4)
        got = (w[..., None] * recog * read).sum(-2)
        cost = (w * (survive * readable).sum(-1)).sum(-1).mean()
        return self.out(got), cost
