"""Re-reading at a bookmark with recognition.

A word scores the cards of its text's memory by face, takes its `top_k` best, jumps to each card's bookmark and reads
up to `max_read` raw tokens of the text from the shelf table (`book`); an ACT-style gate decides after each token
whether to stop, the card checks that what was read matches it, and the expected number of tokens read is the cost.
Behaviour of the reference `Reread` (full2.py:184-280); parameter names are the reference's (`offset, norm, query,
halt_v, halt_h, recog_r, recog_c, out`) so its checkpoints load.

On the GPU the pass is three fused steps: card scores (`csrc/memops.cu`, shared with the memory read), then one
kernel for pick / gather / halting / recognition with its own backward (`csrc/reread.cu`) and the output projection.
The PyTorch statement below is the CPU path and the oracle of the kernel tests.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import _ext


class _RereadCore(torch.autograd.Function):
    """(scores, bookmarks, text, shelf, small weights) -> (what was read and recognised (B,S,Db), tokens read (B,S))."""

    @staticmethod
    def forward(ctx, sc, pos, qpos, rows, ids, table, offset, hv, hb, hh, Wr, cp, k):
        got, costw, top_j, p = _ext.C().reread_fwd(sc, pos, qpos, rows, ids, table, offset, hv, hb, hh, Wr, cp, int(k))
        _ext.count()
        ctx.save_for_backward(sc, pos, qpos, rows, ids, table, offset, hv, hb, hh, Wr, cp, top_j, p)
        return got, costw

    @staticmethod
    def backward(ctx, dgot, dcostw):
        sc, pos, qpos, rows, ids, table, offset, hv, hb, hh, Wr, cp, top_j, p = ctx.saved_tensors
        dgot = torch.zeros_like(sc[..., :1]).expand(*sc.shape[:2], table.shape[1]) if dgot is None else dgot
        dcostw = torch.zeros_like(hh) if dcostw is None else dcostw
        dsc, dtable, doff, dhv, dhb, dhh, dWr, dcp = _ext.C().reread_bwd(
            dgot.contiguous().float(), dcostw.contiguous().float(), top_j, p, sc, pos, qpos, rows, ids, table, offset, hv,
            hb, hh, Wr, cp)
        _ext.count()
        return (dsc, None, None, None, None, dtable.to(table.dtype), doff, dhv.view_as(hv), dhb.view_as(hb),
                dhh.view_as(hh), dWr, dcp, None)


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

    # ------------------------------------------------------------------------------------------ pieces (PyTorch)
    def _scores(self, q, faces, valid):
        """Best cosine over a card's chain of faces, times sqrt(d_face); -1e4 on empty cards."""
        cos = torch.einsum("bsf,bclf->bscl", q, F.normalize(faces, dim=-1)).amax(-1)
        return (cos * math.sqrt(self.df)).masked_fill(~valid[:, None], -1e4)

    def _tokens_at(self, mark, qpos, ids, rows):
        """Token ids at `mark + 0..R-1` of each row's text and whether each position is already written."""
        at = mark[..., None] + torch.arange(self.R, device=mark.device)
        seen = at < qpos[:, :, None, None]
        text = ids[rows]                                                    # (B, Tb)
        B = at.shape[0]
        tok = text.gather(1, at.clamp(0, ids.shape[1] - 1).reshape(B, -1)).view(at.shape)
        return tok, seen

    def _halting(self, v, hh, seen):
        """(weight of every token in the read, probability of still reading at every token)."""
        stop = torch.sigmoid(self.halt_v(v).squeeze(-1) + hh[:, :, None, None])
        stop = torch.where(seen, stop, torch.ones_like(stop))
        stop = torch.cat([stop[..., :-1], torch.ones_like(stop[..., :1])], -1)          # the last token always stops
        going = torch.cat([torch.ones_like(stop[..., :1]), (1 - stop[..., :-1]).cumprod(-1)], -1)
        return going * stop * seen, going * seen

    def _core_torch(self, sc, pos, qpos, rows, ids, table, hh, cp):
        B, S, C = sc.shape
        k = min(self.k, C)
        best, pick = sc.topk(k, -1)
        w = F.softmax(best.float(), -1).type_as(sc) * (best > -1e3)
        mark = pos.gather(1, pick.reshape(B, -1)).view(B, S, k)
        tok, seen = self._tokens_at(mark, qpos, ids, rows)
        v = F.embedding(tok, table).float() + self.offset
        share, going = self._halting(v, hh, seen)
        read = torch.einsum("bskr,bskrd->bskd", share, v)
        card = cp.gather(1, pick.reshape(B, -1, 1).expand(-1, -1, cp.shape[-1])).view(B, S, k, -1)
        agree = F.cosine_similarity(self.recog_r(read), card, dim=-1, eps=1e-12)
        got = torch.einsum("bsk,bskd->bsd", w * torch.sigmoid(4 * agree), read)
        return got, (w * going.sum(-1)).sum(-1)

    # ------------------------------------------------------------------------------------------ forward
    def forward(self, h, ids, table, faces, contents, pos, valid, qpos, rows=None):
        """h (B,S,d) words of a segment; ids (Bt,T) token ids of the texts and `table` (V,Db) the shelf;
        cards: faces (B,C,L,f), contents (B,C,d), pos/valid (B,C); qpos (B,S) text positions of the words;
        rows (B,) text of every batch row.  Returns (addition to h, expected tokens read per word)."""
        B, S = h.shape[:2]
        if rows is None:
            rows = torch.arange(B, device=h.device)
        n = self.norm(h)
        q = F.normalize(self.query(n), dim=-1)
        hh = self.halt_h(n).squeeze(-1)
        cp = self.recog_c(contents)
        C = faces.shape[1]
        fused = (_ext.use_cuda(h) and h.dtype == torch.float32 and faces.dtype == torch.float32 and self.df == 64
                 and table.shape[1] == 128 and self.R <= 4 and self.k <= 8 and C <= 512 and faces.shape[2] <= 255
                 and cp.dtype == torch.float32)
        if fused:
            from .memory import _ReadScores
            zero = torch.zeros((), device=h.device)
            sc, _ = _ReadScores.apply(q, faces, valid, zero, C, math.sqrt(self.df))
            got, costw = _RereadCore.apply(
                sc.contiguous(), pos.contiguous(), qpos.contiguous(), rows.contiguous(), ids.contiguous(),
                table.contiguous(), self.offset, self.halt_v.weight, self.halt_v.bias, hh.contiguous(),
                self.recog_r.weight, cp.contiguous(), min(self.k, C))
        else:
            got, costw = self._core_torch(self._scores(q, faces, valid), pos, qpos, rows, ids, table, hh, cp)
        return self.out(got), costw.mean()
