"""Plain PyTorch statements of every op in this package.

These are the CPU path and the numerics oracle: each CUDA kernel in `csrc/` is tested against the function of the
same name here, run in fp32.  Nothing in this file is tuned; clarity wins.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# ----------------------------------------------------------------------------------------------- norms / acts
def rmsnorm(x, weight, eps=None):
    """fp32 normalise, multiply by weight, return in fp32 (the caller casts once)."""
    xf = x.float()
    if eps is None:
        eps = torch.finfo(x.dtype if x.dtype != torch.bfloat16 else torch.float32).eps
    r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return xf * r * weight.float()


def relu2(x):
    r = F.relu(x)
    return r * r


def swiglu(gu):
    g, u = gu.chunk(2, -1)
    return F.silu(g) * u


# ----------------------------------------------------------------------------------------------- rope / attention
def rope_angles(T, hd, device, base=10000.0, pos=None, pcut=0.0):
    """`pcut` > 0: only the frequencies whose wavelength 2 pi / inv is at most `pcut` words rotate; the other
    dimensions carry no position at all (memarch_jax/memarch_jax/prims.py:48-58 of the reference's JAX port)."""
    inv = 1.0 / base ** (torch.arange(0, hd, 2, device=device).float() / hd)
    if pcut > 0:
        inv = torch.where(2 * math.pi / inv <= pcut, inv, torch.zeros_like(inv))
    p = torch.arange(T, device=device).float() if pos is None else pos.float()
    ang = p[:, None] * inv[None]
    return ang.cos(), ang.sin()


def apply_rope(x, cos, sin, half=False):
    """x (..., T, hd); cos/sin (T, hd/2).  Interleaved pairs (0::2, 1::2) or halves layout (baseline.py:13-32)."""
    if half:
        x1, x2 = x.chunk(2, -1)
        return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], -1).type_as(x)
    x1, x2 = x[..., 0::2], x[..., 1::2]
    return torch.stack([x1 * cos - x2 * sin, x1 * sin + x2 * cos], -1).flatten(-2).type_as(x)


def window_attention(q, k, v, window=None, rope_half=False, pos=None, qk_norm=False):
    """Causal attention with RoPE and an optional sliding window `q - kv < window`.

    q, k, v: (B, T, H, hd).  Returns (B, T, H, hd).  Dense masked softmax in fp32: the oracle, not a fast path.
    """
    B, T, H, hd = q.shape
    q, k, v = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    if qk_norm:
        q, k = F.rms_norm(q, (hd,)), F.rms_norm(k, (hd,))
    cos, sin = rope_angles(T, hd, q.device, pos=pos)
    q, k = apply_rope(q, cos, sin, rope_half), apply_rope(k, cos, sin, rope_half)
    s = torch.einsum("bhqd,bhkd->bhqk", q.float(), k.float()) * hd ** -0.5
    i = torch.arange(T, device=q.device)
    ok = i[None, :] <= i[:, None]
    if window is not None and window < T:
        ok = ok & (i[:, None] - i[None, :] < window)
    s = s.masked_fill(~ok, float("-inf"))
    p = s.softmax(-1)
    o = torch.einsum("bhqk,bhkd->bhqd", p, v.float()).to(v.dtype)
    return o.permute(0, 2, 1, 3)


# ----------------------------------------------------------------------------------------------- cross entropy
def ce_rows(logits, y, gate=None, hit=None):
    """Per-row loss and d(loss)/d(logits) for plain CE or the pointer mixture.

    Mixture (fused_ops.py:104-134): P = (1-g)·softmax(x)[y] + g·hit, loss = -log max(P, 1e-30),
    dlogits = w·(softmax - onehot) with w = (1-g)·p_y/P, dloss/dg = (p_y - hit)/P.
    Returns (loss (n,), grad (n, V) fp32, dg (n,) or None).
    """
    lf = logits.float()
    lse = torch.logsumexp(lf, -1)
    xy = lf.gather(-1, y[:, None])[:, 0]
    sm = (lf - lse[:, None]).exp()
    oh = F.one_hot(y, lf.shape[-1]).to(sm.dtype)
    if gate is None:
        return lse - xy, sm - oh, None
    py = (xy - lse).exp()
    P = ((1 - gate) * py + gate * hit).clamp(min=1e-30)
    w = (1 - gate) * py / P
    return -torch.log(P), w[:, None] * (sm - oh), (py - hit) / P


def linear_ce(h, w, y, bias=None, gate=None, hit=None, cand=None, cval=None, chunk=4096, mm_dtype=None):
    """Sum of per-row losses of `h @ w.T (+bias)` against `y`, with grads made in the same pass.

    Returns (loss_sum, gh (N,d), gw (V,d) fp32, gbias (V,) or None, dgate (N,) or None, dcval or None).
    `mm_dtype` rounds the matmul operands and the logits the way the bf16 GPU path does.
    """
    N, d = h.shape
    V = w.shape[0]
    dt = mm_dtype or h.dtype
    hd, wd = h.to(dt), w.to(dt)
    gh = torch.empty(N, d, dtype=dt, device=h.device)
    gw = torch.zeros(V, d, dtype=torch.float32, device=h.device)
    gb = torch.zeros(V, dtype=torch.float32, device=h.device) if bias is not None else None
    dg = torch.empty(N, dtype=torch.float32, device=h.device) if gate is not None else None
    dcv = torch.empty_like(cval, dtype=torch.float32) if cval is not None else None
    total = torch.zeros((), dtype=torch.float32, device=h.device)
    for i in range(0, N, chunk):
        sl = slice(i, i + chunk)
        logits = hd[sl] @ wd.T
        if bias is not None:
            logits = (logits.float() + bias.float()).to(dt)
        if cand is not None:
            logits = logits.float().scatter_add(-1, cand[sl], cval[sl].float()).to(dt)
        loss, G, dgi = ce_rows(logits, y[sl], None if gate is None else gate[sl].float(),
                               None if hit is None else hit[sl].float())
        total = total + loss.sum()
        Gd = G.to(dt)
        gh[sl] = Gd @ wd
        gw += (Gd.T @ hd[sl]).float()
        if gb is not None:
            gb += G.sum(0)
        if dg is not None:
            dg[sl] = dgi
        if dcv is not None:
            dcv[sl] = G.gather(-1, cand[sl])
    return total, gh, gw, gb, dg, dcv


def chunk_lse(h, w, bias, y, ch, mm_dtype=torch.bfloat16):
    """(lse, logit of the target) per row with vocabulary chunks of `ch` (full2.py:753-790)."""
    hb, wb = h.to(mm_dtype), w.to(mm_dtype)
    parts = []
    for c0 in range(0, w.shape[0], ch):
        lo = (hb @ wb[c0:c0 + ch].T).float()
        if bias is not None:
            lo = lo + bias[c0:c0 + ch].float()
        parts.append(torch.logsumexp(lo, -1))
    lse = torch.logsumexp(torch.stack(parts, -1), -1)
    ly = (hb.float() * wb[y].float()).sum(-1)
    if bias is not None:
        ly = ly + bias[y].float()
    return lse, ly


# ----------------------------------------------------------------------------------------------- anchors
def select_anchors(s, tau, A):
    """Causal anchor choice (full2.py:1668-1676).

    s (B,T) surprise; anchor = s > tau; keep the first A anchors of each text; idx (B,A) = kept positions in
    text order followed by the remaining positions in order; valid (B,A) marks real anchors.
    """
    B, T = s.shape
    anchor = s > tau
    keep = anchor & (anchor.cumsum(1) <= A)
    pos = torch.arange(T, device=s.device)
    idx = ((~keep).long() * T + pos).argsort(dim=-1, stable=True)[:, :A]
    valid = keep.gather(1, idx)
    return idx, valid


def tau_quantile(s, frac, limit=100_000):
    return torch.quantile(s[:, 1:].reshape(-1)[:limit].float(), 1 - frac)


# ----------------------------------------------------------------------------------------------- locks / phrases
def find_locks(x, vocab, n_keys=3, lock_bucket=None):
    """Keys and locks (full2.py:1499-1535): for every position the last earlier occurrence of the same 1-, 2- and
    3-gram ending here; the candidate is the token that followed it.  Only the longest firing lock stays on.

    Returns cand (B,T,n) int64, on (B,T,n) bool, bucket (B,T) int64, src (B,T,n) int64.
    """
    B, T = x.shape
    V = vocab
    pos = torch.arange(T, device=x.device).expand(B, T)
    prev = torch.cat([torch.full_like(x[:, :1], V), x[:, :-1]], 1)
    keys = [x, prev * (V + 1) + x]
    if n_keys >= 3:
        prev2 = torch.cat([torch.full_like(x[:, :2], V), x[:, :-2]], 1)
        keys.append((prev2 * (V + 1) + prev) * (V + 1) + x)
    cands, ons, srcs = [], [], []
    for key in keys:
        order = key.argsort(dim=1, stable=True)
        ks, ps = key.gather(1, order), pos.gather(1, order)
        same = torch.cat([torch.zeros_like(ks[:, :1], dtype=torch.bool), ks[:, 1:] == ks[:, :-1]], 1)
        lastp = torch.cat([torch.full_like(ps[:, :1], -1), ps[:, :-1]], 1)
        last = torch.full_like(x, -1).scatter(1, ps, torch.where(same, lastp, torch.full_like(lastp, -1)))
        ok = last >= 0
        src = (last + 1).clamp(max=T - 1)
        cand = x.gather(1, src)
        cands.append(torch.where(ok, cand, torch.zeros_like(cand)))
        srcs.append(torch.where(ok, src, torch.zeros_like(src)))
        ons.append(ok)
    if lock_bucket is not None:
        for k in range(len(ons) - 1):
            ons[k] = ons[k] & ~torch.stack(ons[k + 1:], 0).any(0)
        bk = lock_bucket[x.clamp(max=lock_bucket.numel() - 1)]
    else:
        bk = torch.zeros_like(x)
    return torch.stack(cands, -1), torch.stack(ons, -1), bk, torch.stack(srcs, -1)


def phrase_index(x, keys, phr_v):
    """Row of the (previous, current) pair in the sorted phrase-table keys; K = absent (full2.py:1441-1450)."""
    ctx = torch.cat([torch.full_like(x[:, :1], -1), x[:, :-1]], 1) * phr_v + x
    K = keys.numel()
    p = torch.searchsorted(keys, ctx).clamp(max=K - 1)
    return torch.where(keys[p] == ctx, p, torch.full_like(p, K))


# ----------------------------------------------------------------------------------------------- MoE routing
def moe_route(xf, router_w, real, k_tok, k_max, E):
    """Router softmax, top-k_max, per-token budget mask, renormalised weights, Switch aux loss (full2.py:497-530)."""
    logits = (xf.to(router_w.dtype) @ router_w.T).float()
    probs = logits.softmax(-1)
    top_p, top_e = probs.topk(k_max, -1)
    keep = torch.arange(k_max, device=xf.device)[None] < k_tok[:, None]
    w = (top_p * keep) / (top_p * keep).sum(-1, keepdim=True).clamp(min=1e-9)
    e_flat = top_e.masked_fill(~keep, E)
    cnt = torch.zeros(E + 1, device=xf.device, dtype=torch.float32).index_add_(
        0, e_flat.reshape(-1), torch.ones(e_flat.numel(), device=xf.device))[:E]
    pm = (probs * real[:, None]).sum(0) / real.sum().clamp(min=1)
    aux = E * (cnt / cnt.sum().clamp(min=1) * pm).sum()
    return probs, top_e, keep, w, e_flat, aux


def moe_slots(e_flat, w, E, C):
    """Capacity slotting in arrival order (full2.py:532-564).

    e_flat (N,k) expert of each (token, choice) with E = nowhere.  A choice takes the next free place of its expert
    in (token, choice) order; choices beyond C places are dropped.
    Returns table (E*C,) slot -> token (N = empty), wtab (E*C,) slot weight, flat_idx (N,k) choice -> slot
    (E*C = dropped), dropped fraction.
    """
    N, k = e_flat.shape
    oh = F.one_hot(e_flat, E + 1)[..., :E]
    rank = (oh.reshape(-1, E).cumsum(0) - 1).view_as(oh)
    place = oh.bool() & (rank < C)
    kept = (e_flat < E).sum().clamp(min=1)
    dropped = 1 - place.sum() / kept
    slot = (torch.arange(E, device=e_flat.device) * C)[None, None] + rank
    flat_idx = torch.where(place, slot, torch.full_like(slot, E * C)).amin(-1)
    tok = torch.arange(N, device=e_flat.device)[:, None].expand(-1, k)
    ok = flat_idx < E * C
    table = torch.full((E * C + 1,), N, device=e_flat.device, dtype=torch.long)
    table = table.scatter(0, flat_idx.reshape(-1), torch.where(ok, tok, torch.full_like(tok, N)).reshape(-1))[:-1]
    wtab = torch.zeros(E * C + 1, device=e_flat.device, dtype=w.dtype)
    wtab = wtab.scatter(0, flat_idx.reshape(-1), (w * ok).reshape(-1))[:-1]
    return table, wtab, flat_idx, dropped


def expert_ffn(x, up, down, act):
    """x (E,C,d) @ up (E,d,H) -> act -> @ down (E,H',d)."""
    h = torch.bmm(x, up.to(x.dtype))
    h = relu2(h) if act == "relu2" else swiglu(h)
    return torch.bmm(h, down.to(x.dtype))


# ----------------------------------------------------------------------------------------------- Instinct update
def _rms(x, dim):
    return x.pow(2).mean(dim, keepdim=True).sqrt()


def instinct_direction(mf, grad, kind, cs=None):
    """Normalised update direction of the Instinct optimizer for one weight (exp_opt.py:239-284).

    kind: vocab | row3 | hsn<n>[e] | hs | hs3 | row | tensor.  `cs` = last step's second-axis mean squares
    (one-pass lagged homeostasis); returns (upd, new_cs).
    """
    eps = 1e-8
    new_cs = None
    if kind == "vocab":
        upd = torch.where(grad.abs().sum(1, keepdim=True) > 0, mf / (_rms(mf, 1) + eps), torch.zeros_like(mf))
    elif kind == "row3":
        upd = mf / (_rms(mf, 1) + eps)
    elif kind.startswith("hsn"):
        n = int(kind[3:-1]) if kind.endswith("e") else int(kind[3:])
        ro, co = (1, 2) if kind.endswith("e") else (1, 0)
        upd = mf / (_rms(mf, ro) + eps)
        for _ in range(n):
            upd = upd / (_rms(upd, co) + eps)
            upd = upd / (_rms(upd, ro) + eps)
    elif kind in ("hs", "hs3"):
        ro, co = (1, 0) if kind == "hs" else (1, 2)
        upd = mf / (_rms(mf, ro) + eps)
        now = upd.pow(2).mean(co, keepdim=True)
        if cs is not None:
            col = torch.where(cs > 0, cs, now)
            new_cs = now
        else:
            col = now
        upd = upd / (col.sqrt() + eps)
        upd = upd / (_rms(upd, ro) + eps)
    elif kind == "row":
        upd = mf / (mf.pow(2).flatten(1).mean(1).sqrt().view(-1, *[1] * (mf.dim() - 1)) + eps)
    else:
        upd = mf / (mf.pow(2).mean().sqrt() + eps)
    return upd, new_cs


def sr_bf16(x, rand16):
    """fp32 -> bf16 stochastic rounding: add a 16-bit random integer below the kept bits, truncate
    (exp_opt.py:189-194).  `rand16` int32 in [0, 65536)."""
    xi = x.contiguous().view(torch.int32)
    return ((xi + rand16) & -65536).view(torch.float32).to(torch.bfloat16)


def lowbias32(x):
    """32-bit integer hash used for counter-based stochastic rounding; x int64 tensor holding uint32 values."""
    m = 0xFFFFFFFF
    x = x & m
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & m
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & m
    x = x ^ (x >> 16)
    return x


def sr_counter(numel, seed, device):
    """Two 16-bit random fields per element from hash(index ^ seed·0x9E3779B9): low for m, high for w."""
    idx = torch.arange(numel, device=device, dtype=torch.int64)
    h = lowbias32(idx ^ ((seed * 0x9E3779B9) & 0xFFFFFFFF))
    return (h & 0xFFFF).to(torch.int32), (h >> 16).to(torch.int32)
