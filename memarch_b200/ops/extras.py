"""Final-norm variants that keep the stream's common vector out of the head (experiment switches of the reference's
JAX port, memarch_jax/memarch_jax/prims.py:24-36 and 100-114).  Plain PyTorch: they run once per step on (B, T, d)."""
from __future__ import annotations

import torch


def dump_proof_norm(x, w, u=None, eps=1e-6):
    """RMSNorm whose output has no component along the stream's common direction:
        y = (x̂ - (x̂ · û) û) · w,   x̂ = x · rsqrt(mean(x²) + eps),   û = u / |u| without gradient.
    The denominator is taken over the full x (same scale as the ordinary norm).  `u` is a running mean of the state;
    None or an all-zero u (first step after a resume) falls back to the mean over the batch."""
    xf = x.float()
    mean_x = xf.reshape(-1, xf.shape[-1]).mean(0).detach()
    if u is None:
        u = mean_x
    else:
        u = u.detach().float()
        u = torch.where((u * u).sum() > 0, u, mean_x)
    uh = u * torch.rsqrt((u * u).sum() + 1e-30)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = y - (y @ uh)[..., None] * uh
    return (y * w.float()).to(torch.promote_types(x.dtype, w.dtype))


def cap_shared(hn, ratio, t0=256):
    """Causal cap of the common vector after the final norm.  With m_t the mean of hn over positions <= t and var_t
    the mean of |hn - m|² over the same positions, the common part is shrunk wherever |m_t| > ratio · sqrt(var_t):
        out_t = hn_t - (1 - s_t) m_t,   s_t = ratio · sqrt(var_t) / |m_t|.
    Positions before t0 and positions with s_t >= 1 come back bit for bit."""
    hf = hn.float()
    T = hf.shape[-2]
    n = torch.arange(1, T + 1, device=hn.device, dtype=torch.float32)[:, None]
    m = hf.cumsum(-2) / n
    e2 = hf.pow(2).sum(-1, keepdim=True).cumsum(-2) / n
    m2 = m.pow(2).sum(-1, keepdim=True)
    var = (e2 - m2).clamp(min=0.0)
    s = (ratio * torch.sqrt(var + 1e-6) / torch.sqrt(m2 + 1e-6)).clamp(max=1.0)     # offsets: finite slope at zero
    s = torch.where((torch.arange(T, device=hn.device) >= t0)[:, None], s, torch.ones_like(s))
    out = hf - m * (1.0 - s)
    return torch.where(s < 1.0, out, hf).to(hn.dtype)
