"""Anchor routing on a B200: the top-k kernel against the PyTorch statement on the same scores, the tensor-core scores
against a plain batched product, and the whole bf16 search against the CPU."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda", 0)


def _torch_choice(S, lval, lp, avalid, nx, H, K, q0, scale):
    G, M, _ = S.shape
    B, A, L = lval.shape
    b = torch.arange(G, device=S.device) // H
    s = (S.view(G, M, A, L) * scale).masked_fill(~lval[b][:, None], -float("inf"))
    s_a, best_l = s.max(-1)
    qi = q0 + torch.arange(M, device=S.device)
    ok = avalid[b][:, None, :] & (nx[b][:, None, :] <= qi[None, :, None])
    s_a = s_a.masked_fill(~ok, -float("inf"))
    top_v, top_i = s_a.topk(K, -1)
    val = top_v > -float("inf")
    pos = lp[b][:, None].expand(G, M, A, L).gather(-1, best_l[..., None]).squeeze(-1).gather(-1, top_i)
    zero = torch.zeros_like(top_i)
    return torch.where(val, top_i, zero), val, torch.where(val, pos, zero)


@pytest.mark.parametrize("B,H,M,A,L,K", [(2, 2, 64, 50, 3, 4), (1, 3, 40, 200, 8, 8), (2, 1, 17, 9, 2, 8), (1, 1, 256, 1024, 8, 4)])
def test_route_topk_kernel_matches_torch(B, H, M, A, L, K):
    from memarch_b200.ops import _ext
    dev = _dev()
    g = torch.Generator(device="cuda").manual_seed(A)
    G = B * H
    S = torch.randn(G, M, A * L, device=dev, generator=g)
    lval = torch.rand(B, A, L, device=dev, generator=g) < 0.8
    lval[:, A // 2] = False                                              # an anchor without any link
    lp = torch.randint(0, 10000, (B, A, L), device=dev, generator=g)
    avalid = torch.rand(B, A, device=dev, generator=g) < 0.9
    q0 = 5
    nx = torch.randint(0, q0 + M + 10, (B, A), device=dev, generator=g)
    nx[:, :3] = 0
    want = _torch_choice(S, lval, lp, avalid, nx, H, K, q0, 0.25)
    got = _ext.C().rope_route_topk(S, lval.to(torch.uint8), lp.int(), avalid.to(torch.uint8), nx.int(), H, K, q0, 0.25)
    assert torch.equal(got[1].bool(), want[1])
    assert torch.equal(got[0], want[0]) and torch.equal(got[2], want[2])
    assert bool(want[1].any()) and (A > 20 or not bool(want[1].all()))     # the smallest case: some queries open fewer than K


def test_bf16_search_on_tensor_cores_matches_cpu():
    from memarch_b200.models import rope_memory as rm
    from memarch_b200.ops import gemm
    dev = _dev()
    torch.manual_seed(0)
    B, H, T, hd = 2, 2, 256, 64
    cfg = rm.RopeCfg(K=4, links=4, win=16, span_cap=24, chunk=128, route="exact", route_bf16=True)
    q, k = torch.randn(B, H, T, hd), torch.randn(B, H, T, hd)
    s = torch.rand(B, T) * 2
    own, apos, avalid = rm.anchors_from_surprise(s.clone(), 1.2, 64)
    want = rm.route_exact(q, k, own, apos, avalid, cfg)                  # CPU: the same bf16-rounded operands
    # the scores themselves
    kl, lval, lp = rm._links(k.to(dev), own.to(dev), apos.to(dev), avalid.to(dev), 4)
    klb = kl.to(torch.bfloat16).reshape(B * H, -1, hd).contiguous()
    qb = q.to(dev).to(torch.bfloat16).reshape(B * H, T, hd).contiguous()
    S = gemm(qb[:, :128].contiguous(), klb, groups=B * H, out_dtype=torch.float32)
    ref = torch.bmm(qb[:, :128].float(), klb.float().transpose(1, 2))
    assert (S - ref).abs().max() < 1e-3 * ref.abs().max().clamp(min=1.0)
    got = rm.route_exact(q.to(dev), k.to(dev), own.to(dev), apos.to(dev), avalid.to(dev), cfg)
    assert torch.equal(got[1].cpu(), want[1])                             # which slots are filled does not depend on rounding
    same = (got[0].cpu() == want[0]) & (got[2].cpu() == want[2])
    assert same.float().mean() > 0.99, float(same.float().mean())         # only the summation order differs


def test_tethered_model_with_the_kernel_search():
    from memarch_b200 import build
    dev = _dev()
    torch.manual_seed(0)
    env = {"NO_MEM": "1", "MOE_ACT": "relu2", "ROPE_MEM": "1", "ROPE_ROUTE": "exact", "ROPE_ROUTE_BF16": "1", "ROPE_WIN": "16",
           "ROPE_SPAN_CAP": "24", "ROPE_LINKS": "4", "ROPE_K": "2", "ROPE_CHUNK": "128"}
    m = build("tiny", 1024, env=env).to(dev).train()
    xy = torch.randint(0, 1024, (2, 129), device=dev)
    out, _ = m(xy[:, :-1])
    loss = m.train_loss(out, xy[:, 1:], True)
    loss.backward()
    assert torch.isfinite(loss) and 0 < float(m.stats["rope_share"]) < 1
    assert all(torch.isfinite(p.grad).all() for p in m.parameters() if p.grad is not None)
