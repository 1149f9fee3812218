"""Re-reading kernels (`csrc/reread.cu`) against the module's PyTorch statement in fp32: picks, output, cost and the
gradient of every input and weight."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(B, S, C, L, d, T, n_texts, seed, some_empty=True, table_dtype=torch.float32):
    g = torch.Generator(device="cuda").manual_seed(seed)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    h = rn(B, S, d)
    faces = rn(B, C, L, 64)
    contents = rn(B, C, d)
    valid = torch.rand(B, C, device="cuda", generator=g) > (0.3 if some_empty else -1.0)
    if some_empty:
        valid[0] = False                                   # a text with an empty memory
        valid[1, 3:] = False                               # fewer real cards than picks
    pos = torch.randint(0, T, (B, C), device="cuda", generator=g)
    qpos = torch.randint(0, T, (B, S), device="cuda", generator=g)
    rows = torch.randint(0, n_texts, (B,), device="cuda", generator=g)
    ids = torch.randint(0, 500, (n_texts, T), device="cuda", generator=g)
    table = (rn(500, 128) * 0.5).to(table_dtype)
    return h, ids, table, faces, contents, pos, valid, qpos, rows


def _run(mod, args, fused, monkeypatch):
    from memarch_b200.ops import _ext
    h, ids, table, faces, contents, pos, valid, qpos, rows = args
    leaves = [t.detach().clone().requires_grad_() for t in (h, table, faces, contents)]
    for p in mod.parameters():
        p.grad = None
    monkeypatch.setattr(_ext, "use_cuda", (lambda t: t.is_cuda) if fused else (lambda t: False))
    o, cost = mod(leaves[0], ids, leaves[1], leaves[2], leaves[3], pos, valid, qpos, rows)
    g = torch.Generator(device="cuda").manual_seed(5)
    go = torch.randn(o.shape, device="cuda", generator=g)
    ((o * go).sum() + 3.0 * cost).backward()
    grads = {"h": leaves[0].grad, "table": leaves[1].grad, "faces": leaves[2].grad, "contents": leaves[3].grad}
    grads.update({n: p.grad.clone() for n, p in mod.named_parameters() if p.grad is not None})
    return o.detach(), cost.detach(), grads


@pytest.mark.parametrize("B,S,C,L,T,table_dtype", [(3, 37, 20, 2, 64, torch.float32), (4, 64, 320, 2, 512, torch.float32),
                                                   (2, 16, 3, 1, 32, torch.float32), (3, 40, 48, 3, 128, torch.bfloat16)])
def test_reread_kernels_match_pytorch(B, S, C, L, T, table_dtype, monkeypatch):
    from memarch_b200.models.reread import Reread
    torch.manual_seed(0)
    d = 96
    mod = Reread(d).cuda()
    with torch.no_grad():                                  # gates away from their neutral start, so every path carries signal
        mod.halt_v.weight.mul_(8)
        mod.halt_h.weight.mul_(4)
        mod.offset.mul_(10)
    args = _case(B, S, C, L, d, T, 5, seed=B * 100 + C, table_dtype=table_dtype)
    o_ref, c_ref, g_ref = _run(mod, args, False, monkeypatch)
    o, c, g = _run(mod, args, True, monkeypatch)
    rel = lambda a, b: float((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-9))
    assert rel(o, o_ref) < 1e-4, rel(o, o_ref)
    assert abs(float(c) - float(c_ref)) < 1e-4 * max(1.0, abs(float(c_ref)))
    assert set(g) == set(g_ref)
    tol = 2e-2 if table_dtype == torch.bfloat16 else 2e-4
    for name in g_ref:
        if g_ref[name].float().norm() == 0:
            assert g[name].float().norm() == 0, name
        else:
            assert rel(g[name], g_ref[name]) < tol, (name, rel(g[name], g_ref[name]))


def test_reread_picks_are_the_topk():
    """The kernel's card choice equals torch.topk on the same scores (discrete decision, exact)."""
    from memarch_b200.ops import _ext
    C_ = _ext.C()
    g = torch.Generator(device="cuda").manual_seed(3)
    B, S, C, k, T = 2, 50, 300, 4, 256
    sc = torch.randn(B, S, C, device="cuda", generator=g)
    sc[:, :, ::7] = -1e4
    z = lambda *s: torch.zeros(*s, device="cuda")
    pos = torch.randint(0, T, (B, C), device="cuda", generator=g)
    qpos = torch.randint(0, T, (B, S), device="cuda", generator=g)
    out = C_.reread_fwd(sc, pos, qpos, torch.arange(B, device="cuda"), torch.randint(0, 50, (B, T), device="cuda", generator=g),
                        torch.randn(50, 128, device="cuda", generator=g), z(4, 128), z(128), z(1), z(B, S), z(64, 128) + 0.01,
                        torch.randn(B, C, 64, device="cuda", generator=g), k)
    top_j, p = out[2], out[3]
    ref_s, ref_j = sc.topk(k, -1)
    assert torch.equal(top_j.long(), ref_j)
    assert torch.allclose(p, torch.softmax(ref_s, -1), atol=1e-6)
