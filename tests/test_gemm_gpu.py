"""tcgen05 GEMM against a plain fp32 PyTorch matmul: every operand-major combination, ragged shapes, grouped launch
and each fused epilogue."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ext():
    from memarch_b200.ops import _ext
    return _ext.C()


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _mk(shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).bfloat16()


SHAPES = [(128, 256, 64), (256, 512, 256), (384, 768, 1024), (2049, 2048, 2048), (136, 264, 200), (4096, 50304, 128),
          (512, 2064, 256), (264, 2072, 128), (136, 2200, 64)]     # ragged last N tile of 16, 24 and 152 columns


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_matches_fp32(M, N, K, a_mn, b_mn):
    """Single-CTA kernel (the pair kernel has its own test below)."""
    from memarch_b200.ops import gemm
    C = _ext()
    C.gemm_set_pair(False)
    if a_mn and M % 8:
        pytest.skip("an MN-major operand is stored (K, M): its row pitch M*2 bytes must be a multiple of 16")
    A = _mk((M, K), seed=1)
    B = _mk((N, K), seed=2)
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    try:
        out = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
        torch.cuda.synchronize()
    finally:
        C.gemm_set_pair(True)
    assert C.gemm_status(0) == 0
    ref = A.float() @ B.float().t()
    assert _rel(out, ref) < 1e-2, (_rel(out, ref), out[:2, :4], ref[:2, :4])


def test_gemm_fp32_accumulate():
    from memarch_b200.ops import gemm
    A, B = _mk((512, 320), seed=3), _mk((256, 320), seed=4)
    out = torch.ones(512, 256, device="cuda")
    gemm(A, B, out=out, out_dtype=torch.float32, accumulate=True)
    gemm(A, B, out=out, out_dtype=torch.float32, accumulate=True)
    ref = 1 + 2 * (A.float() @ B.float().t())
    assert _rel(out, ref) < 2e-3


def test_gemm_grouped_and_strided_views():
    from memarch_b200.ops import gemm
    E, Cn, d, H = 4, 200, 256, 384
    x, up = _mk((E, Cn, d), seed=5), _mk((E, d, H), 0.1, seed=6)
    y = gemm(x, up, b_mn=True, groups=E)
    ref = torch.bmm(x.float(), up.float())
    assert _rel(y, ref) < 1e-2
    big = _mk((1000, 512), seed=7)
    w = _mk((256, 512), seed=8)
    out = torch.zeros(1000, 256, device="cuda", dtype=torch.bfloat16)
    gemm(big[128:640], w, out=out[128:640])
    assert _rel(out[128:640], big[128:640].float() @ w.float().t()) < 1e-2
    assert out[:128].abs().sum() == 0 and out[640:].abs().sum() == 0


def test_gemm_epilogues():
    from memarch_b200.ops import gemm
    M, N, K = 300, 512, 256
    A, B = _mk((M, K), seed=9), _mk((N, K), 0.1, seed=10)
    acc = A.float() @ B.float().t()
    h = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    a = torch.empty_like(h)
    gemm(A, B, out=h, out2=a, epi=1)
    assert _rel(a, acc) < 1e-2
    assert _rel(h, torch.relu(a.float()) ** 2) < 1e-2
    da = gemm(A, B, epi=2, aux=a)
    assert _rel(da, acc * 2 * torch.relu(a.float())) < 1e-2
    sc = torch.rand(M, device="cuda")
    ys = gemm(A, B, epi=4, aux=sc)
    assert _rel(ys, acc * sc[:, None]) < 1e-2
    H = N // 2
    hs = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    gu = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    gemm(A, B, out=hs, out2=gu, epi=3)
    assert _rel(gu, acc) < 1e-2
    g, u = gu.float().chunk(2, -1)
    assert _rel(hs, torch.nn.functional.silu(g) * u) < 1e-2


def test_linear_autograd_matches_torch():
    from memarch_b200.ops import basic
    x = _mk((512, 256), seed=11).requires_grad_()
    w = _mk((384, 256), 0.1, seed=12).requires_grad_()
    y = basic._Linear.apply(x, w)
    go = _mk((512, 384), seed=13)
    y.backward(go)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    (xr @ wr.t()).backward(go.float())
    assert _rel(y, xr @ wr.t()) < 1e-2
    assert _rel(x.grad, xr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 512, 256), (2049, 2048, 2048), (4096, 50304, 128), (264, 264, 200),
                                   (512, 2064, 256), (264, 2072, 128), (520, 2200, 64)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_pair_kernel_matches_fp32(M, N, K, a_mn, b_mn):
    """cta_group::2 kernel (two SMs per 256x256 tile) on the same checks as the single-CTA kernel."""
    from memarch_b200.ops import gemm
    C = _ext()
    if a_mn and M % 8:
        pytest.skip("MN-major A needs M % 8 == 0")
    A, B = _mk((M, K), seed=21), _mk((N, K), seed=22)
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    C.gemm_set_pair(True)
    try:
        out = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
        torch.cuda.synchronize()
        st = C.gemm_status(0)
    finally:
        C.gemm_set_pair(True)
    assert st == 0
    assert _rel(out, A.float() @ B.float().t()) < 1e-2


def test_pair_kernel_grouped_epilogues():
    from memarch_b200.ops import gemm
    C = _ext()
    E, Cn, d, H = 3, 600, 256, 512
    x, up = _mk((E, Cn, d), seed=23), _mk((E, d, H), 0.1, seed=24)
    C.gemm_set_pair(True)
    try:
        h = torch.empty(E, Cn, H, device="cuda", dtype=torch.bfloat16)
        a = torch.empty_like(h)
        gemm(x, up, b_mn=True, out=h, out2=a, epi=1, groups=E)
        hs = torch.empty(E, Cn, H // 2, device="cuda", dtype=torch.bfloat16)
        gu = torch.empty_like(h)
        gemm(x, up, b_mn=True, out=hs, out2=gu, epi=3, groups=E)
        torch.cuda.synchronize()
        st = C.gemm_status(0)
    finally:
        C.gemm_set_pair(True)
    assert st == 0
    acc = torch.bmm(x.float(), up.float())
    assert _rel(a, acc) < 1e-2 and _rel(h, torch.relu(a.float()) ** 2) < 1e-2
    assert _rel(gu, acc) < 1e-2
    g, u = gu.float().chunk(2, -1)
    assert _rel(hs, torch.nn.functional.silu(g) * u) < 1e-2


def test_gemm_is_deterministic_and_leaves_the_status_clean():
    """Same inputs, two launches of each kernel variant: identical bits (a race between roles would show as a
    difference), status word still zero."""
    from memarch_b200.ops import gemm
    C = _ext()
    A, B = _mk((1024, 512), seed=31), _mk((768, 512), seed=32)
    for pair in (False, True):
        C.gemm_set_pair(pair)
        try:
            o1 = gemm(A, B).clone()
            o2 = gemm(A, B).clone()
            e1 = gemm(A.view(2, 512, 512), B.view(2, 384, 512).transpose(1, 2).contiguous(), b_mn=True, epi=1,
                      out=torch.empty(2, 512, 384, device="cuda", dtype=torch.bfloat16),
                      out2=torch.empty(2, 512, 384, device="cuda", dtype=torch.bfloat16), groups=2).clone()
            e2 = gemm(A.view(2, 512, 512), B.view(2, 384, 512).transpose(1, 2).contiguous(), b_mn=True, epi=1,
                      out=torch.empty(2, 512, 384, device="cuda", dtype=torch.bfloat16),
                      out2=torch.empty(2, 512, 384, device="cuda", dtype=torch.bfloat16), groups=2).clone()
            torch.cuda.synchronize()
        finally:
            C.gemm_set_pair(True)
        assert torch.equal(o1, o2) and torch.equal(e1, e2)
        assert C.gemm_status(0) == 0
