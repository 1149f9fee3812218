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
    from memarch_b200.ops import _ext as ext
    f0 = ext.gemm_flops
    y = gemm(x, up, b_mn=True, groups=E)
    assert ext.gemm_flops - f0 == 2 * Cn * H * d * E                        # the work counter behind bench.py's GEMM share
    ref = torch.bmm(x.float(), up.float())
    assert _rel(y, ref) < 1e-2
    big = _mk((1000, 512), seed=7)
    w = _mk((256, 512), seed=8)
    out = torch.zeros(1000, 256, device="cuda", dtype=torch.bfloat16)
    f0 = ext.gemm_flops
    gemm(big[128:640], w, out=out[128:640])
    assert ext.gemm_flops - f0 == 2 * 512 * 256 * 512
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


# ------------------------------------------------------------------------------------------------ pair kernel, staged epilogue
def _epilogue_suite(direct, tall=False):
    """Every epilogue of the CTA-pair kernel on ragged shapes, through TMA stores or through the coalesced row stores
    (`direct`: the path peer buffers and segmented outputs take); `tall`: the 512-row tile variant."""
    from memarch_b200.ops import gemm
    C = _ext()
    C.gemm_set_debug((8 if direct else 0) | (64 if tall else 32))
    try:
        M, N, K = (1100 if tall else 600), 720, 320              # ragged M (row tiles of 256 / 512) and N (720 = 2*256 + 208)
        A, B = _mk((M, K), seed=41), _mk((N, K), 0.1, seed=42)
        acc = A.float() @ B.float().t()
        assert _rel(gemm(A, B), acc) < 1e-2
        h = torch.full((M, N), 7.0, device="cuda", dtype=torch.bfloat16)
        a = torch.full((M, N), 7.0, device="cuda", dtype=torch.bfloat16)
        gemm(A, B, out=h, out2=a, epi=1)
        assert _rel(a, acc) < 1e-2 and _rel(h, torch.relu(a.float()) ** 2) < 1e-2
        assert _rel(gemm(A, B, epi=2, aux=a), acc * 2 * torch.relu(a.float())) < 1e-2
        sc = torch.rand(M, device="cuda")
        assert _rel(gemm(A, B, epi=4, aux=sc), acc * sc[:, None]) < 1e-2
        f = torch.ones(M, N, device="cuda")
        gemm(A, B, out=f, out_dtype=torch.float32, accumulate=True)
        gemm(A, B, out=f, out_dtype=torch.float32, accumulate=True)
        assert _rel(f, 1 + 2 * acc) < 2e-3
        assert _rel(gemm(A, B, out_dtype=torch.float32), acc) < 2e-3
        # SwiGLU over column halves with and without the pre-activation copy; H = 360 is ragged too
        H = N // 2
        hs = torch.empty(M, H + 8, device="cuda", dtype=torch.bfloat16)[:, :H]       # a strided view (pitch 368)
        gu = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        gemm(A, B, out=hs, out2=gu, epi=3)
        assert _rel(gu, acc) < 1e-2
        g, u = gu.float().chunk(2, -1)
        assert _rel(hs, torch.nn.functional.silu(g) * u) < 1e-2
        hs2 = gemm(A, B, epi=3)
        assert _rel(hs2, hs) < 1e-3
        # a view into a larger output: rows and columns around it stay untouched
        big = torch.zeros(M + 64, N + 64, device="cuda", dtype=torch.bfloat16)
        gemm(A, B, out=big[32:32 + M, 64:64 + N])
        assert _rel(big[32:32 + M, 64:64 + N], acc) < 1e-2
        assert big[:32].abs().sum() == 0 and big[32 + M:].abs().sum() == 0
        assert big[:, :64].abs().sum() == 0 and big[:, 64 + N:].abs().sum() == 0
        torch.cuda.synchronize()
        assert C.gemm_status(0) == 0
    finally:
        C.gemm_set_debug(0)


def test_pair_staged_epilogue_tma_stores():
    _epilogue_suite(False)


def test_pair_staged_epilogue_direct_stores():
    _epilogue_suite(True)


@pytest.mark.parametrize("direct", [False, True])
def test_pair_tall_tiles(direct):
    """512-row tiles (two MMA row blocks per B tile, single-buffered accumulators) on the same suite."""
    _epilogue_suite(direct, tall=True)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_pair_tall_tiles_operand_layouts(a_mn, b_mn):
    from memarch_b200.ops import gemm
    C = _ext()
    M, N, K = 1536, 520, 1088
    A, B = _mk((M, K), seed=81), _mk((N, K), 0.1, seed=82)
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    C.gemm_set_debug(64)
    try:
        o1 = gemm(a, b, a_mn=a_mn, b_mn=b_mn).clone()
        o2 = gemm(a, b, a_mn=a_mn, b_mn=b_mn).clone()
        torch.cuda.synchronize()
        st = C.gemm_status(0)
    finally:
        C.gemm_set_debug(0)
    assert st == 0 and torch.equal(o1, o2)
    assert _rel(o1, A.float() @ B.float().t()) < 1e-2


@pytest.mark.parametrize("direct", [False, True])
def test_pair_group_extents(direct):
    """Per-group extents: padded rows are not computed (count_mode 1), padded contraction positions are not read
    (count_mode 2); results equal the full computation on zero-padded operands."""
    from memarch_b200.ops import gemm
    C = _ext()
    C.gemm_set_debug(8 if direct else 0)
    try:
        E, Cn, d, H = 4, 777, 256, 384
        cnt = torch.tensor([0, 300, 512, 777], device="cuda", dtype=torch.int32)
        x = _mk((E, Cn, d), seed=51)
        mask = (torch.arange(Cn, device="cuda")[None] < cnt[:, None])
        x = x * mask[..., None]
        up = _mk((E, d, H), 0.1, seed=52)
        ref = torch.bmm(x.float(), up.float())
        h = torch.full((E, Cn, H), 3.0, device="cuda", dtype=torch.bfloat16)
        a = torch.full((E, Cn, H), 3.0, device="cuda", dtype=torch.bfloat16)
        gemm(x, up, b_mn=True, out=h, out2=a, epi=1, groups=E, counts=cnt, count_mode=1)
        assert _rel(a, ref) < 1e-2 and _rel(h, torch.relu(a.float()) ** 2) < 1e-2
        assert (a * ~mask[..., None]).abs().sum() == 0 and (h * ~mask[..., None]).abs().sum() == 0
        y = gemm(x, up, b_mn=True, groups=E, counts=cnt, count_mode=1)
        assert _rel(y, ref) < 1e-2
        # weight gradient: contraction over the rows
        dy = _mk((E, Cn, H), seed=53) * mask[..., None]
        dref = torch.bmm(x.float().transpose(1, 2), dy.float())
        dw = gemm(x, dy, a_mn=True, b_mn=True, groups=E, counts=cnt, count_mode=2)
        assert _rel(dw, dref) < 1e-2
        assert dw[0].abs().sum() == 0
        dwf = torch.ones(E, d, H, device="cuda")
        gemm(x, dy, a_mn=True, b_mn=True, groups=E, counts=cnt, count_mode=2, out=dwf, out_dtype=torch.float32,
             accumulate=True)
        assert _rel(dwf, 1 + dref) < 2e-3
        torch.cuda.synchronize()
        assert C.gemm_status(0) == 0
    finally:
        C.gemm_set_debug(0)


@pytest.mark.parametrize("act", ["swiglu", "relu2"])
def test_linear_act_autograd_matches_fp32(act):
    """Linear with the activation in the GEMM epilogue against plain fp32 autograd."""
    from memarch_b200.ops import basic
    x = _mk((640, 256), seed=61).requires_grad_()
    w = _mk((768, 256), 0.1, seed=62).requires_grad_()
    h = basic.linear_act(x, w, act)
    go = _mk(tuple(h.shape), seed=63)
    h.backward(go)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    pre = xr @ wr.t()
    if act == "swiglu":
        g, u = pre.chunk(2, -1)
        hr = torch.nn.functional.silu(g) * u
    else:
        hr = torch.relu(pre) ** 2
    hr.backward(go.float())
    assert _rel(h, hr) < 2e-2
    assert _rel(x.grad, xr.grad) < 2e-2 and _rel(w.grad, wr.grad) < 2e-2


@pytest.mark.parametrize("act", ["swiglu", "relu2"])
def test_expert_ffn_with_counts_equals_padded(act):
    """Expert FFN forward + backward with per-expert fill counts equals the padded computation."""
    from memarch_b200 import ops
    E, Cn, d, H = 4, 520, 256, 512
    cnt = torch.tensor([520, 0, 130, 300], device="cuda", dtype=torch.int32)
    mask = (torch.arange(Cn, device="cuda")[None] < cnt[:, None])[..., None]
    x0 = _mk((E, Cn, d), seed=71) * mask
    up0, down0 = _mk((E, d, 2 * H if act == "swiglu" else H), 0.1, seed=72), _mk((E, H, d), 0.1, seed=73)
    go = _mk((E, Cn, d), seed=74) * mask
    res = []
    for counts in (None, cnt):
        x, up, down = (t.clone().requires_grad_() for t in (x0, up0, down0))
        y = ops.expert_ffn(x, up, down, act, counts=counts)
        y.backward(go)
        res.append((y, x.grad, up.grad, down.grad))
    for a, b in zip(*res):
        assert _rel(b, a) < 1e-3, (_rel(b, a))
    assert _ext().gemm_status(0) == 0


@pytest.mark.parametrize("act,fuse", [("swiglu", False), ("swiglu", True), ("relu2", True)])
def test_ffn_node_matches_fp32(act, fuse, monkeypatch):
    """Feed-forward half of a light block as one autograd node (activation backward in the dgrad GEMM's epilogue,
    ragged hidden width) against fp32 autograd."""
    from memarch_b200.ops import basic
    monkeypatch.setattr(basic, "FUSE_DSWIGLU", fuse)
    M, d, H = 520, 256, 328
    x = _mk((M, d), seed=91).requires_grad_()
    wu = _mk(((2 * H if act == "swiglu" else H), d), 0.1, seed=92).requires_grad_()
    wd = _mk((d, H), 0.1, seed=93).requires_grad_()
    y = basic.ffn(x, wu, wd, act)
    go = _mk((M, d), seed=94)
    y.backward(go)
    xr, ur, dr = (t.detach().float().requires_grad_() for t in (x, wu, wd))
    pre = xr @ ur.t()
    if act == "swiglu":
        g, u = pre.chunk(2, -1)
        hr = torch.nn.functional.silu(g) * u
    else:
        hr = torch.relu(pre) ** 2
    (hr @ dr.t()).backward(go.float())
    assert _rel(y, hr @ dr.t()) < 2e-2
    for a, b in ((x.grad, xr.grad), (wu.grad, ur.grad), (wd.grad, dr.grad)):
        assert _rel(a, b) < 2e-2, _rel(a, b)
    assert _ext().gemm_status(0) == 0


# ------------------------------------------------------------------------------------------------ int8 tensor cores
@pytest.mark.parametrize("G,M,N,K", [(1, 128, 256, 128), (1, 300, 520, 272), (1, 2049, 2048, 2048), (3, 200, 384, 256),
                                      (1, 40, 72, 48)])
def test_int8_gemm_is_exact(G, M, N, K):
    """kind::i8 GEMM: integer products are exact, so the fp32 output equals (a · bᵀ in int64) x row scale x column
    scale to fp32 rounding; ragged M / N / K tails and grouped launch included."""
    C = _ext()
    g = torch.Generator(device="cuda").manual_seed(G * 1000 + M)
    shp = (lambda *s: s) if G == 1 else (lambda *s: (G, *s))
    a = torch.randint(-127, 128, shp(M, K), device="cuda", generator=g, dtype=torch.int8)
    b = torch.randint(-127, 128, shp(N, K), device="cuda", generator=g, dtype=torch.int8)
    sa = torch.rand(shp(M), device="cuda", generator=g) + 0.5
    sb = torch.rand(shp(N), device="cuda", generator=g) + 0.5
    out = C.gemm_i8(a, b, sa, sb, True)
    torch.cuda.synchronize()
    assert C.gemm_status(0) == 0
    ref = (a.double() @ b.double().transpose(-1, -2)) * sa.double()[..., :, None] * sb.double()[..., None, :]
    assert (out.double() - ref).abs().max() <= 1e-6 * ref.abs().max()
    o16 = C.gemm_i8(a, b, sa, sb, False)
    assert o16.dtype == torch.bfloat16 and _rel(o16, ref) < 4e-3


def test_int8_row_quantiser_and_linear():
    from memarch_b200.ops import int8
    C = _ext()
    x = _mk((300, 272), seed=71)
    q, s = C.quant_rows_i8(x)
    qr, sr = int8.fq(x, 1)
    assert torch.equal(q.float(), qr.float()) and torch.allclose(s, sr.squeeze(1), rtol=1e-6)
    # linear through the int8 tensor cores against the floating-point statement of the same quantised product
    w = _mk((520, 272), 0.1, seed=72)
    y = int8.quant_mm(x, w, torch.float32)
    qw, sw = int8.fq(w, 1)
    ref = (qr.float() @ qw.float().t()) * sr * sw.t()
    assert _rel(y, ref) < 1e-5
    xg = x.clone().requires_grad_()
    wg = w.clone().requires_grad_()
    go = _mk((300, 520), seed=73)
    int8.linear_i8(xg, wg).backward(go)
    xr, wr = x.float().requires_grad_(), w.float().requires_grad_()
    (xr @ wr.t()).backward(go.float())
    assert _rel(xg.grad, xr.grad) < 3e-2 and _rel(wg.grad, wr.grad) < 2e-2          # int8 quantisation error
    assert C.gemm_status(0) == 0


@pytest.mark.parametrize("act", ["relu2", "swiglu"])
def test_frozen_int8_bank_on_tensor_cores(act, monkeypatch):
    """Bank layer with int8 storage: the tensor-core int8 forward against the dequantised bf16 path of the same
    weights (difference = quantisation of the activations), input gradient included."""
    from memarch_b200.models.moe import AnchorMoE
    torch.manual_seed(0)
    moe = AnchorMoE(256, E=4, k_avg=2, k_max=2, bank=True, act=act, w_dtype=torch.bfloat16, bank_q="int8").cuda()
    moe.rebank([True, True, False, False])                       # experts 0, 1 move into the int8 bank
    assert moe.up_f.dtype == torch.int8 and moe.up_f.shape[0] == 2
    xe = (torch.randn(2, 300, 256, device="cuda") * 0.5).bfloat16()
    go = torch.randn(2, 300, 256, device="cuda").bfloat16()
    res = []
    for on in ("1", "0"):
        monkeypatch.setenv("MEMARCH_BANK_I8", on)
        x = xe.clone().requires_grad_()
        y = moe._ffn_frozen(x)
        y.backward(go)
        res.append((y.detach().float(), x.grad.float()))
    assert _rel(res[0][0], res[1][0]) < 3e-2, _rel(res[0][0], res[1][0])
    assert _rel(res[0][1], res[1][1]) < 3e-2, _rel(res[0][1], res[1][1])
    assert not torch.equal(res[0][0], res[1][0])                 # the int8 path did run
    assert _ext().gemm_status(0) == 0
