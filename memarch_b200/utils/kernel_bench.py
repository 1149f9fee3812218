"""Kernel micro-benchmarks with parity checks (the role of the reference's bench_fused.py:48-107).

    python -m memarch_b200.utils.kernel_bench gemm --m 8192 --n 8192 --k 8192
    python -m memarch_b200.utils.kernel_bench ce --rows 8192 --d 2064 --vocab 50304
    python -m memarch_b200.utils.kernel_bench instinct --kind hs3 --shape 8,2048,6144
    python -m memarch_b200.utils.kernel_bench experts --e 8 --c 2049 --d 2048 --h 6144
    python -m memarch_b200.utils.kernel_bench reread --rows 256 --words 128 --cards 320

Each command checks the kernel against the PyTorch fp32 statement on the same inputs, then times it with CUDA events
after warm-up (inputs larger than L2, or an L2 flush between iterations) and prints achieved TFLOP/s or GB/s next to
the measured peaks in MEASURED_PEAKS.json when that file is present.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def timeit(fn, iters=10, warm=3, flush=True):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def report(name, ms, flops=None, nbytes=None, extra=""):
    hbm, tf, src = peaks()
    s = f"{name}: {ms:.3f} ms"
    if flops:
        a = flops / ms / 1e9
        s += f"  {a:.0f} TFLOP/s = {a / tf:.2f} of {src} cuBLAS bf16 {tf:.0f}"
    if nbytes:
        a = nbytes / ms / 1e6
        s += f"  {a:.0f} GB/s = {a / hbm:.2f} of {src} copy {hbm:.0f}"
    print(s + ("  " + extra if extra else ""), flush=True)


def cmd_gemm(a):
    from memarch_b200.ops import gemm
    M, N, K, G = a.m, a.n, a.k, a.groups
    if a.i8:
        from memarch_b200.ops import _ext
        C = _ext.C()
        qa = torch.randint(-127, 128, (G, M, K), device="cuda", dtype=torch.int8)
        qb = torch.randint(-127, 128, (G, N, K), device="cuda", dtype=torch.int8)
        sa, sb = torch.rand(G, M, device="cuda") + 0.5, torch.rand(G, N, device="cuda") + 0.5
        o = C.gemm_i8(qa, qb, sa, sb, True)
        ref = (qa[:1, :256].double() @ qb[:1].double().transpose(1, 2)) * sa[:1, :256, None].double() * sb[:1, None].double()
        print(f"parity (first 256 rows) rel err {rel(o[:1, :256], ref):.2e}")
        report(f"tcgen05 int8 gemm (kind::i8, dequantising epilogue) M{M} N{N} K{K} G{G}",
               timeit(lambda: C.gemm_i8(qa, qb, sa, sb, False), a.iters, flush=not a.no_flush), 2.0 * M * N * K * G,
               extra="(integer operations; the denominator is the bf16 figure)")
        return
    A = torch.randn(G, M, K, device="cuda").bfloat16()
    B = torch.randn(G, N, K, device="cuda").bfloat16()
    Bm = B.transpose(1, 2).contiguous() if a.b_mn else B
    Am = A.transpose(1, 2).contiguous() if a.a_mn else A
    out = torch.empty(G, M, N, device="cuda", dtype=torch.bfloat16)
    run = lambda: gemm(Am, Bm, a_mn=a.a_mn, b_mn=a.b_mn, out=out, groups=G)
    run()
    ref = torch.bmm(A[:1, :256].float(), B[:1].float().transpose(1, 2))
    print(f"parity (first 256 rows) rel err {rel(out[:1, :256], ref):.2e}")
    fl = 2.0 * M * N * K * G
    report(f"tcgen05 gemm M{M} N{N} K{K} G{G} a_mn={int(a.a_mn)} b_mn={int(a.b_mn)}", timeit(run, a.iters, flush=not a.no_flush), fl)
    if not a.no_lib:
        report("library bmm (same shape)", timeit(lambda: torch.bmm(A, B.transpose(1, 2), out=out), a.iters, flush=not a.no_flush), fl)


def cmd_ce(a):
    from memarch_b200 import ops
    from memarch_b200.ops import ref
    N, d, V = a.rows, a.d, a.vocab
    h = torch.randn(N, d, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(V, d, device="cuda") * 0.02).bfloat16().requires_grad_()
    y = torch.randint(0, V, (N,), device="cuda")
    g = torch.rand(N, device="cuda") * 0.3 if a.mix else None
    hit = (torch.rand(N, device="cuda") > 0.7).float() if a.mix else None
    loss = ops.linear_ce(h, w, y, gate=g, hit=hit)
    n = min(N, 512)
    tot, gh, gw, _, _, _ = ref.linear_ce(h[:n].detach().float(), w.detach().float(), y[:n], None, g[:n] if a.mix else None,
                                         hit[:n] if a.mix else None)
    l2 = ops.linear_ce(h[:n].detach().requires_grad_(), w, y[:n], gate=g[:n] if a.mix else None, hit=hit[:n] if a.mix else None)
    print(f"parity ({n} rows) loss rel err {abs(l2.item() - tot.item()) / tot.item():.2e}")
    fl = 6.0 * N * d * V
    report(f"fused linear+CE{'+mix' if a.mix else ''} fwd (grads made in forward) N{N} d{d} V{V}",
           timeit(lambda: ops.linear_ce(h, w, y, gate=g, hit=hit), a.iters, flush=False), fl)


def cmd_instinct(a):
    from memarch_b200.config import OptConfig
    from memarch_b200.optim import Instinct
    shape = tuple(int(s) for s in a.shape.split(","))
    p = (torch.randn(*shape, device="cuda") * 0.05).to(torch.bfloat16 if a.bf16 else torch.float32).requires_grad_()
    opt = Instinct([p], OptConfig(lr=1e-3, norm="hs", scale=0.12, m_bf16=True, rel_every=1 << 30, hs_lag=a.lag))
    g = torch.randn_like(p)
    opt.prepare(torch.tensor(3.0, device="cuda"), torch.randn(64, device="cuda"))
    kind = opt.spec(p)[0]
    n = p.numel()
    per = (2 if a.bf16 else 4) * 2 + 2 * 2 + (8 if a.bf16 else 0)       # minimal traffic: g, p r/w, m r/w, master r/w
    report(f"instinct step kind={kind}{' lagged' if a.lag else ''} shape={shape}", timeit(lambda: opt.update(p, g), a.iters), nbytes=float(n) * per,
           extra=f"(algorithmic {per} B/weight, one pass)")


def cmd_reread(a):
    """Re-reading kernels on the shapes of a memory model's step: rows = texts x segments, S words each, C cards."""
    import math
    from memarch_b200.models.reread import Reread
    from memarch_b200.ops import _ext
    torch.manual_seed(0)
    B, S, Cn, d, T = a.rows, a.words, a.cards, a.d, a.text
    mod = Reread(d).cuda()
    g = torch.Generator(device="cuda").manual_seed(1)
    rn = lambda *s_: torch.randn(*s_, device="cuda", generator=g)
    h, faces, contents = rn(B, S, d).requires_grad_(), rn(B, Cn, 2, 64), rn(B, Cn, d)
    valid = torch.rand(B, Cn, device="cuda", generator=g) > 0.2
    pos = torch.randint(0, T, (B, Cn), device="cuda", generator=g)
    qpos = torch.randint(0, T, (B, S), device="cuda", generator=g)
    n_texts = max(1, B // 8)
    rows = torch.randint(0, n_texts, (B,), device="cuda", generator=g)
    ids = torch.randint(0, 50000, (n_texts, T), device="cuda", generator=g)
    table = (rn(50304, 128) * 0.5).requires_grad_()

    def step():
        o, cost = mod(h, ids, table, faces, contents, pos, valid, qpos, rows)
        (o.sum() + cost).backward()
        h.grad = table.grad = None

    use = _ext.use_cuda
    step()
    o1, c1 = mod(h, ids, table, faces, contents, pos, valid, qpos, rows)
    _ext.use_cuda = lambda t: False
    try:
        o0, c0 = mod(h[:8], ids, table, faces[:8], contents[:8], pos[:8], valid[:8], qpos[:8], rows[:8])
        t_torch = timeit(step, max(2, a.iters // 3), flush=False)
    finally:
        _ext.use_cuda = use
    o1s, _ = mod(h[:8], ids, table, faces[:8], contents[:8], pos[:8], valid[:8], qpos[:8], rows[:8])
    print(f"parity (8 rows) output rel err {rel(o1s, o0):.2e}")
    t_k = timeit(step, a.iters, flush=False)
    print(f"re-reading forward + backward, {B * S} words x {Cn} cards: kernels {t_k:.3f} ms, PyTorch statement {t_torch:.3f} ms", flush=True)


def cmd_experts(a):
    from memarch_b200 import ops
    E, C, d, H = a.e, a.c, a.d, a.h
    x = torch.randn(E, C, d, device="cuda").bfloat16().requires_grad_()
    up = (torch.randn(E, d, H, device="cuda") * d ** -0.5).bfloat16().requires_grad_()
    down = (torch.randn(E, H, d, device="cuda") * H ** -0.5).bfloat16().requires_grad_()
    y = ops.expert_ffn(x, up, down, "relu2")
    yr = torch.bmm(torch.relu(torch.bmm(x[:1].float(), up[:1].float())) ** 2, down[:1].float())
    print(f"parity (expert 0) rel err {rel(y[:1], yr):.2e}")
    go = torch.randn_like(y)

    def fb():
        x.grad = up.grad = down.grad = None
        ops.expert_ffn(x, up, down, "relu2").backward(go)
    report(f"expert FFN relu2 fwd+bwd E{E} C{C} d{d} H{H}", timeit(fb, a.iters), 3 * 2 * 2.0 * E * C * d * H)


def cmd_attn(a):
    """Own tcgen05 attention forward against the library SDPA: parity and TFLOP/s over the visited blocks."""
    import torch.nn.functional as F
    from memarch_b200.ops.attention import _lib_window, own_attention
    B, H, T, W = a.batch, a.heads, a.seq, a.window
    q, k, v = (torch.randn(B, H, T, 64, device="cuda").bfloat16() for _ in range(3))
    o = own_attention(q, k, v, W)
    ref_o = F.scaled_dot_product_attention(q, k, v, is_causal=True) if not W or W >= T else _lib_window(q, k, v, W)
    print(f"parity rel err {rel(o, ref_o):.2e}")
    vis = (T * (T + 1) / 2) if not W or W >= T else (T * W - W * (W - 1) / 2)
    flops = 4.0 * B * H * vis * 64
    report(f"own attention fwd B{B} H{H} T{T} window {W}", timeit(lambda: own_attention(q, k, v, W), a.iters), flops)
    lib = (lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True)) if not W or W >= T else (lambda: _lib_window(q, k, v, W))
    report("library SDPA fwd (same shape)", timeit(lib, a.iters), flops)
    # forward + backward (3.5x the forward FLOPs: 2 products forward, 5 backward)
    import importlib
    A = importlib.import_module("memarch_b200.ops.attention")
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    go = torch.randn_like(q)

    def fb(f):
        def run():
            qg.grad = kg.grad = vg.grad = None
            f(qg, kg, vg).backward(go)
        return run
    own_f = lambda x, y, z: own_attention(x, y, z, W)
    lib_f = (lambda x, y, z: F.scaled_dot_product_attention(x, y, z, is_causal=True)) if not W or W >= T else \
        (lambda x, y, z: A._flash_window(x, y, z, W))
    fb(own_f)()
    g_own = [t.grad.clone() for t in (qg, kg, vg)]
    fb(lib_f)()
    print("backward parity rel err (dq, dk, dv):", " ".join(f"{rel(x, y.grad):.2e}" for x, y in zip(g_own, (qg, kg, vg))))
    report("own attention fwd+bwd", timeit(fb(own_f), a.iters), 3.5 * flops)
    report("library fwd+bwd (flash, window arguments where windowed)", timeit(fb(lib_f), a.iters), 3.5 * flops)


class _Clocks:
    """SM clock and board power sampled through NVML (read-only queries) on a thread while a loop runs."""

    def __init__(self, index=0, every=0.02):
        import threading
        self.index, self.every, self.sm, self.pw = index, every, [], []
        self._stop = threading.Event()
        self._th = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            while not self._stop.is_set():
                self.sm.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                self.pw.append(pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0)
                self._stop.wait(self.every)
        except Exception:    # noqa: BLE001 - no NVML: the sweep prints times only
            pass

    def __enter__(self):
        self._th.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._th.join(timeout=2)

    def summary(self):
        if not self.sm:
            return None, None
        h = self.sm[len(self.sm) // 3:]            # drop the ramp
        w = self.pw[len(self.pw) // 3:]
        return sum(h) / len(h), sum(w) / len(w)


def sustained(fn, seconds=0.6):
    """Back-to-back launches for `seconds`; returns (ms per launch, mean SM MHz, mean W)."""
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); fn(); e1.record(); torch.cuda.synchronize()
    n = max(8, int(seconds * 1e3 / max(e0.elapsed_time(e1), 1e-3)))
    with _Clocks() as c:
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
    mhz, w = c.summary()
    return e0.elapsed_time(e1) / n, mhz, w


def cmd_sweep(a):
    """The linears of the headline model and the square case, own pair kernel against the library GEMM: burst time
    (L2 flushed), sustained time with the SM clock and power seen, and tensor-pipe share = achieved / (clock x 148 SMs
    x 8192 FLOP per clock)."""
    from memarch_b200.ops import _ext, gemm
    C = _ext.C()
    shapes = {"square8k": (8192, 8192, 8192, 0, 0), "qkv": (32768, 6144, 2048, 0, 0), "o": (32768, 2048, 2048, 0, 0),
              "up": (32768, 16384, 2048, 0, 0), "down": (32768, 2048, 8192, 0, 0),
              "dgrad_up": (32768, 2048, 16384, 0, 1), "wgrad_up": (16384, 2048, 32768, 1, 1),
              "wgrad_qkv": (6144, 2048, 32768, 1, 1), "wgrad_down": (2048, 8192, 32768, 1, 1),
              "dgrad_qkv": (32768, 2048, 6144, 0, 1), "head": (4096, 50304, 2064, 0, 0)}
    names = a.shapes.split(",") if a.shapes else list(shapes)
    def parse(x):
        f = [int(t) for t in x.split(":")] + [0]
        return f[0], f[1]
    variants = [("lib", None, 0, 0)] + [("own" + (f"+dbg{d}" if d else "") + (f"+gm{gm}" if gm else ""), 1, d, gm)
                                         for d, gm in map(parse, a.variants.split(","))]
    for nm in names:
        M, N, K, a_mn, b_mn = shapes[nm]
        A = torch.randn(M, K, device="cuda").bfloat16()
        B = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
        Am = A.t().contiguous() if a_mn else A
        Bm = B.t().contiguous() if b_mn else B
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ref = A[:256].float() @ B.float().t()
        fl = 2.0 * M * N * K
        for label, v, d, gm in variants:
            if v is None:
                run = lambda: torch.matmul(A, B.t(), out=out)
            else:
                C.gemm_set_debug(d, gm)
                run = lambda: gemm(Am, Bm, a_mn=bool(a_mn), b_mn=bool(b_mn), out=out)
            run()
            err = rel(out[:256], ref)
            burst = timeit(run, a.iters)
            ms, mhz, w = sustained(run, a.seconds)
            share = (fl / ms / 1e9) / (mhz * 1e6 * 148 * 8192 / 1e12) if mhz else float("nan")
            print(f"{nm:10s} M{M} N{N} K{K} {label:14s} err {err:.1e}  burst {burst:.3f} ms {fl / burst / 1e9:6.0f} TF | sustained "
                  f"{ms:.3f} ms {fl / ms / 1e9:6.0f} TF at {mhz or 0:.0f} MHz {w or 0:.0f} W -> tensor share {share:.2f}", flush=True)
        C.gemm_set_debug(0, 0)
        st = C.gemm_status(0)
        if st:
            print(f"  status word {st} after {nm}", flush=True)
        del A, B, Am, Bm, out
        torch.cuda.empty_cache()


def cmd_route(a):
    """Anchor search of the long-range read: bf16 tensor-core scores + `rope_route_topk` against the PyTorch statement
    (fp32 einsum, masked max over links, top-k) on the same inputs."""
    import dataclasses
    from memarch_b200.models import rope_memory as rm
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    B, H, T, hd, A = a.batch, a.heads, a.seq, 64, a.anchors
    q, k = torch.randn(B, H, T, hd, device=dev), torch.randn(B, H, T, hd, device=dev)
    s = torch.rand(B, T, device=dev) * 2
    tau = float(s.flatten().kthvalue(int(s.numel() * (1 - A / T))).values)
    own, apos, avalid = rm.anchors_from_surprise(s.clone(), tau, A)
    cfg = rm.RopeCfg(K=4, links=8, win=64, span_cap=256, chunk=256, route="exact", route_bf16=True)
    plain = dataclasses.replace(cfg, route_bf16=False)
    fast = rm.route_exact(q, k, own, apos, avalid, cfg)
    slow = rm.route_exact(q, k, own, apos, avalid, plain)
    same = ((fast[0] == slow[0]) & (fast[1] == slow[1])).float().mean().item()
    flops = 2.0 * B * H * T * A * 8 * hd
    report(f"route kernel  B{B} H{H} T{T} A{A} L8", timeit(lambda: rm.route_exact(q, k, own, apos, avalid, cfg), a.iters),
           flops, extra=f"same choice as the fp32 statement on {same:.4f} of the slots; anchors {float(avalid.float().sum(1).mean()):.0f}")
    report("route PyTorch fp32", timeit(lambda: rm.route_exact(q, k, own, apos, avalid, plain), max(3, a.iters // 3)), flops)


def main(argv=None):
    ap = argparse.ArgumentParser(prog="memarch_b200 bench-kernel")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8192); g.add_argument("--n", type=int, default=8192)
    g.add_argument("--k", type=int, default=8192); g.add_argument("--groups", type=int, default=1)
    g.add_argument("--a-mn", dest="a_mn", action="store_true"); g.add_argument("--b-mn", dest="b_mn", action="store_true")
    g.add_argument("--no-lib", action="store_true"); g.add_argument("--no-flush", action="store_true")
    g.add_argument("--i8", action="store_true", help="the int8 tensor-core GEMM instead of the bf16 one")
    c = sub.add_parser("ce")
    c.add_argument("--rows", type=int, default=8192); c.add_argument("--d", type=int, default=2064)
    c.add_argument("--vocab", type=int, default=50304); c.add_argument("--mix", action="store_true")
    i = sub.add_parser("instinct")
    i.add_argument("--shape", default="8,2048,6144"); i.add_argument("--bf16", action="store_true", default=True)
    i.add_argument("--fp32", dest="bf16", action="store_false"); i.add_argument("--lag", action="store_true")
    r = sub.add_parser("reread")
    r.add_argument("--rows", type=int, default=256); r.add_argument("--words", type=int, default=128)
    r.add_argument("--cards", type=int, default=320); r.add_argument("--d", type=int, default=1024)
    r.add_argument("--text", type=int, default=1024)
    e = sub.add_parser("experts")
    e.add_argument("--e", type=int, default=8); e.add_argument("--c", type=int, default=2049)
    e.add_argument("--d", type=int, default=2048); e.add_argument("--h", type=int, default=6144)
    t = sub.add_parser("attn")
    t.add_argument("--batch", type=int, default=32); t.add_argument("--heads", type=int, default=32)
    t.add_argument("--seq", type=int, default=1024); t.add_argument("--window", type=int, default=0)
    t.add_argument("--iters", type=int, default=10)
    rt = sub.add_parser("route")
    rt.add_argument("--batch", type=int, default=4); rt.add_argument("--heads", type=int, default=8)
    rt.add_argument("--seq", type=int, default=4096); rt.add_argument("--anchors", type=int, default=1024)
    w = sub.add_parser("sweep")
    w.add_argument("--shapes", default=""); w.add_argument("--variants", default="0", help="dbg[:group_m],...")
    w.add_argument("--seconds", type=float, default=0.6)
    for p in (g, c, i, e, w, r, rt):
        p.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    sys.path.insert(0, ROOT)
    {"gemm": cmd_gemm, "ce": cmd_ce, "instinct": cmd_instinct, "experts": cmd_experts, "attn": cmd_attn, "sweep": cmd_sweep,
     "reread": cmd_reread, "route": cmd_route}[a.cmd](a)


if __name__ == "__main__":
    main()
