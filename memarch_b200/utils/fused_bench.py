"""Micro-benchmarks of the fused compute + collective paths, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m memarch_b200.utils.fused_bench [--e 8 --c 2049 --d 2048 --h 6144 --mb 256]

Reports, timed with CUDA events on every rank and reduced with max over ranks:
  * device-side barrier latency;
  * one-shot all-reduce (peer loads / NVLS multimem) against `dist.all_reduce`: time, bus bandwidth
    2 (W-1)/W x bytes / time, fraction of the measured 770 GB/s peer-copy bandwidth per direction;
  * expert-parallel FFN layer (dispatch + up GEMM + activation + down GEMM + combine), forward and forward+backward:
    fused path against the NCCL all-to-all path, with the roofline of the fused path = the slower of
    GEMM FLOPs / measured bf16 peak and off-chip bytes / link bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

LINK_GBS = 770.0            # measured peer copy, per direction per GPU
PEAK_TF = 1392.0            # measured sustained bf16 (overridden by MEASURED_PEAKS.json when present)


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        d = json.load(open(os.path.join(here, "MEASURED_PEAKS.json")))
        return float(d.get("bf16_tflops_sustained", PEAK_TF))
    except Exception:   # noqa: BLE001
        return PEAK_TF


def timed(fn, iters, world):
    for _ in range(2):
        fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--e", type=int, default=8)
    ap.add_argument("--c", type=int, default=2049)
    ap.add_argument("--d", type=int, default=2048)
    ap.add_argument("--h", type=int, default=6144)
    ap.add_argument("--mb", type=int, default=256, help="all-reduce message size in MiB")
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args(argv)
    from ..parallel import ParallelEngine, init_distributed
    from ..parallel.engine import _AllToAll
    from ..parallel.fused import FusedParallel, _FusedExpertFFN
    from ..ops import _ext
    from ..ops.moe import expert_ffn
    rank, W, local = init_distributed()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    eng = ParallelEngine(rank, W, local, fused=True)
    fp = FusedParallel(eng)
    heap = fp.heap
    C = _ext.C()
    say = (lambda *x: print(*x, flush=True)) if rank == 0 else (lambda *x: None)
    peak = _peaks()
    ok, why = fp.selftest()
    say(f"[fused-bench] W={W} self-test: {why}")

    # ---- barrier
    ms = timed(lambda: heap.barrier(2), 50, W)
    say(f"device barrier: {ms * 1e3:.1f} us")

    # ---- all-reduce
    n = a.mb * (1 << 20) // 2
    buf, bh = heap.alloc((n,), torch.bfloat16)
    out, oh = heap.alloc((n,), torch.bfloat16)
    buf.normal_()
    ip, op = [int(p) for p in bh.buffer_ptrs], [int(p) for p in oh.buffer_ptrs]
    nbytes = n * 2
    bus = lambda t_ms: 2 * (W - 1) / W * nbytes / (t_ms * 1e-3) / 1e9

    def ar(mi, mo):
        heap.barrier(1)
        C.peer_allreduce(ip, op, mi, mo, 0, n, True, rank, 1.0 / W)
        heap.barrier(1)
    t = timed(lambda: ar(0, 0), a.iters, W)
    say(f"all-reduce {a.mb} MiB bf16, peer loads/stores: {t:.3f} ms, bus {bus(t):.0f} GB/s = {bus(t) / LINK_GBS:.2f} of measured link")
    try:
        mi, mo = int(bh.multicast_ptr), int(oh.multicast_ptr)
    except Exception:   # noqa: BLE001
        mi = mo = 0
    if mi and mo and os.environ.get("MEMARCH_NVLS", "1") == "1":
        t = timed(lambda: ar(mi, mo), a.iters, W)
        say(f"all-reduce {a.mb} MiB bf16, NVLS multimem:     {t:.3f} ms, bus {bus(t):.0f} GB/s = {bus(t) / LINK_GBS:.2f} of measured link")
    x = buf.clone()
    t = timed(lambda: dist.all_reduce(x), a.iters, W)
    say(f"all-reduce {a.mb} MiB bf16, NCCL:              {t:.3f} ms, bus {bus(t):.0f} GB/s = {bus(t) / LINK_GBS:.2f} of measured link")

    # ---- expert-parallel FFN layer
    E, Cn, d, H = a.e, a.c, a.d, a.h
    El = E // W
    torch.manual_seed(1 + rank)
    xe = torch.randn(E, Cn, d, device=dev).bfloat16().requires_grad_()
    up = (torch.randn(El, d, H, device=dev) * d ** -0.5).bfloat16().requires_grad_()
    down = (torch.randn(El, H, d, device=dev) * H ** -0.5).bfloat16().requires_grad_()
    go = torch.randn(E, Cn, d, device=dev).bfloat16()
    gname = (eng.group or dist.group.WORLD).group_name if W > 1 else None

    def fused_fwd():
        return _FusedExpertFFN.apply(xe, up, down, fp.ep, "bench", "relu2", rank * El, El, True)

    def nccl_fwd():
        if W == 1:
            return expert_ffn(xe, up, down, "relu2")
        r = _AllToAll.apply(xe, gname).view(W, El, Cn, d).transpose(0, 1).reshape(El, W * Cn, d)
        y = expert_ffn(r, up, down, "relu2")
        y = y.view(El, W, Cn, d).transpose(0, 1).reshape(E, Cn, d).contiguous()
        return _AllToAll.apply(y, gname)

    def fb(f):
        def run():
            xe.grad = up.grad = down.grad = None
            f().backward(go)
        return run
    flops_f = 2 * 2.0 * E * Cn * d * H                       # this rank's experts see W x Cn rows each: El x W x Cn = E x Cn
    off = (W - 1) / W * E * Cn * d * 2                        # bytes leaving / entering this GPU per exchange
    roof_f = max(flops_f / (peak * 1e12), 2 * off / (LINK_GBS * 1e9)) * 1e3
    roof_fb = max(3 * flops_f / (peak * 1e12), 4 * off / (LINK_GBS * 1e9)) * 1e3
    with torch.no_grad():
        tf = timed(fused_fwd, a.iters, W)
        tn = timed(nccl_fwd, a.iters, W)
    say(f"EP FFN layer forward  E{E} C{Cn} d{d} H{H}: fused {tf:.3f} ms ({roof_f / tf:.2f} of its roofline {roof_f:.3f} ms), "
        f"NCCL path {tn:.3f} ms")
    tfb = timed(fb(fused_fwd), a.iters, W)
    tnb = timed(fb(nccl_fwd), a.iters, W)
    say(f"EP FFN layer fwd+bwd: fused {tfb:.3f} ms ({roof_fb / tfb:.2f} of its roofline {roof_fb:.3f} ms), NCCL path {tnb:.3f} ms")
    # ---- data-parallel optimizer step of replicated weights: row-sharded (reduce-scatter + update of the owned rows +
    #      all-gather of the new bf16 rows) against all-reduce + full update on every rank
    import types
    from ..config import OptConfig
    from ..optim import Instinct
    from ..parallel.fused import FusedGradReduce
    R_, C_, nw = 2048, 8192, 8
    res = {}
    for mode in ("sharded", "replicated", "nccl"):
        torch.manual_seed(5)
        ps = [torch.nn.Parameter((torch.randn(R_, C_, device=dev) * 0.02).bfloat16()) for _ in range(nw)]
        opt = Instinct(ps, OptConfig(lr=1e-3, norm="hs", scale=0.12, m_bf16=True, rel_every=1 << 30))
        opt.prepare(torch.tensor(3.0, device=dev), torch.randn(64, device=dev))
        opt.n_step = 1                                         # no |g|/|w| sums in the timed steps
        gs = [torch.randn(R_, C_, device=dev).bfloat16() for _ in range(nw)]
        if mode == "nccl":
            def step():
                for p_, g_ in zip(ps, gs):
                    g2 = g_.clone()
                    if W > 1:
                        dist.all_reduce(g2)
                    opt.update(p_, g2.div_(W))
        else:
            dp = FusedGradReduce(heap)
            dp.shard = mode == "sharded"
            dp.trainer = types.SimpleNamespace(opt=opt, params=ps)
            dp.allocate(ps)

            def step(dp=dp):
                for p_, g_ in zip(ps, gs):
                    dp.grad_ready(p_, g_)
                dp.flush()
        res[mode] = timed(step, a.iters, W) / nw
    n_el = R_ * C_
    link_ms = (W - 1) / W * n_el * 2 / (LINK_GBS * 1e9) * 1e3           # rows in (reduce) and out (gather) run in both directions at once
    hbm_ms = (8 + 28 / W) * n_el / 6.45e12 * 1e3                          # staging, peers' reads, statistics and update of the owned rows, incoming rows
    roof = max(link_ms, hbm_ms)
    say(f"DP optimizer step per {R_}x{C_} bf16 weight ({nw} in flight): row-sharded {res['sharded'] * 1e3:.0f} us "
        f"({roof / res['sharded']:.2f} of its roofline {roof * 1e3:.0f} us = max(link {link_ms * 1e3:.0f}, HBM {hbm_ms * 1e3:.0f})), "
        f"all-reduce + full update {res['replicated'] * 1e3:.0f} us, NCCL all-reduce + full update {res['nccl'] * 1e3:.0f} us")
    torch.cuda.synchronize()
    heap.check()
    if W > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
