"""Fused peer-memory paths on 2 GPUs against the NCCL-only baseline mode: expert-parallel FFN (forward + all grads)
and the data-parallel gradient mean + optimizer step.  Skipped with fewer than 2 GPUs."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0", MEMARCH_NVLS="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.parallel import ParallelEngine
    from memarch_b200.train import Trainer
    res = {}
    for mode in ("nccl", "fused"):
        torch.manual_seed(0)
        m = build("tiny", 2048, bf16_experts=True, moe_act="relu2").cuda()
        eng = ParallelEngine(rank, world, rank, fused=mode == "fused")
        tr = Trainer(m, TrainConfig(batch=4, micro=4, seq=256, lr=1e-3, warmup=2, steps=10),
                     OptConfig(norm="hs", scale=0.12, m_bf16=True, rel_every=2), stage="ABX", parallel=eng)
        g = torch.Generator(device="cuda").manual_seed(1 + rank)
        losses = []
        for s in range(3):
            xy = torch.randint(0, 2048, (4, 257), device="cuda", generator=g)
            losses.append(float(tr.step(xy, s)))
        torch.cuda.synchronize()
        if eng.fused_impl is not None:
            eng.fused_impl.heap.check()
            res["selftest"] = eng.fused_impl.selftest()
            res["n_sharded"] = len(eng.fused_impl.dp.sharded)
            eng.before_checkpoint()                     # rows of the sharded weights kept by the other rank come home
        res[mode] = (losses, {k: v.detach().float().cpu().numpy() for k, v in m.state_dict().items()
                              if v.dtype.is_floating_point and 0 < v.numel() < 1 << 22})
    q.put((rank, res))
    dist.barrier()
    dist.destroy_process_group()


def test_fused_matches_nccl_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import numpy as np
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_worker, args=(r, 2, 29731, q)) for r in range(2)]
    for p in ps:
        p.start()
    out = [q.get(timeout=240) for _ in ps]
    for p in ps:
        p.join(60)
    for rank, res in out:
        assert res["selftest"] == (True, "ok"), (rank, res["selftest"])
        assert res["n_sharded"] > 0, "the row-sharded optimizer path was not taken"
        ln, lf = res["nccl"][0], res["fused"][0]
        for a, b in zip(ln, lf):
            assert abs(a - b) < 5e-3 * max(1.0, abs(a)), (rank, ln, lf)
        worst = max((np.abs(v - res["fused"][1][k]).max() / (np.abs(v).max() + 1e-6), k) for k, v in res["nccl"][1].items())
        print(f"rank {rank}: losses {ln} / {lf}; largest weight difference {worst[0]:.2e} of the weight's range ({worst[1]})")
        # bf16 weights stepped with stochastic rounding by two different reduction orders: a few bf16 steps apart
        assert worst[0] < 2e-2, worst


def _single_rank(q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29741", RANK="0", WORLD_SIZE="1", LOCAL_RANK="0",
                      MEMARCH_NVLS="0")
    import torch.distributed as dist
    torch.cuda.set_device(0)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.parallel import ParallelEngine
    from memarch_b200.train import Trainer
    res = {}
    for mode in ("plain", "fused"):
        torch.manual_seed(0)
        m = build("tiny", 2048, bf16_experts=True, moe_act="relu2").cuda()
        eng = ParallelEngine(0, 1, 0, fused=True) if mode == "fused" else None
        tr = Trainer(m, TrainConfig(batch=4, micro=4, seq=256, lr=1e-3, warmup=2, steps=10),
                     OptConfig(norm="hs", scale=0.12, m_bf16=True, rel_every=2), stage="ABX", parallel=eng)
        g = torch.Generator(device="cuda").manual_seed(1)
        losses = []
        for s in range(3):
            losses.append(float(tr.step(torch.randint(0, 2048, (4, 257), device="cuda", generator=g), s)))
        torch.cuda.synchronize()
        if eng is not None:
            eng.fused_impl.heap.check()
            res["selftest"] = eng.fused_impl.selftest()
            res["n_sharded"] = len(eng.fused_impl.dp.sharded)
        res[mode] = (losses, {k: v.detach().float().cpu().numpy() for k, v in m.state_dict().items()
                              if v.dtype.is_floating_point and 0 < v.numel() < 1 << 22})
        if eng is not None:
            # a bank layer with frozen experts runs the fused exchange twice (learning and frozen experts) over shared
            # gradient buffers: the input gradient must equal the local computation, rows of the other bank included
            from memarch_b200.models.moe import AnchorMoE
            torch.manual_seed(3)
            moe = AnchorMoE(256, E=4, k_avg=2, k_max=2, bank=True, act="relu2", w_dtype=torch.bfloat16).cuda()
            moe.grow_bank(4)
            xe0 = (torch.randn(moe.E, 300, 256, device="cuda") * 0.5).bfloat16()
            go = torch.randn(moe.E, 300, 256, device="cuda").bfloat16()
            outs = []
            for fused in (False, True):
                xe = xe0.clone().requires_grad_()
                moe.up.grad = moe.down.grad = None
                moe._counts = None
                if fused:
                    eng.fused_impl.ep.ffn(moe, xe).backward(go)            # twice: stale rows of an earlier call must not leak
                    xe.grad = moe.up.grad = moe.down.grad = None
                    y = eng.fused_impl.ep.ffn(moe, xe)
                else:
                    y = moe._experts(xe, None, 300)
                y.backward(go)
                outs.append((y.detach().float(), xe.grad.float(), moe.up.grad.float(), moe.down.grad.float()))
            rel = lambda a, b: float((a - b).norm() / b.norm().clamp(min=1e-9))
            res["bank_err"] = [rel(a, b) for a, b in zip(outs[1], outs[0])]
    q.put(res)
    dist.destroy_process_group()


def test_fused_kernels_on_one_rank_match_plain_path():
    """World size 1: the fused kernels (segmented GEMM through symmetric buffers, barrier, one-shot all-reduce) run
    against this GPU's own buffers and must reproduce the plain single-GPU step."""
    import numpy as np
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_single_rank, args=(q,))
    p.start()
    res = q.get(timeout=240)
    p.join(60)
    assert res["selftest"] == (True, "ok"), res["selftest"]          # the pre-run check of the peer paths itself
    assert res["n_sharded"] > 0, "the row-sharded optimizer path was not taken"
    assert max(res["bank_err"]) < 1e-2, res["bank_err"]              # y, d xe, d up, d down of a layer with frozen experts
    for a, b in zip(res["plain"][0], res["fused"][0]):
        assert abs(a - b) < 5e-3 * max(1.0, abs(a)), (res["plain"][0], res["fused"][0])
    for k, v in res["plain"][1].items():
        w = res["fused"][1][k]
        assert np.abs(v - w).max() / (np.abs(v).max() + 1e-6) < 2e-2, k            # a few bf16 steps (stochastic rounding)


def test_bounded_barrier_wait_runs_out_and_reports():
    """A device-side barrier whose peer never arrives: the wait gives up after its limit, the status word says so,
    `SymmetricHeap.check` raises, and the device keeps working.  The "peer" is a second flag array in this GPU's own
    memory that nobody signals, so nothing waits on another process and nothing faults."""
    import time
    from memarch_b200.ops import _ext
    from memarch_b200.parallel.fused import SymmetricHeap
    C = _ext.C()
    assert C.peer_status_read() == 0
    mine = torch.zeros(256, dtype=torch.int32, device="cuda")
    other = torch.zeros(256, dtype=torch.int32, device="cuda")
    t0 = time.time()
    C.peer_barrier([mine.data_ptr(), other.data_ptr()], 0, 0, 5.0)        # rank 0 of 2, limit 5 ms
    torch.cuda.synchronize()
    assert time.time() - t0 < 2.0
    heap = SymmetricHeap.__new__(SymmetricHeap)                           # only `check` is exercised
    heap.wait_ms = 5.0
    with pytest.raises(RuntimeError, match="peer wait timed out"):
        heap.check()
    assert C.peer_status_read() == 0                                      # read-and-clear
    x = torch.arange(1024, device="cuda", dtype=torch.float32)
    assert float((x * 2).sum()) == 1023 * 1024                            # the context is alive
    # a complete barrier of one rank still passes afterwards
    C.peer_barrier([mine.data_ptr()], 0, 1, 5.0)
    torch.cuda.synchronize()
    assert C.peer_status_read() == 0
