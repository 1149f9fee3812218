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
        ln, lf = res["nccl"][0], res["fused"][0]
        for a, b in zip(ln, lf):
            assert abs(a - b) < 2e-2 * max(1.0, abs(a)), (rank, ln, lf)
        for k, v in res["nccl"][1].items():
            w = res["fused"][1][k]
            den = np.abs(v).max() + 1e-6
            assert np.abs(v - w).max() / den < 5e-2, (rank, k)


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
        res[mode] = (losses, {k: v.detach().float().cpu().numpy() for k, v in m.state_dict().items()
                              if v.dtype.is_floating_point and 0 < v.numel() < 1 << 22})
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
    for a, b in zip(res["plain"][0], res["fused"][0]):
        assert abs(a - b) < 2e-2 * max(1.0, abs(a)), (res["plain"][0], res["fused"][0])
    for k, v in res["plain"][1].items():
        w = res["fused"][1][k]
        assert np.abs(v - w).max() / (np.abs(v).max() + 1e-6) < 5e-2, k
