"""Multi-rank semantics on CPU (gloo, world_size 2): expert parallelism + data parallelism reproduce the single-rank
run when every rank sees the same data, and average over ranks when they see different data."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run_single(xys, steps):
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.train import Trainer
    torch.manual_seed(0)
    m = build("tiny", 512)
    tr = Trainer(m, TrainConfig(batch=xys[0].shape[0], micro=xys[0].shape[0], seq=64, lr=1e-3, warmup=2, steps=10),
                 OptConfig(norm="hs", scale=0.12, rel_every=1), stage="ABX")
    losses = [float(tr.step(xys[s], s)) for s in range(steps)]
    return losses, {k: v.detach().clone() for k, v in m.state_dict().items()}


def _worker(rank, world, port, same, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.parallel import ParallelEngine
    from memarch_b200.train import Trainer
    torch.manual_seed(0)
    m = build("tiny", 512)
    eng = ParallelEngine(rank, world, 0, fused=False)
    tr = Trainer(m, TrainConfig(batch=4, micro=4, seq=64, lr=1e-3, warmup=2, steps=10),
                 OptConfig(norm="hs", scale=0.12, rel_every=1), stage="ABX", parallel=eng)
    g = torch.Generator().manual_seed(1 if same else 1 + rank)
    losses = []
    for s in range(3):
        xy = torch.randint(0, 512, (4, 65), generator=g)
        losses.append(float(tr.step(xy, s)))
    sd = {k: v.detach().float().numpy().copy() for k, v in m.state_dict().items()
          if v.dtype.is_floating_point and ("heavy" not in k or "router" in k or "norm" in k)}
    q.put((rank, losses, sd, float(m.tau)))
    dist.barrier()
    dist.destroy_process_group()


def _spawn(same, port):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_worker, args=(r, 2, port, same, q)) for r in range(2)]
    for p in ps:
        p.start()
    out = sorted([q.get(timeout=300) for _ in ps], key=lambda t: t[0])
    for p in ps:
        p.join(60)
    return out


def test_same_data_on_two_ranks_equals_one_rank():
    g = torch.Generator().manual_seed(1)
    xys = [torch.randint(0, 512, (4, 65), generator=g) for _ in range(3)]
    ref_losses, ref_sd = _run_single(xys, 3)
    out = _spawn(True, 29641)
    for rank, losses, sd, tau in out:
        for a, b in zip(losses, ref_losses):
            assert abs(a - b) < 2e-4 * max(1, abs(b)), (rank, losses, ref_losses)
        for k, v in sd.items():
            assert torch.allclose(torch.from_numpy(v), ref_sd[k].float(), atol=2e-4, rtol=1e-3), k


def test_different_data_ranks_stay_in_sync():
    out = _spawn(False, 29643)
    (_, l0, sd0, tau0), (_, l1, sd1, tau1) = out
    assert l0 != l1                                  # different data -> different local losses
    assert abs(tau0 - tau1) < 1e-6                   # shared anchor threshold
    for k in sd0:
        assert abs(sd0[k] - sd1[k]).max() < 1e-6, k                   # replicated weights identical on both ranks


def _w_vocab_and_shard(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank), "WORLD_SIZE": str(world)})
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from memarch_b200.config import OptConfig
    from memarch_b200.optim.instinct import Instinct
    from memarch_b200.parallel import vocab
    torch.manual_seed(0)
    V, d, N = 50, 16, 24
    table, head = torch.randn(V, d), torch.randn(V, d)
    ids, h, y = torch.randint(0, V, (N,)), torch.randn(N, d), torch.randint(0, V, (N,))
    ts, lo = vocab.shard_rows(table, rank, world)
    hs, _ = vocab.shard_rows(head, rank, world)
    ts.requires_grad_(True); hs.requires_grad_(True)
    hh = h.clone().requires_grad_(True)
    e = vocab.take(ts, ids, lo)
    loss = vocab.ce(hh + e * 0.1, hs, y, lo, chunk=7)
    loss.backward()
    # row-sharded homeostasis: this rank's rows of a (12, 8) weight
    torch.manual_seed(1)
    w, g = torch.randn(12, 8), torch.randn(12, 8)
    n = 12 // world
    p = torch.nn.Parameter(w[rank * n:(rank + 1) * n].clone())
    p._row_shard = (world, 12, None)
    opt = Instinct([p], OptConfig(lr=1e-2, norm="hs", scale=1.0))
    opt.prepare(torch.tensor(1.0), torch.ones(4))
    opt.update(p, g[rank * n:(rank + 1) * n].clone())
    q.put((rank, loss.item(), ts.grad.numpy(), hs.grad.numpy(), hh.grad.numpy(), p.detach().numpy()))
    dist.barrier()
    dist.destroy_process_group()


def test_vocab_parallel_and_row_sharded_homeostasis_match_single_rank():
    import torch.multiprocessing as mp
    import torch.nn.functional as F
    from memarch_b200.config import OptConfig
    from memarch_b200.optim.instinct import Instinct
    world, port = 2, 29631
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_w_vocab_and_shard, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in ps]
    res = sorted([q.get(timeout=120) for _ in ps], key=lambda r: r[0])
    [p.join(30) for p in ps]
    torch.manual_seed(0)
    V, d, N = 50, 16, 24
    table, head = torch.randn(V, d, requires_grad=True), torch.randn(V, d, requires_grad=True)
    ids, h, y = torch.randint(0, V, (N,)), torch.randn(N, d, requires_grad=True), torch.randint(0, V, (N,))
    loss = F.cross_entropy((h + table[ids] * 0.1) @ head.t(), y, reduction="sum")
    loss.backward()
    assert abs(res[0][1] - loss.item()) < 1e-3 and abs(res[1][1] - loss.item()) < 1e-3
    n = V // world
    for r in range(world):
        assert np.allclose(res[r][2], table.grad[r * n:(r + 1) * n].numpy(), atol=1e-4)
        assert np.allclose(res[r][3], head.grad[r * n:(r + 1) * n].numpy(), atol=1e-4)
        assert np.allclose(res[r][4], h.grad.numpy(), atol=1e-4)
    torch.manual_seed(1)
    w, g = torch.randn(12, 8), torch.randn(12, 8)
    p = torch.nn.Parameter(w.clone())
    opt = Instinct([p], OptConfig(lr=1e-2, norm="hs", scale=1.0))
    opt.prepare(torch.tensor(1.0), torch.ones(4))
    opt.update(p, g.clone())
    got = np.concatenate([res[0][5], res[1][5]])
    assert np.allclose(got, p.detach().numpy(), atol=1e-6)


def _w_vocab_dp(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank), "WORLD_SIZE": str(world)})
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from memarch_b200.parallel import vocab
    torch.manual_seed(0)
    V, d, N = 50, 16, 12
    table, head = torch.randn(V, d), torch.randn(V, d)
    ids, h, y = torch.randint(0, V, (world, 3, 4)), torch.randn(world, N, d), torch.randint(0, V, (world, N))
    ts, lo = vocab.shard_rows(table, rank, world)
    hs, _ = vocab.shard_rows(head, rank, world)
    ts.requires_grad_(True); hs.requires_grad_(True)
    hh = h[rank].clone().requires_grad_(True)                  # this rank's own tokens
    e = vocab.take_dp(ts, ids[rank], lo)
    assert e.shape == (3, 4, d)
    loss = vocab.ce_dp(hh + e.view(N, d) * 0.1, hs, y[rank], lo, chunk=5)
    loss.backward()
    q.put((rank, loss.item(), ts.grad.numpy(), hs.grad.numpy(), hh.grad.numpy()))
    dist.barrier()
    dist.destroy_process_group()


def test_vocab_parallel_with_rank_local_data_matches_the_whole_batch():
    import torch.multiprocessing as mp
    import torch.nn.functional as F
    world, port = 2, 29633
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_w_vocab_dp, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in ps]
    res = sorted([q.get(timeout=120) for _ in ps], key=lambda r: r[0])
    [p.join(30) for p in ps]
    torch.manual_seed(0)
    V, d, N = 50, 16, 12
    table, head = torch.randn(V, d, requires_grad=True), torch.randn(V, d, requires_grad=True)
    ids, h, y = torch.randint(0, V, (world, 3, 4)), torch.randn(world, N, d, requires_grad=True), torch.randint(0, V, (world, N))
    x = h + table[ids].view(world, N, d) * 0.1
    loss = F.cross_entropy(x.view(-1, d) @ head.t(), y.view(-1), reduction="sum")
    loss.backward()
    n = V // world
    for r in range(world):
        assert abs(res[r][1] - loss.item()) < 1e-3
        assert np.abs(res[r][2] - table.grad[r * n:(r + 1) * n].numpy()).max() < 1e-4
        assert np.abs(res[r][3] - head.grad[r * n:(r + 1) * n].numpy()).max() < 1e-4
        assert np.abs(res[r][4] - h.grad[r].numpy()).max() < 1e-4


def _w_ring(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from memarch_b200.parallel.engine import _Ring, ring_exchange
    torch.manual_seed(10 + rank)
    x = torch.randn(world * 2, 5, 3)
    want = torch.empty_like(x)
    dist.all_to_all_single(want, x)
    got = ring_exchange(x)
    xg = x.clone().requires_grad_(True)
    y = _Ring.apply(xg, None)
    wgt = torch.arange(y.numel(), dtype=torch.float32).view_as(y) * (rank + 1)
    (y * wgt).sum().backward()
    gwant = torch.empty_like(x)
    dist.all_to_all_single(gwant, wgt)                       # the cotangent travels back by the same permutation
    q.put((rank, bool(torch.equal(got, want)), bool(torch.equal(xg.grad, gwant))))
    dist.barrier()
    dist.destroy_process_group()


def test_ring_exchange_equals_all_to_all_on_three_ranks():
    world, port = 3, 29637
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_w_ring, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in ps]
    res = [q.get(timeout=120) for _ in ps]
    [p.join(30) for p in ps]
    assert len(res) == 3 and all(fwd and bwd for _, fwd, bwd in res)


def _w_dedup(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from memarch_b200.models.moe import AnchorMoE
    from memarch_b200.parallel.engine import NcclExpertExchange
    torch.manual_seed(0)
    moe = AnchorMoE(32, E=4, k_avg=2, k_max=4, budget=True, act="relu2")       # two experts per rank
    eng = NcclExpertExchange(rank, world)
    moe.ep_shard(rank, world, eng)
    moe.train()
    g = torch.Generator().manual_seed(3 + rank)                                  # every rank its own tokens
    x0 = torch.randn(2, 24, 32, generator=g)
    sur = torch.rand(2, 24, generator=g) * 4
    go = torch.randn(2, 24, 32, generator=g)
    res = {}
    s_mean = moe.s_mean.clone()
    for mode in ("plain", "dedup", "capped"):
        eng.dedup, eng.dedup_cap = mode != "plain", 0.25 if mode == "capped" else 1.0
        moe.s_mean.copy_(s_mean)
        x = x0.clone().requires_grad_(True)
        moe.up.grad = moe.down.grad = moe.router.weight.grad = None
        y = moe(x, sur)
        y.backward(go)
        res[mode] = (y.detach().clone(), x.grad.clone(), moe.up.grad.clone(), moe.router.weight.grad.clone(),
                     float(moe.dropped))
    # a bank layer (experts with the "stopped changing" wave): the error probe reads the word gradients in the
    # deduplicated exchange and the per-place gradients in the plain one - same numbers
    torch.manual_seed(1)
    bank = AnchorMoE(32, E=4, k_avg=2, k_max=2, bank=True, act="relu2")
    bank.ep_shard(rank, world, eng)
    bank.train()
    errs = {}
    for mode in ("plain", "dedup"):
        eng.dedup, eng.dedup_cap = mode == "dedup", 1.0
        bank.err.zero_()
        x = x0.clone().requires_grad_(True)
        yb = bank(x, None)
        yb.backward(go)
        errs[mode] = (bank.err.clone().numpy(), yb.detach().numpy())
    res["bank_err"] = [errs["plain"][0], errs["dedup"][0], errs["plain"][1], errs["dedup"][1]]
    q.put((rank, {k: [t.numpy() if torch.is_tensor(t) else t for t in v] for k, v in res.items()}))
    dist.barrier()
    dist.destroy_process_group()


def test_deduplicated_expert_exchange_matches_the_plain_one():
    world, port = 2, 29641
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_w_dedup, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in ps]
    res = [q.get(timeout=180) for _ in ps]
    [p.join(30) for p in ps]
    for _, r in res:
        for a, b in zip(r["plain"][:4], r["dedup"][:4]):
            assert np.abs(a - b).max() < 2e-5 * max(1.0, np.abs(a).max())
        assert abs(r["plain"][4] - r["dedup"][4]) < 1e-6                          # same drops
        assert r["capped"][4] > r["plain"][4] + 0.05                              # pairs beyond the parcel are dropped
        assert np.isfinite(r["capped"][0]).all() and np.abs(r["capped"][0] - r["plain"][0]).max() > 1e-3
        e_plain, e_dedup, y_plain, y_dedup = r["bank_err"]
        assert np.abs(y_plain - y_dedup).max() < 2e-5 * max(1.0, np.abs(y_plain).max())
        assert e_plain.max() > 0 and np.abs(e_plain - e_dedup).max() < 1e-5 * e_plain.max() + 1e-9


def _w_vp_model(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from memarch_b200.models.blocks import TransformerLM
    torch.manual_seed(0)
    V, d, T = 64, 32, 12
    full = TransformerLM(V, d=d, layers=2, heads=2, fused_ce=False)
    torch.manual_seed(0)
    vpm = TransformerLM(V, d=d, layers=2, heads=2, fused_ce=False).vocab_shard(rank, world)
    g = torch.Generator().manual_seed(7)
    xy_all = torch.randint(0, V, (2 * world, T + 1), generator=g)          # the whole batch, rank r owns rows 2r, 2r+1
    mine = xy_all[2 * rank:2 * rank + 2]
    full.train(); vpm.train()
    out, _ = vpm(mine[:, :-1])
    loss = vpm.train_loss(out, mine[:, 1:])
    loss.backward()
    out_f, _ = full(xy_all[:, :-1])
    loss_f = full.train_loss(out_f, xy_all[:, 1:])
    loss_f.backward()
    res = {"loss": (float(loss), float(loss_f))}
    # replicated weights: the rank mean of the local gradients is the gradient of the whole-batch mean loss
    gq = vpm.blocks[0].qkv.weight.grad.clone()
    dist.all_reduce(gq)
    res["qkv"] = float((gq / world - full.blocks[0].qkv.weight.grad).abs().max() / full.blocks[0].qkv.weight.grad.abs().max())
    lo, hi = rank * V // world, (rank + 1) * V // world
    for nm, a, b in (("emb", vpm.emb.weight.grad, full.emb.weight.grad[lo:hi]), ("head", vpm.head.weight.grad, full.head.weight.grad[lo:hi])):
        res[nm] = float((a - b).abs().max() / b.abs().max().clamp(min=1e-9))
    res["rows"] = (tuple(vpm.emb.weight.shape), tuple(vpm.head.weight.shape))
    q.put((rank, res))
    dist.barrier()
    dist.destroy_process_group()


def test_vocab_parallel_transformer_matches_the_unsharded_one():
    """TransformerLM with its word tables row-sharded over 2 ranks, each rank on its own rows of the batch: loss and
    gradients equal those of the unsharded model on the whole batch (replicated weights after the data-parallel mean,
    table shards after their 1/W hook)."""
    world, port = 2, 29655
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_w_vp_model, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in ps]
    res = [q.get(timeout=180) for _ in ps]
    [p.join(30) for p in ps]
    for _, r in res:
        assert r["rows"] == ((32, 32), (32, 32))
        assert abs(r["loss"][0] - r["loss"][1]) < 1e-5
        assert r["qkv"] < 1e-4 and r["emb"] < 1e-4 and r["head"] < 1e-4, r


def _w_vp_main(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from memarch_b200.config import ModelConfig
    from memarch_b200.models.memarch import MemArchLM
    V, T = 64, 24

    def make():
        torch.manual_seed(0)
        c = ModelConfig(vocab=V, d=32, heads=2, light_a=1, light_b=1, heavy=1, final=1, window=16, seg=8, moe="",
                        no_mem=True, frac=0.3, cap=0.5, induct="lock", induct_mix=True, induct_in=True)
        return MemArchLM(c).train()
    full, vpm = make(), make()
    vpm.vocab_shard(rank, world)
    g = torch.Generator().manual_seed(7)
    xy_all = torch.randint(0, 12, (2 * world, T + 1), generator=g)        # few distinct words: the locks fire often
    mine = xy_all[2 * rank:2 * rank + 2]
    out, _ = vpm(mine[:, :-1])
    loss = vpm.train_loss(out, mine[:, 1:])
    loss.backward()
    out_f, _ = full(xy_all[:, :-1])
    loss_f = full.train_loss(out_f, xy_all[:, 1:])
    loss_f.backward()
    lm = loss.detach().clone()
    dist.all_reduce(lm)
    res = {"loss": (float(lm / world), float(loss_f)), "tau": (float(vpm.tau), float(full.tau))}
    for nm in ("light_a.0.qkv.weight", "heavy.0.up.weight", "l_head.0.weight", "norm.weight"):
        a, b = dict(vpm.named_parameters())[nm].grad.clone(), dict(full.named_parameters())[nm].grad
        dist.all_reduce(a)
        res[nm] = float((a / world - b).abs().max() / b.abs().max().clamp(min=1e-9))
    lo, hi = rank * V // world, (rank + 1) * V // world
    for nm in ("emb.weight", "head.weight", "l_head.1.weight"):
        a, b = dict(vpm.named_parameters())[nm].grad, dict(full.named_parameters())[nm].grad[lo:hi]
        res[nm] = float((a - b).abs().max() / b.abs().max().clamp(min=1e-9))
        res[nm + ".rows"] = a.shape[0]
    q.put((rank, res))
    dist.barrier()
    dist.destroy_process_group()


def test_vocab_parallel_main_model_matches_the_unsharded_one():
    """MemArchLM with emb, head and the light head's output table row-sharded over 2 ranks, each rank on its own rows
    of the batch: the rank-mean loss, the replicated weights' rank-mean gradients and the shards' gradients equal
    those of the unsharded model on the whole batch."""
    world, port = 2, 29671
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_w_vp_main, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in ps]
    res = [q.get(timeout=240) for _ in ps]
    [p.join(30) for p in ps]
    for _, r in res:
        assert abs(r["loss"][0] - r["loss"][1]) < 1e-5, r
        for nm in ("light_a.0.qkv.weight", "heavy.0.up.weight", "l_head.0.weight", "norm.weight", "emb.weight", "head.weight",
                   "l_head.1.weight"):
            assert r[nm] < 2e-4, (nm, r)
        assert r["emb.weight.rows"] == 32 and r["l_head.1.weight.rows"] == 32


def _w_loop(rank, world, port, folder, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import io
    import json
    from memarch_b200.parallel import ParallelEngine
    from memarch_b200.train.loop import train
    from test_runtime_cpu import Args
    env = {"VOCAB": "1024", "NO_MEM": "1", "WATCHDOG": "0", "RANK": str(rank), "WORLD_SIZE": str(world),
           "CORPUS": json.dumps({"web": 0.7, "code": 0.3}), "CORPUS_ROOT": folder,
           "REMIND_P": "1.0", "REMIND_N": "4", "REMIND_DIST": "4", "REMIND_TOK0": "100", "REMIND_SYNTH": "3", "VAL_BATCHES": "2",
           "REMIND_PACK": "1", "REMIND_PACK_ROUND": "16", "REMIND_BLANK": "1", "REMIND_WIN": "8", "REMIND_THR": "0.0",
           "REMIND_LAG": "1", "REMIND_W": "1.0", "REMIND_MEAN": "1", "UROBOROS": "1", "ROLLBACK": "0",
           "OPT_KW": json.dumps({"norm": "hs", "scale": 0.12})}
    buf = io.StringIO()
    log = train(Args(seq=48, batch=2, micro=2, steps=4, eval_every=2), "cpu", env=env, out=buf,
                parallel=ParallelEngine(rank, world, 0, fused=False))["tiny"]
    moves = [ln for ln in buf.getvalue().splitlines() if ln.startswith(("episodes:", "reminders:", "hoop:"))]
    q.put((rank, moves, [e["val"] for e in log]))
    dist.barrier()
    dist.destroy_process_group()


def test_curricula_stay_in_step_across_ranks(tmp_path):
    """Two ranks with different text: the needle curriculum (which sets batch shapes) and the hoop's budget move on
    rank-summed statistics, so both ranks log the same moves at the same batches and the run does not stall."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from test_runtime_cpu import make_corpus
    make_corpus(str(tmp_path), n_shards=4, docs=60)
    world, port = 2, 29683
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_w_loop, args=(r, world, port, str(tmp_path), q)) for r in range(world)]
    [p.start() for p in ps]
    res = sorted([q.get(timeout=400) for _ in ps], key=lambda t: t[0])
    [p.join(30) for p in ps]
    (_, m0, v0), (_, m1, v1) = res
    strip = lambda ms: [ln.split("(accuracy")[0] + ln.split(")", 1)[-1] if "(accuracy" in ln else ln for ln in ms]
    assert m0 and strip(m0) == strip(m1), (m0, m1)
    assert any(ln.startswith("episodes: step 0 -> 1") for ln in m0)
    assert all(torch.isfinite(torch.tensor(v0 + v1)))


def _w_ckpt(rank, world, port, folder, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.parallel import ParallelEngine
    from memarch_b200.train import Trainer
    from memarch_b200.train.ckpt import Checkpointer

    def make(seed):
        torch.manual_seed(seed)
        m = build("tiny", 512)
        eng = ParallelEngine(rank, world, 0, fused=False)
        return m, Trainer(m, TrainConfig(batch=4, micro=4, seq=64, lr=1e-3, warmup=2, steps=10),
                          OptConfig(norm="hs", scale=0.12, rel_every=1), stage="ABX", parallel=eng)

    g = torch.Generator().manual_seed(11 + rank)                          # every rank its own data
    xs = [torch.randint(0, 512, (4, 65), generator=g) for _ in range(6)]
    m, tr = make(0)
    for s in range(3):
        tr.step(xs[s], s)
    ck = Checkpointer(folder, rid="run", rank=rank, world=world)
    ck.save(tr, 3, log=[{"step": 3}], corpus_state={"rank": rank})
    ck.wait()
    dist.barrier()
    want = [float(tr.step(xs[s], s)) for s in range(3, 6)]
    mine = {k: v.detach().clone() for k, v in m.state_dict().items() if k.endswith((".up", ".down"))}
    m2, tr2 = make(5)                                                       # another init: everything comes from the files
    nxt, log = Checkpointer(folder, rid="run", rank=rank, world=world).load(tr2)
    got = [float(tr2.step(xs[s], s)) for s in range(3, 6)]
    same_experts = all(torch.equal(v, m2.state_dict()[k]) for k, v in mine.items())
    files = sorted(os.listdir(folder))
    q.put((rank, nxt, log, want, got, same_experts, files, {k: tuple(v.shape) for k, v in mine.items()}))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_checkpoint_resumes_every_rank_from_its_own_file(tmp_path):
    """Expert-parallel run on 2 gloo ranks: each rank saves its own experts, optimizer state and data position to its
    own file, rank 0 adds the manifest; two freshly initialised ranks resume from those files and continue with the
    same losses and the same expert weights as the uninterrupted run."""
    world, port = 2, 29667
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_w_ckpt, args=(r, world, port, str(tmp_path), q)) for r in range(world)]
    [p.start() for p in ps]
    res = sorted([q.get(timeout=300) for _ in ps], key=lambda t: t[0])
    [p.join(60) for p in ps]
    for rank, nxt, log, want, got, same_experts, files, shapes in res:
        assert nxt == 4 and log == [{"step": 3}]
        assert got == want, (rank, want, got)
        assert same_experts
        assert {"latest.json", "latest.rank0of2.pt", "latest.rank1of2.pt"} <= set(files), files
        assert all(s[0] * world == 4 or s[0] * world == 8 for s in shapes.values()), shapes     # half of the experts each


def _w_chunks(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from memarch_b200.models.moe import AnchorMoE
    from memarch_b200.parallel.engine import NcclExpertExchange
    torch.manual_seed(0)
    moe = AnchorMoE(32, E=4, k_avg=2, k_max=4, budget=True, act="relu2")
    eng = NcclExpertExchange(rank, world)
    moe.ep_shard(rank, world, eng)
    moe.train()
    g = torch.Generator().manual_seed(3 + rank)
    x0 = torch.randn(2, 24, 32, generator=g)
    sur = torch.rand(2, 24, generator=g) * 4
    go = torch.randn(2, 24, 32, generator=g)
    res = {}
    s_mean = moe.s_mean.clone()
    for K in (1, 2, 3):
        eng.chunks = K
        moe.s_mean.copy_(s_mean)
        x = x0.clone().requires_grad_(True)
        moe.up.grad = moe.down.grad = moe.router.weight.grad = None
        y = moe(x, sur)
        y.backward(go)
        res[K] = [t.detach().clone().numpy() for t in (y, x.grad, moe.up.grad, moe.down.grad, moe.router.weight.grad)]
    from memarch_b200.parallel import engine
    q.put((rank, res, len(engine._IN_FLIGHT)))
    dist.barrier()
    dist.destroy_process_group()


def test_chunked_expert_exchange_equals_the_single_exchange():
    """K-chunk pipelined expert exchange (exchange of slice k+1 in flight under the FFN of slice k, forward and
    backward): outputs and every gradient equal the one-exchange form for K = 2 and 3; nothing is left in flight."""
    world, port = 2, 29671
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_w_chunks, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in ps]
    res = [q.get(timeout=180) for _ in ps]
    [p.join(30) for p in ps]
    for _, r, left in res:
        assert left == 0
        for K in (2, 3):
            for a, b in zip(r[1], r[K]):
                assert np.abs(a - b).max() < 1e-6 * max(1.0, np.abs(a).max()), K
