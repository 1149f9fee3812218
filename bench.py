"""Headline benchmark: training throughput of the 2.25 B anchor-MoE model `Fv2moeK8h8d2048` at 32 768 tokens per
GPU per step (batch 32 x seq 1024, bf16, Instinct optimizer stepping inside backward), on N GPUs of one node.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 10 --warmup 3
    python bench.py --impl reference ...        # the unmodified reference from baseline/_ref, same metric and config

Prints ONE JSON line from rank 0.  `value` is whole-job tokens/s timed on the device (CUDA events, max over ranks);
`e2e` is the same metric through the public API with the per-step host->device copy of the batch from pinned memory
and a device->host read of the loss inside the timed region.  Data: synthetic seeded Markov/Zipf tokens; weights:
random init + phrasebook artefacts built from that synthetic corpus.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MODEL = "Fv2moeK8h8d2048"
BATCH, SEQ, VOCAB, PHR_V, D_MODEL = 32, 1024, 50304, 50257, 2048
BASELINE_TOK_S = 32768 / 0.448          # the reference's published 448 ms/step on 1x RTX PRO 6000 (README.md:26)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--seq", type=int, default=SEQ)
    ap.add_argument("--mode", default="fused", choices=["fused", "nccl"], help="multi-GPU: fused kernels or NCCL-only")
    ap.add_argument("--art", default=os.environ.get("MEMARCH_ART", os.path.join(tempfile.gettempdir(), "memarch_art")))
    ap.add_argument("--corpus-tokens", type=int, default=8_000_000)
    ap.add_argument("--phrase-k", type=int, default=262144)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--graph", type=int, default=0, help="replay the step as a CUDA graph after 3 eager steps (0 = eager)")
    ap.add_argument("--wave", type=int, default=0, help="frozen bank experts per layer added to the 8 learning ones")
    ap.add_argument("--mem", action="store_true", help="keep the card memory and re-reading on (the headline recipe has NO_MEM=1)")
    ap.add_argument("--config", type=int, default=2, choices=[1, 2, 3, 4],
                    help="benchmark configuration: 2 = the headline 2.25 B anchor-MoE model (default); 1 = dense ~300 M "
                         "model with card memory; 3 = config 2 with 40 frozen bank experts per layer (wave training); "
                         "4 = long context, 16 384-token texts with memory, re-reading and anchor MoE")
    a = ap.parse_args()
    if a.config == 1:
        a.model, a.mem = "dense_v2_300m", True
    elif a.config == 3:
        a.wave = a.wave or 40
    elif a.config == 4:
        a.model, a.batch, a.seq, a.mem = "longctx_1024", 4, 16384, True
    if a.graph:
        # one graph is captured after three eager steps and a second one at the first step that also measures
        # |g|/|w| (every 8th step of the recipe): both captures must fall into the warm-up
        a.warmup = max(a.warmup, 10)
    return a


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                p = [s.strip() for s in line.split(",")]
                if len(p) < 9 or not p[1].replace(".", "").isdigit():
                    continue
                sm.append(float(p[1])); mx.append(float(p[2]))
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ artefacts
def build_artifacts(art, d, n_tokens, phrase_k, device, rank, world):
    """Seeded synthetic corpus + phrasebook artefacts (rank 0 builds, the others wait for the marker file)."""
    import numpy as np
    import torch
    tag = os.path.join(art, f"d{d}_n{n_tokens}_k{phrase_k}")
    done = os.path.join(tag, "COMPLETE")
    if rank == 0 and not os.path.exists(done):
        from memarch_b200.data import phrasebook
        from memarch_b200.data.synth import MarkovCorpus
        os.makedirs(tag, exist_ok=True)
        t0 = time.time()
        toks = MarkovCorpus(vocab=PHR_V, seed=0).stream(n_tokens, text_len=2048, seed=1)
        np.save(os.path.join(tag, "tokens.npy"), toks.astype(np.int32))
        cnt = phrasebook.token_counts(toks, VOCAB)
        np.save(os.path.join(tag, "token_counts.npy"), cnt)
        ph = phrasebook.bigram_init(toks, d, PHR_V, device=device)
        torch.save({k: v.cpu() for k, v in ph.items()}, os.path.join(tag, "bigram.pt"))
        tg = phrasebook.phrase_table(toks, ph["head"], phrase_k, PHR_V, device=device)
        torch.save({k: v.cpu() for k, v in tg.items()}, os.path.join(tag, "trigram.pt"))
        torch.save(phrasebook.lock_trust(toks, VOCAB, cnt, device=device).cpu(), os.path.join(tag, "lock_trust.pt"))
        open(done, "w").write(f"{time.time() - t0:.1f}s")
        print(f"[bench] artefacts built in {time.time() - t0:.1f}s -> {tag}", file=sys.stderr, flush=True)
    t0 = time.time()
    while not os.path.exists(done):
        time.sleep(1.0)
        if time.time() - t0 > 1800:
            raise RuntimeError("artefacts were not built in time")
    return tag


def model_width(name):
    """Width of a registry model (the phrasebook artefacts are built for it); the headline model's width otherwise."""
    try:
        from memarch_b200.config import preset
        return int(preset(name, VOCAB, {}).d)
    except Exception:   # noqa: BLE001 - plain transformer names and legacy models carry no phrasebook
        return D_MODEL


def recipe_env(tag):
    """The reference's published 2.25 B recipe (scripts/g4_1b_b.py:5-8) with artefacts from `tag`."""
    return {
        "FUSED": "ours", "BF16_EXPERTS": "1", "MOE_ACT": "relu2", "LR_SCHED": "wsd", "WSD_FRAC": "0.5", "WARMUP": "50",
        "OPT_KW": json.dumps({"norm": "hs", "scale": 0.12, "m_bf16": True, "rel_every": 8}),
        "PHRASE_INIT": os.path.join(tag, "bigram.pt"), "PHRASE3": os.path.join(tag, "trigram.pt"), "SURP_PHRASE": "1",
        "NO_MEM": "1", "INDUCT": "lock", "LOCK_TRUST": os.path.join(tag, "lock_trust.pt"), "INDUCT_IN": "1",
        "INDUCT_MIX": "1", "WAVE_WARM": "1000000", "TOKEN_COUNTS": os.path.join(tag, "token_counts.npy"),
        "VOCAB": str(VOCAB), "PHR_V": str(PHR_V),
    }


def dist_setup(args):
    import torch
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        import datetime
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if not dist.is_initialized():
            dist.init_process_group("nccl", timeout=datetime.timedelta(minutes=30), device_id=torch.device("cuda", local))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}"
    return rank, world, local


def timed_loop(step_fn, steps, warmup, world, sampler=None):
    """W untimed steps, then exactly K steps between CUDA events, barrier + synchronize on both sides, max over ranks."""
    import torch
    import torch.distributed as dist
    for s in range(warmup):
        step_fn(s)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(warmup, warmup + steps):
        step_fn(s)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item() / steps, clocks


def emit(args, impl, world, ms, e2e, clocks, launches, info):
    """One JSON line.  `config` holds only what defines the measured problem (the same keys and values in both
    arms); everything descriptive (mode, losses, kernel status, self-test errors, memory) goes to `info`."""
    tok = args.batch * args.seq * world
    value = tok / (ms / 1e3)
    out = {"metric": "train_tokens_per_sec", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3), "higher_is_better": True,
           "scaling": "weak", "vs_baseline": round(value / BASELINE_TOK_S, 3), "dtype": "bf16",
           "data": "synthetic (seed-0 order-1 Markov chain, Zipf(1.1) marginal, 10% copies); random-init weights + "
                   "phrasebook artefacts built from the synthetic corpus",
           "impl": impl,
           "config": {"model": args.model, "benchmark_config": args.config, "global_batch": args.batch * world,
                      "seq_len": args.seq, "tokens_per_gpu_per_step": args.batch * args.seq,
                      "parallelism": f"dp{world}+ep{world}" if world > 1 else "single",
                      "wave_frozen_experts": args.wave, "memory": bool(args.mem),
                      "l2": "per-step working set (activations + weights) far exceeds the 126 MB L2"},
           "info": info, "clocks": clocks, "gpu_launches": launches}
    if e2e is not None:
        out["e2e"] = e2e
    print_json(out)


# ------------------------------------------------------------------------------------------------ our arm
def run_ours(args):
    import numpy as np
    import torch
    rank, world, local = dist_setup(args)
    dev = torch.device("cuda", local)
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.config import opt_from_env, train_from_env
    from memarch_b200.data.synth import HostFeeder, TokenStore
    from memarch_b200.ops import _ext
    from memarch_b200.train import Trainer
    _ext.load(required=True)
    tag = build_artifacts(args.art, model_width(args.model), args.corpus_tokens, args.phrase_k, dev, rank, world)
    env = recipe_env(tag)
    if args.mem:
        env.pop("NO_MEM", None)
    torch.manual_seed(0)
    with torch.device(dev):                      # parameters are created on the GPU (same seed on every rank)
        model = build(args.model, VOCAB, env=env)
    if args.wave:
        for b in model.heavy:
            b.grow_bank(args.wave)
    model = model.to(dev)
    ocfg = opt_from_env(OptConfig(lr=6e-4), env)
    tcfg = train_from_env(TrainConfig(name=args.model, stage="ABX", steps=2000, batch=args.batch, micro=args.batch,
                                      seq=args.seq, lr=6e-4, read_cost=0.01), env)
    parallel = None
    selftest = None
    if world > 1:
        from memarch_b200.parallel import ParallelEngine
        parallel = ParallelEngine(rank, world, local, fused=args.mode == "fused")
        if parallel.init_fused() is not None:
            # the peer paths are checked on this set of GPUs before the run; if anything is off, the run uses NCCL
            ok, why = parallel.fused_impl.selftest()
            selftest = dict(parallel.fused_impl.selftest_errors, ok=ok)
            if not ok:
                print(f"[bench] rank {rank}: fused self-test failed ({why}); using the NCCL mode", file=sys.stderr, flush=True)
                args.mode = "nccl"
                parallel = ParallelEngine(rank, world, local, fused=False)
    tr = Trainer(model, tcfg, ocfg, stage="ABX", parallel=parallel, graph=bool(args.graph))
    toks = np.load(os.path.join(tag, "tokens.npy"))
    store = TokenStore(toks, seed=1 + rank, device=dev)
    losses = []

    def step_dev(s):
        losses.append(tr.step(store.batch(args.batch, args.seq), s))

    n0, f0 = _ext.launch_count, _ext.gemm_flops
    sampler = ClockSampler(local) if rank == 0 else None
    ms, clocks = timed_loop(step_dev, args.steps, args.warmup, world, sampler)
    per_step_launches = (_ext.launch_count - n0) / (args.steps + args.warmup)
    # tensor-core work of this package's own GEMMs per step and GPU (nominal 2MNK; attention and the optimizer's
    # element-wise work are not in it), against the measured sustained cuBLAS rate when the driver wrote one
    gemm_tflop = (_ext.gemm_flops - f0) / (args.steps + args.warmup) / 1e12
    peak = None
    try:
        peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("bf16_tflops_sustained") or 0) or None
    except (OSError, ValueError, AttributeError):
        pass
    e2e = None
    if not args.no_e2e:
        feeder = HostFeeder(toks, seed=100 + rank, device=dev, B=args.batch, T=args.seq)
        host_loss = []

        def step_e2e(s):
            xy = feeder.next()                       # pinned host memory -> device, this step's inputs
            loss = tr.step(xy, args.warmup + args.steps + s)
            host_loss.append(loss.item())            # device -> host read of the step's result

        ms2, _ = timed_loop(step_e2e, args.steps, 1, world)
        e2e = {"value": round(args.batch * args.seq * world / (ms2 / 1e3), 1), "unit": "tokens/s",
               "ms_per_step": round(ms2, 3), "h2d_bytes_per_step": feeder.bytes_per_batch, "d2h_bytes_per_step": 4,
               "last_loss": host_loss[-1]}
    st = _ext.C().gemm_status(local)
    peer_st = int(_ext.C().peer_status_read()) if parallel is not None and parallel.fused_impl is not None else 0
    if st or peer_st:
        raise RuntimeError(f"a bounded device wait ran out during the benchmark (GEMM status {st}, peer status {peer_st})")
    if rank == 0:
        first, last = float(losses[0]), float(losses[-1])
        emit(args, "ours", world, ms, e2e, clocks, int(per_step_launches * args.steps),
             {"parallel_detail": "replicated weights + expert parallel" if world > 1 else "single",
              "mode": args.mode if world > 1 else "single", "selftest": selftest,
              "loss_first": round(first, 4), "loss_last": round(last, 4), "kernel_status": st, "peer_status": peer_st,
              "losses": [round(float(l), 4) for l in losses[:16]],
              "gemm_tflop_per_step": round(gemm_tflop, 2),
              "gemm_tflops_achieved": round(gemm_tflop / (ms / 1e3), 1),
              "gemm_share_of_measured_sustained": round(gemm_tflop / (ms / 1e3) / peak, 3) if peak else None,
              "launches_per_step": round(per_step_launches, 1), "cuda_graph": bool(args.graph) and not tr._graph_failed,
              "params_b": round(sum(p.numel() for p in model.parameters()) / 1e9, 3),
              "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
              "stats": {k: round(float(v), 4) for k, v in model.stats.items()}})
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------ reference arm
def run_reference(args):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.exists(os.path.join(ref_dir, "fastloop.py")):
        print_json({"impl": "reference", "unavailable": "baseline/_ref/fastloop.py not present (reference is a "
                    "flat script tree without packaging metadata; copy the reference checkout there)"})
        return
    try:
        _run_reference(args, ref_dir)
    except Exception as e:   # noqa: BLE001 - the reason goes into the JSON line
        import traceback
        traceback.print_exc()
        if int(os.environ.get("RANK", 0)) == 0:
            print_json({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"})


def _run_reference(args, ref_dir):
    import numpy as np
    import torch
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    tag = build_artifacts(args.art, model_width(args.model), args.corpus_tokens, args.phrase_k, dev, rank, world)
    os.environ.update(recipe_env(tag))
    os.environ["DEVICE"] = "cuda"
    if world > 1:
        os.environ.update({"FSDP": "1", "EP": "1", "MASTER_ADDR": os.environ.get("MASTER_ADDR", "127.0.0.1")})
    # The per-weight compiled optimizer step of the reference (exp_opt.py:386-399) rebuilds `_instinct_step_impl`
    # without its default arguments and raises "missing 2 required positional arguments: 'cs' and 'seed_t'" on
    # torch 2.11; its own OPT_ALL=1 switch (one compiled optimizer program after backward, fastloop.py:342) is the
    # stock path that runs, and is what FSDP forces anyway (fastloop.py:307).
    os.environ.setdefault("OPT_ALL", "1")
    if os.environ.get("REF_EAGER") == "1":
        os.environ["NO_COMPILE"] = "1"
    cache = os.path.join(tempfile.gettempdir(), "memarch_ref_cache")
    os.environ.setdefault("TORCHINDUCTOR_CACHE_DIR", os.path.join(cache, "inductor"))
    os.environ.setdefault("TRITON_CACHE_DIR", os.path.join(cache, "triton"))
    sys.path.insert(0, ref_dir)
    cwd = os.getcwd()
    os.chdir(ref_dir)
    try:
        import fastloop                                    # the reference's own training loop, unmodified
    finally:
        os.chdir(cwd)
    fastloop.dist_init()
    ns = argparse.Namespace(batch=args.batch, micro=args.batch, seq=args.seq, lr=6e-4, read_cost=0.01, steps=2000)
    tr = fastloop.Trainer(args.model, "ABX", ns)
    toks = np.load(os.path.join(tag, "tokens.npy"))
    data = fastloop.GPUData(toks, seed=1 + rank)
    losses = []

    def step_dev(s):
        losses.append(tr.step(data.batch(args.batch, args.seq), s))

    sampler = ClockSampler(local) if rank == 0 else None
    ms, clocks = timed_loop(step_dev, args.steps, args.warmup, world, sampler)
    e2e = None
    if not args.no_e2e:
        from memarch_b200.data.synth import HostFeeder
        feeder = HostFeeder(toks, seed=100 + rank, device=dev, B=args.batch, T=args.seq)
        host_loss = []

        def step_e2e(s):
            loss = tr.step(feeder.next(), args.warmup + args.steps + s)
            host_loss.append(loss.item())

        ms2, _ = timed_loop(step_e2e, args.steps, 1, world)
        e2e = {"value": round(args.batch * args.seq * world / (ms2 / 1e3), 1), "unit": "tokens/s",
               "ms_per_step": round(ms2, 3), "h2d_bytes_per_step": feeder.bytes_per_batch, "d2h_bytes_per_step": 4,
               "last_loss": host_loss[-1]}
    if rank == 0:
        emit(args, "reference", world, ms, e2e, clocks, 0,
             {"parallel_detail": "FSDP2 + expert parallel" if world > 1 else "single",
              "mode": ("eager" if os.environ.get("NO_COMPILE") else "torch.compile") + "+OPT_ALL",
              "loss_first": round(float(losses[0]), 4), "loss_last": round(float(losses[-1]), 4),
              "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)})
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


_JSON_FD = None


def _claim_stdout():
    """stdout carries the JSON line only: keep a private copy of the real stdout for it and point descriptor 1 at
    stderr, so that anything a library prints (NCCL's version banner comes through C stdio) lands on stderr."""
    global _JSON_FD
    sys.stdout.flush()
    _JSON_FD = os.dup(1)
    os.dup2(2, 1)


def print_json(obj):
    line = (json.dumps(obj) + "\n").encode()
    if _JSON_FD is None:
        sys.stdout.write(line.decode())
        sys.stdout.flush()
    else:
        os.write(_JSON_FD, line)


if __name__ == "__main__":
    _claim_stdout()
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
