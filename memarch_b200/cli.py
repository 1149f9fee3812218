"""Command line: `python -m memarch_b200 <mode> ...`.

  speed          time training steps of (model, stage) pairs, print the SPEED line (fastloop.py `speed`)
  train          full training run with evaluation, checkpoints and guards (fastloop.py `train`)
  bench-kernel   kernel micro-benchmarks with parity and fraction of the measured peaks (bench_fused.py)
  profile        torch.profiler table + device time per kernel family for a few steps (profile_step.py)
  sync-audit     run steps with host-synchronisation warnings on and report where the host waited (sync_audit.py)
  corpus         write the seeded synthetic corpus as shards + phrasebook artefacts (tools/phr/*.py, data/tokenize)

The run shape comes from the flags below, the model from its registry name, everything else from the same
environment switches the reference reads (OPT_KW, MOE_ACT, PHRASE_INIT, ...).
"""
from __future__ import annotations

import argparse
import os
import sys


def parser():
    p = argparse.ArgumentParser(prog="memarch_b200")
    p.add_argument("mode", choices=["speed", "train", "bench-kernel", "profile", "sync-audit", "corpus"])
    p.add_argument("--models", nargs="+", default=["Fv2moeKs8"])
    p.add_argument("--stages", nargs="+", default=["ABX"])
    p.add_argument("--stage", default="ABX")
    p.add_argument("--steps", type=int, default=4000)
    p.add_argument("--batch", type=int, default=32)
    p.add_argument("--micro", type=int, default=0)
    p.add_argument("--seq", type=int, default=1024)
    p.add_argument("--lr", type=float, default=6e-4)
    p.add_argument("--read_cost", type=float, default=0.01)
    p.add_argument("--eval_every", type=int, default=250)
    p.add_argument("--tokens", type=int, default=8_000_000)
    p.add_argument("--warmup", type=int, default=15)
    p.add_argument("--n", type=int, default=30)
    p.add_argument("--device", default=None)
    p.add_argument("--out", default="artefacts")
    return p


def main(argv=None):
    args, rest = parser().parse_known_args(argv)
    if rest and args.mode != "bench-kernel":
        parser().error(f"unrecognised arguments: {rest}")
    if not args.micro:
        args.micro = args.batch
    if args.mode == "bench-kernel":
        from .utils import kernel_bench
        return kernel_bench.main(rest)
    if args.mode == "corpus":
        from .data.phrasebook import write_corpus
        return write_corpus(args.out, tokens=args.tokens, d=int(os.environ.get("D_MODEL", 256)),
                            vocab=int(os.environ.get("VOCAB", 50304)))
    parallel = None
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world > 1:
        from .parallel import ParallelEngine, init_distributed
        rank, world, local = init_distributed()
        parallel = ParallelEngine(rank, world, local, fused=os.environ.get("MEMARCH_MODE", "fused") == "fused")
        args.device = f"cuda:{local}"
    if args.mode == "speed":
        from .train.loop import speed
        speed(args, args.device)
    elif args.mode == "train":
        from .train.loop import train
        train(args, args.device, parallel=parallel)
    elif args.mode == "profile":
        from .utils.profile import profile_steps
        profile_steps(args, args.device)
    elif args.mode == "sync-audit":
        from .utils.profile import sync_audit
        sync_audit(args, args.device)
    return 0


if __name__ == "__main__":
    sys.exit(main())
