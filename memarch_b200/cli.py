"""Command line: `python -m memarch_b200 <mode> ...`.

  speed          time training steps of (model, stage) pairs, print the SPEED line (fastloop.py `speed`)
  train          full training run with evaluation, checkpoints and guards (fastloop.py `train`)
  bench-kernel   kernel micro-benchmarks with parity and fraction of the measured peaks (bench_fused.py)
  profile        torch.profiler table + device time per kernel family for a few steps (profile_step.py)
  sync-audit     run steps with host-synchronisation warnings on and report where the host waited (sync_audit.py)
  corpus         write the seeded synthetic corpus as shards + phrasebook artefacts (tools/phr/*.py, data/tokenize)
  recipe         the published scale test as one command (scripts/g4_1b_b.py): for the dense comparator and for the
                 anchor-MoE model under the published switches, time the step, derive the number of steps that fills
                 --budget_s seconds of training, then train with evaluations; artefacts come from --out (built on
                 first use); --dry prints the plan and the environment without running

The run shape comes from the flags below, the model from its registry name, everything else from the same
environment switches the reference reads (OPT_KW, MOE_ACT, PHRASE_INIT, ...).
"""
from __future__ import annotations

import argparse
import os
import sys


def parser():
    p = argparse.ArgumentParser(prog="memarch_b200")
    p.add_argument("mode", choices=["speed", "train", "bench-kernel", "profile", "sync-audit", "corpus", "recipe"])
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
    p.add_argument("--budget_s", type=float, default=1500.0, help="recipe: seconds of training per model")
    p.add_argument("--dry", action="store_true", help="recipe: print the plan only")
    return p


RECIPE_MODELS = (("T", "Td2048L16", False), ("ours", "Fv2moeK8h8d2048", True))


def recipe_steps(ms, budget_s):
    """Steps that fill the time budget at `ms` per step: a multiple of 50, at least 500 (scripts/g4_1b_b.py:21)."""
    return max(500, int(budget_s / (ms / 1000.0)) // 50 * 50)


def recipe(args, out=None):
    """Speed run, then training run, for the dense comparator and the anchor-MoE model."""
    import copy
    import json
    from .config import published_recipe_env
    out = out or sys.stdout
    env_file = os.path.join(args.out, "env.json")
    if not os.path.exists(env_file) and not args.dry:
        from .data.phrasebook import write_corpus
        write_corpus(args.out, tokens=args.tokens, d=int(os.environ.get("D_MODEL", 2048)),
                     vocab=int(os.environ.get("VOCAB", 50304)))
    art = json.load(open(env_file)) if os.path.exists(env_file) else {}
    common = {k: v for k, v in published_recipe_env(args.out).items()
              if k in ("FUSED", "BF16_EXPERTS", "MOE_ACT", "LR_SCHED", "WSD_FRAC", "WARMUP", "OPT_KW")}
    plan = []
    for tag, model, ours in RECIPE_MODELS:
        env = dict(common, **{k: v for k, v in art.items() if k in ("VOCAB", "PHR_V", "DATA")})
        if ours:
            env.update(published_recipe_env(args.out))
            env.update(art)
        if args.dry:
            print(f"[recipe] {tag} {model}: speed --stages ABX --batch {args.batch} --warmup 10 --n 10, then train "
                  f"--steps max(500, {args.budget_s:.0f} s / step time) --lr 6e-4\n  env: {json.dumps(env)}", file=out)
            plan.append({"tag": tag, "model": model, "env": env})
            continue
        saved = dict(os.environ)
        os.environ.update({k: str(v) for k, v in env.items()})
        try:
            from .train.loop import speed, train
            a = copy.copy(args)
            a.models, a.stages, a.stage, a.warmup, a.n = [model], ["ABX"], "ABX", 10, 10
            ms = speed(a, args.device, out=out)[-1]["ms"]
            a.steps = recipe_steps(ms, args.budget_s)
            a.eval_every, a.lr = max(50, a.steps // 12 // 50 * 50), 6e-4
            print(f"[recipe] {tag} {model}: {ms:.1f} ms/step -> {a.steps} steps", file=out, flush=True)
            log = train(a, args.device, out=out)[model]
            plan.append({"tag": tag, "model": model, "ms": ms, "steps": a.steps, "log": log})
        finally:
            os.environ.clear()
            os.environ.update(saved)
    return plan


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
    if args.mode == "recipe":
        recipe(args)
        return 0
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
