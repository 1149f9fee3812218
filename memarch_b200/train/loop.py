"""`speed` and `train`: the two run modes of the reference's training script (fastloop.py:580-652, 769-935).

`speed` times steps of one or several (model, stage) pairs on the device and prints the reference's line
`SPEED <name> <stage> <ms>/step <TFLOP/s> MFU <mem> loss <stats>`, also written to `results/speed.json`.
`train` runs the full schedule: data (shard corpus with exact resume, a token file, or the seeded synthetic corpus),
sequence / anchor / panic schedules, batch prefetch with the word-only preparation on a side stream, weight EMA for
evaluation, fixed-window validation, periodic atomic checkpoints, NaN / spike / rollback guards and the hang watchdog.
Between evaluation points nothing reads from the device.
"""
from __future__ import annotations

import json
import math
import os
import sys
import time

import numpy as np
import torch

from ..config import OptConfig, TrainConfig, opt_from_env, train_from_env
from .trainer import Trainer, val_loss


# ------------------------------------------------------------------------------------------------ measurement
def matmul_peak(device, n=8192, iters=20):
    """Measured bf16 GEMM throughput of this GPU in TFLOP/s (fastloop.py:518-533): the MFU denominator."""
    if os.environ.get("PEAK_TFLOPS"):
        return float(os.environ["PEAK_TFLOPS"])
    if torch.device(device).type != "cuda":
        return float("nan")
    a = torch.randn(n, n, device=device, dtype=torch.bfloat16)
    b = torch.randn(n, n, device=device, dtype=torch.bfloat16)
    for _ in range(3):
        a @ b
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        a @ b
    e1.record()
    torch.cuda.synchronize()
    return 2 * n ** 3 * iters / (e0.elapsed_time(e1) * 1e-3) / 1e12


def step_flops(model, batch, seq):
    """Useful FLOPs of one training step (forward + backward = 3 x forward matmul FLOPs), counted from the shapes:
    light / final blocks on every token, heavy layers on the anchor slots only (top-k experts each), both heads,
    causal-window attention.  The reference counts the same with a FLOP-counting mode on the unfused model
    (fastloop.py:536-577); here the count is closed-form so it needs no second copy of the model."""
    if os.environ.get("STEP_FLOPS"):
        return float(os.environ["STEP_FLOPS"])
    c = getattr(model, "cfg", None)
    N = batch * seq
    if c is None:                                            # plain transformer: 6 x params x tokens + attention
        p = sum(q.numel() for n, q in model.named_parameters() if q.dim() >= 2 and "emb" not in n)
        d = model.emb.weight.shape[1]
        L = len(getattr(model, "blocks", []))
        return 6.0 * p * N + 3 * 2 * 2 * L * N * seq * d / 2
    d, V = c.d, c.vocab
    f = 0.0
    blocks = list(model.light_a) + list(model.light_b) + list(model.final)
    for b in blocks:
        lin = sum(p.numel() for n, p in b.named_parameters() if p.dim() == 2)
        f += 2.0 * lin * N
        ctx = min(seq, c.window) if c.window else seq
        f += 2 * 2 * N * d * (ctx / 2 if ctx >= seq else ctx)          # QK^T and PV over the visible keys
    A = max(1, round(seq * c.cap)) * batch
    for h in model.heavy:
        if hasattr(h, "up") and torch.is_tensor(h.up) and h.up.dim() == 3:
            k = getattr(h, "k", 2)
            f += 2.0 * A * k * (h.up.shape[1] * h.up.shape[2] + h.down.shape[1] * h.down.shape[2])
            f += 2.0 * A * d * h.up.shape[0]
        else:
            f += 2.0 * A * sum(p.numel() for p in h.parameters() if p.dim() == 2)
    f += 2.0 * N * d * V                                               # output head
    if hasattr(model, "l_head"):
        f += 2.0 * N * sum(p.numel() for p in model.l_head.parameters() if p.dim() == 2) if not hasattr(model, "sp_lse") else 0
    if hasattr(model, "memory") and not c.no_mem:
        f += 2.0 * N * 6 * d * d / max(1, c.seg // max(1, c.memory.write))
    return 3.0 * f


def make_trainer(name, stage, args, device, env=None, parallel=None):
    """Model by registry name + optimizer and schedule from the environment switches (the reference's Trainer ctor,
    fastloop.py:217-348)."""
    from ..build import build
    env = os.environ if env is None else env
    vocab = int(env.get("VOCAB", 50304))
    torch.manual_seed(int(env.get("SEED", 0)))
    dev = torch.device(device)
    if dev.type == "cuda":
        with torch.device(dev):
            model = build(name, vocab, env=env)
    else:
        model = build(name, vocab, env=env)
    model = model.to(dev)
    ocfg = opt_from_env(OptConfig(lr=args.lr), env)
    tcfg = train_from_env(TrainConfig(name=name, stage=stage, steps=args.steps, batch=args.batch, micro=args.micro,
                                      seq=args.seq, lr=args.lr, read_cost=args.read_cost), env)
    return Trainer(model, tcfg, ocfg, stage=stage, parallel=parallel)


def _time_steps(step_fn, n, device):
    if torch.device(device).type == "cuda":
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for s in range(n):
            step_fn(s)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n
    t0 = time.perf_counter()
    for s in range(n):
        step_fn(s)
    return (time.perf_counter() - t0) * 1e3 / n


def speed(args, device=None, out=None):
    out = out or sys.stdout
    from ..data.synth import MarkovCorpus, TokenStore
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    env = os.environ
    vocab = int(env.get("VOCAB", 50304))
    if env.get("DATA"):
        toks = np.load(env["DATA"], mmap_mode="r")
    else:
        toks = MarkovCorpus(vocab=min(vocab, int(env.get("PHR_V", vocab))), seed=0).stream(max(2_000_000, 4 * args.batch * args.seq), text_len=2048, seed=1)
    peak = matmul_peak(device)
    results = []
    for name in args.models:
        for stage in args.stages:
            tr = make_trainer(name, stage, args, device)
            store = TokenStore(toks, seed=1, device=tr.device)
            if env.get("SPEED_FROZEN") and hasattr(tr.model, "heavy"):
                for b in tr.model.heavy:
                    if hasattr(b, "grow_bank"):
                        b.grow_bank(int(float(env["SPEED_FROZEN"]) * b.E))
            last = {}

            def one(s, tr=tr, store=store, last=last, stage=stage):
                last["loss"] = tr.step(store.batch(args.batch, args.seq), s)
                if stage == "base":                          # the plain loop reads the loss on the host every step
                    last["loss"] = torch.as_tensor(float(last["loss"]))
            for s in range(args.warmup):
                one(s)
            ms = _time_steps(one, args.n, device)
            fl = step_flops(tr.model, args.batch, args.seq)
            tfs = fl / (ms * 1e-3) / 1e12
            mem = torch.cuda.max_memory_allocated() / 2 ** 30 if tr.device.type == "cuda" else 0.0
            stats = "".join(f"  {k} {float(v):.2f}" for k, v in getattr(tr.model, "stats", {}).items()
                            if torch.is_tensor(v) and v.numel() == 1)
            mfu = tfs / peak if peak == peak else float("nan")
            print(f"SPEED {name} {stage}  {ms:.1f} ms/step  {args.batch * args.seq / ms * 1e3:,.0f} tok/s  {tfs:.1f} TFLOP/s  "
                  f"MFU {100 * mfu:.1f}% (of measured {peak:.0f})  mem {mem:.1f} GB  loss {float(last['loss']):.3f}{stats}",
                  file=out, flush=True)
            results.append({"name": name, "stage": stage, "ms": ms, "tflops": tfs, "mfu": mfu, "mem_gb": mem,
                            "loss": float(last["loss"]), "flops_per_step": fl})
            del tr
            if torch.cuda.is_available():
                torch.cuda.empty_cache()
    os.makedirs("results", exist_ok=True)
    json.dump(results, open("results/speed.json", "w"))
    return results


# ------------------------------------------------------------------------------------------------ data for `train`
class _NpyData:
    """Token file: the first 2 M tokens (or the same share of a shorter file) are validation, the rest training."""

    def __init__(self, path_or_array, device, tokens=None):
        from ..data.synth import TokenStore
        allt = np.load(path_or_array, mmap_mode="r") if isinstance(path_or_array, str) else path_or_array
        n_val = min(2_000_000, max(len(allt) // 20, 1))
        self.val, self.train = TokenStore(allt[:n_val], 0, device), TokenStore(allt[n_val:], 1, device)
        self.corpus = None

    def batch(self, B, T):
        return self.train.batch(B, T)

    def state_dict(self):
        return self.train.state_dict()

    def load_state_dict(self, sd):
        self.train.load_state_dict(sd)


class _CorpusData:
    """Shard corpus through the pinned host loader; validation windows come from VAL_NPY, from the held-out tail of
    each source's last shard (HELDOUT_TOK > 0: training never sees it) or from another seed of the same corpus
    (small overlap: a monitoring number, fastloop.py:774-778)."""

    def __init__(self, seq, device, env, rank, world):
        from ..data.loader import HostLoader, ShardCorpus
        from ..data.synth import TokenStore
        w, root = json.loads(env["CORPUS"]), env["CORPUS_ROOT"]
        held = int(env.get("HELDOUT_TOK", 0))           # tail of every source's last shard kept out of training
        self.corpus = ShardCorpus(w, root, seq=seq, seed=int(env.get("CORPUS_SEED", 0)), rank=rank, world=world,
                                  heldout_tok=held)
        if env.get("KINDS"):
            # layer-pool training: every step is one kind of text, KINDS = {"kind": {"source": weight}}; the batch
            # carries its kind and the step's combination of layers (validation stays on the CORPUS mix)
            from ..data.reminders import KindCorpus
            from ..models.fishki import pools
            kinds = json.loads(env["KINDS"])
            sets = pools(len(kinds), int(env["FISH_N"]), int(env.get("FISH_POOL", 17)))
            reseed = int(env.get("DATA_RESEED", -1))         # a control: other documents, the same schedule of kinds and layers
            self.corpus = KindCorpus(kinds, sets, int(env.get("FISH_C", 2)), root, seq=seq,
                                     seed=int(env.get("CORPUS_SEED", 0)), rank=rank, world=world,
                                     doc_seed=reseed if reseed >= 0 else None)
        self.loader, self.device, self.seq = None, device, seq
        if env.get("VAL_NPY"):
            self.val = TokenStore(np.load(env["VAL_NPY"]), 0, device)
        elif held:                                      # validation = exactly the held-out text, every document once
            vc = ShardCorpus(w, root, seq=seq, seed=10 ** 6, heldout_tok=held, split="eval")
            self.val = TokenStore(vc.batch(max(2, min(held, 160 * 1024) // seq)).reshape(-1), 0, device)
        else:
            vc = ShardCorpus(w, root, seq=seq, seed=10 ** 6)
            self.val = TokenStore(vc.batch(max(2, 160 * 1024 // seq)).reshape(-1), 0, device)
        self._B, self._n = None, 0
        self.host_prep = None                            # set by the loop with CPU_PREP=1 (`model.host_prep()`)
        # recall needles written into the training text (REMIND_P > 0): p schedule, optional distance ladder
        self.remind = None
        if float(env.get("REMIND_P", 0) or 0) > 0:
            from ..data.reminders import Reminders
            lad = [int(v) for v in env["REMIND_LADDER"].split(",")] if env.get("REMIND_LADDER") else None
            floats = lambda k: [float(v) for v in env[k].split(",")] if env.get(k) else None
            pack = None
            if env.get("REMIND_PACK") == "1":        # stage one as short episode rows with their own curriculum
                pack = dict(gap=int(env.get("REMIND_PACK_GAP", 0)), round_to=int(env.get("REMIND_PACK_ROUND", 1)),
                            rows_mult=int(env.get("REMIND_PACK_MULT", 1)), frac=floats("REMIND_PACK_FRAC"),
                            win_ref=int(env["REMIND_WIN_REF"]) if env.get("REMIND_WIN_REF") else None,
                            tail=env.get("REMIND_TAIL") == "1", strict=env.get("REMIND_STRICT") == "1",
                            far_frac=float(env["REMIND_FAR_FRAC"]) if env.get("REMIND_FAR_FRAC") else None,
                            far_win=int(env.get("REMIND_FAR_WIN", 2048)), rank=rank)
            mix = (floats("REMIND_MIX"), int(env.get("REMIND_MIX_LEN", 250))) if env.get("REMIND_MIX") else None
            self.remind = Reminders(float(env["REMIND_P"]), seq, n=int(env.get("REMIND_N", 16)),
                                    dist=int(env.get("REMIND_DIST", min(2048, seq // 4))), seed=int(env.get("CORPUS_SEED", 0)),
                                    tok0=int(env.get("REMIND_TOK0", 1000)), V=int(env["VOCAB"]) if env.get("VOCAB") else None,
                                    p0=float(env["REMIND_P0"]) if env.get("REMIND_P0") else None,
                                    warm=int(env.get("REMIND_WARM", 0)), decay=int(env.get("REMIND_DECAY", 0)), ladder=lad,
                                    thr=float(env.get("REMIND_THR", 0.9)), win=int(env.get("REMIND_WIN", 800)),
                                    lag=int(env.get("REMIND_LAG", 5)), doc_eos=self.corpus.eos,
                                    dmin=int(env.get("REMIND_DMIN", 0)), synth=int(env.get("REMIND_SYNTH", 0)),
                                    near=float(env.get("REMIND_NEAR", 0.0)), near_max=int(env.get("REMIND_NEAR_MAX", 0)),
                                    per_row=int(env.get("REMIND_PER_ROW", 1)),
                                    far_log=float(env["REMIND_FAR_LOG"]) if env.get("REMIND_FAR_LOG") else None,
                                    blank=env.get("REMIND_BLANK") == "1", same_fmt=env.get("REMIND_SAME_FMT") == "1",
                                    pack=pack, mix=mix)

    def _xform(self, xy, n):
        extra = None
        if self.remind is not None:
            xy, extra = self.remind(xy, n=n)
        if self.host_prep is not None:                   # token-only preparation on this (the loader's) thread
            import torch
            with torch.no_grad():
                pr = self.host_prep(torch.from_numpy(np.ascontiguousarray(xy[:, :-1], dtype=np.int64)))
            extra = dict(extra or {}, **{"prep_" + k: v.numpy() for k, v in pr.items()})
        return xy, extra

    def batch(self, B, T):
        assert T == self.seq, "the corpus serves windows of one fixed length"
        if self.loader is None or self._B != B:
            if self.loader is not None:
                st = self.loader.state_dict()
                self.loader.close()
                self.corpus.load_state_dict(st)
                self._n = st.get("loader_n", self._n)
            from ..data.loader import HostLoader
            self.loader, self._B = HostLoader(self.corpus, B, device=self.device, first=self._n,
                                              xform=self._xform if (self.remind is not None or self.host_prep is not None) else None), B
        return self.loader.next()

    @property
    def extra(self):
        return self.loader.extra if self.loader is not None else None

    def state_dict(self):
        sd = self.loader.state_dict() if self.loader is not None else dict(self.corpus.state_dict(), loader_n=self._n)
        if self.remind is not None:
            sd = dict(sd, remind=self.remind.state())
        return sd

    def load_state_dict(self, sd):
        if self.loader is not None:
            self.loader.close()
            self.loader = None
        self.corpus.load_state_dict(sd)
        self._n = sd.get("loader_n", 0)
        if self.remind is not None and sd.get("remind"):
            self.remind.load(sd["remind"])


def make_data(args, device, env=None, rank=0, world=1):
    env = os.environ if env is None else env
    if env.get("CORPUS"):
        return _CorpusData(args.seq, device, env, rank, world)
    if env.get("DATA"):
        return _NpyData(env["DATA"], device)
    from ..data.synth import MarkovCorpus
    vocab = int(env.get("VOCAB", 50304))
    n = int(getattr(args, "tokens", 0) or 8_000_000)
    return _NpyData(MarkovCorpus(vocab=min(vocab, int(env.get("PHR_V", vocab))), seed=0).stream(n, text_len=2048, seed=1), device)


# ------------------------------------------------------------------------------------------------ train
def _schedules(args, env, tr):
    ss, au = env.get("SEQ_SCHED"), env.get("AUTO_SCHED")
    s_short, s_frac = (int(ss.split(":")[0]), float(ss.split(":")[1])) if ss else (args.seq, 0.0)
    micro0 = args.micro

    def cfg(step):
        seq = s_short if step <= s_frac * args.steps else args.seq
        fr = cp = None
        if au and hasattr(tr.model, "frac"):
            a_end, a_frac = (float(x) for x in au.split(":"))
            fr, cp = (a_frac, min(1.0, a_frac * 1.25)) if step <= a_end * args.steps else (0.2, 0.25)
        return seq, fr, cp

    def apply(c):
        seq, fr, cp = c
        tr.cfg.micro = micro0 * (args.seq // seq)
        if fr is not None and tr.model.frac != fr:
            tr.model.frac, tr.model.cap = fr, cp
            for b in tr.model.heavy:
                if hasattr(b, "fill"):
                    b.fill = fr / cp
        return seq
    return cfg, apply, micro0


def device_status(tr):
    """Read the status words of the GEMM and peer kernels (host sync); raise if a bounded device wait ran out."""
    from ..ops import _ext
    if tr.device.type != "cuda" or not _ext.available():
        return
    st = _ext.C().gemm_status(tr.device.index or 0)
    if st:
        raise RuntimeError(f"a GEMM kernel gave up a bounded wait (status {st}); results since the last check are not valid")
    par = getattr(tr, "parallel", None)
    if par is not None:
        par.check()


def train(args, device=None, env=None, out=None, parallel=None):
    """Returns {model name: log} where log = [{step, time, val}, ...] (also written to results/<name>_<stage>.json)."""
    from .ckpt import Checkpointer, run_id
    from .guards import NanGuard, RollbackGuard, SpikeLog, Watchdog
    out = out or sys.stdout
    env = os.environ if env is None else env
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    rank, world = int(env.get("RANK", 0)), int(env.get("WORLD_SIZE", env.get("WORLD", 1)))
    from .diag import Diag
    diag = Diag(env, out)
    data = make_data(args, device, env, rank, world)
    diag.phase("data ready")
    bpu = float(env.get("BYTES_PER_UNIT", 4.6361))
    logs = {}
    for name in args.models:
        tr = make_trainer(name, args.stage, args, device, env, parallel)
        diag.phase(f"model {name} and optimizer built")
        if env.get("CPU_PREP") == "1" and hasattr(tr.model, "host_prep") and hasattr(data, "host_prep"):
            if data.loader is not None:                  # a loader started for an earlier model: restart it with the new tables
                st_ = data.state_dict()
                data.load_state_dict(st_)
            data.host_prep = tr.model.host_prep()        # locks, phrase indices and phrase surprise on the loader's thread
        cfg, apply, micro0 = _schedules(args, env, tr)
        log, train_time = [], 0.0
        ck = None
        if env.get("CKPT_DIR"):
            ck = Checkpointer(env["CKPT_DIR"], rid=run_id(name, getattr(tr.model, "cfg", None)), keep=int(env.get("CKPT_KEEP", 0)),
                              mirror=env.get("CKPT_MIRROR") or None, rank=rank, world=world if parallel is not None else 1)
        ck_every = int(env.get("CKPT_EVERY", 0))
        start = 1
        if ck is not None:
            # RESUME_FORCE=1: take a checkpoint written under other run arguments, knowingly
            start, log0 = ck.load(tr, data, strict_run=env.get("RESUME_FORCE") != "1")
            log += log0
            if start > 1:
                print(f"resuming at step {start} from {ck.path}", file=out, flush=True)
        # resume check in two runs (memarch_jax/memarch_jax/train_tpu.py:14-15): A with STOP_AT, CKPT_EVERY, NO_FINAL_CKPT
        # and LOSS_LOG; B in the same CKPT_DIR with STOP_AT and COMPARE=<A's log> prints RESUME_TEST PASS|FAIL for
        # the steps it repeated.  The learning-rate schedule always follows --steps, not STOP_AT.
        last = min(args.steps, int(env.get("STOP_AT", 0)) or args.steps)
        loss_log = open(env["LOSS_LOG"], "a") if env.get("LOSS_LOG") else None
        cmp_ref = None
        if env.get("COMPARE"):
            cmp_ref = {r["step"]: r["loss"] for r in map(json.loads, open(env["COMPARE"]))}
        cmp_n, cmp_max, cmp_tol = 0, 0.0, float(env.get("CMP_TOL", 1e-3))
        # named evaluation sets beside the validation text: EVAL_SETS='{"code": "code_val.npy", ...}' (token arrays);
        # EVAL_ONLY=1 evaluates the checkpoint of CKPT_DIR on all of them and returns without training
        # (memarch_jax/memarch_jax/train_tpu.py: eval sets, --eval_only, --eval_at_resume)
        eval_sets = {}
        if env.get("EVAL_SETS"):
            from ..data.synth import TokenStore
            eval_sets = {k: TokenStore(np.load(v), 0, device) for k, v in json.loads(env["EVAL_SETS"]).items()}

        def run_evals():
            ev_ = {k: float(val_loss(tr.model, st_, args.seq, n=int(env.get("EVAL_BATCHES", 20)))) for k, st_ in eval_sets.items()}
            fish_ = getattr(tr.model, "fish", None)
            if fish_ is not None and env.get("EVAL_NOFISH") == "1":
                # what the layer pool contributes: the same validation with every pool layer's output zeroed
                with torch.no_grad():
                    keep_ = fish_.down.detach().clone()
                    fish_.down.zero_()
                    ev_["val_nofish"] = float(val_loss(tr.model, data.val, args.seq, n=int(env.get("VAL_BATCHES", 20))))
                    fish_.down.copy_(keep_)
            rm_e = getattr(data, "remind", None)
            if rm_e is not None and env.get("REMIND_EVAL") is not None:
                ev_.update(recall_by_distance(tr.model, data.val, args.seq, rm_e, env["REMIND_EVAL"],
                                              getattr(tr.model, "window", args.seq)))
            return ev_
        if env.get("EVAL_ONLY") == "1" or (env.get("EVAL_AT_RESUME") == "1" and start > 1):
            ev = dict(run_evals(), val=float(val_loss(tr.model, data.val, args.seq, n=int(env.get("VAL_BATCHES", 20)))))
            print(f"{name}[{args.stage}]  eval at step {start - 1}: " + "  ".join(f"{k} {v:.4f}" for k, v in ev.items()),
                  file=out, flush=True)
            log.append({"step": start - 1, "eval_only": True, **ev})
            if env.get("EVAL_ONLY") == "1":
                if loss_log is not None:
                    loss_log.close()
                logs[name] = log
                del tr
                continue
        if start > 1 and env.get("FISH_RESET") == "1" and hasattr(tr.model, "fish"):
            # resume with the layer pool back at its initial weights and without optimizer momentum
            from ..models.fishki import FishPool
            old, mc_ = tr.model.fish, tr.model.cfg
            torch.manual_seed(int(env.get("SEED", 0)))
            fresh = FishPool(mc_.d, n=mc_.fish_n, hf=mc_.fish_hf, kinds=mc_.fish_kinds, pool=mc_.fish_pool, center=mc_.fish_center)
            with torch.no_grad():
                for nm in ("up", "down", "norm"):
                    p_ = getattr(old, nm)
                    p_.copy_(getattr(fresh, nm).to(p_))
                    i_ = getattr(tr.opt, "idx", {}).get(id(p_))
                    if i_ is not None:
                        tr.opt.m[i_].zero_()
                        if tr.opt.w[i_] is not None:
                            tr.opt.w[i_].copy_(p_.float())
            print("layer pool reset to its initial weights", file=out, flush=True)
        ramp, text_seen = int(env.get("TEXT_LR_RAMP", 0)), 0
        fish_full = int(env.get("FISH_FULL_FROM", -1))
        if start > 1 and env.get("OPT_RESET_GAIN") == "1" and hasattr(tr.opt, "gain"):
            tr.opt.gain.fill_(1.0)                              # resume with every card's gains back at 1
        rm0 = getattr(data, "remind", None)
        if rm0 is not None and rm0.pack is not None and env.get("REMIND_PACK_LEVEL") and len(rm0.pack.changes) == 1:
            # resume from a checkpoint without the episode curriculum's state: continue from this step of the table
            rm0.pack.changes = [(0, min(int(env["REMIND_PACK_LEVEL"]), len(rm0.pack.steps) - 1))]
        nan = NanGuard(int(env.get("NAN_EVERY", 10)))
        nan_at = int(env.get("TRAIN_NAN_AT", 0))              # inject a non-finite loss at this step (on the host)
        spikes = SpikeLog(float(env.get("SPIKE", 2.0)))
        rb = RollbackGuard(tr, ratio=float(env.get("RB_RATIO", 1.5)), lr_mul=float(env.get("RB_LR", 0.5)),
                           warm=int(env.get("RB_WARM", 50)),
                           kinds=getattr(tr.opt, "K", 1) if getattr(tr.ocfg, "card_by_kind", False) else 1) \
            if env.get("ROLLBACK") == "1" else None
        dog = Watchdog(float(env.get("WATCHDOG", 180)), 120.0) if env.get("WATCHDOG", "180") != "0" else None
        ema_start, ema_beta = float(env.get("EMA_START", 0) or 0), float(env.get("EMA_BETA", 0.98))
        ema_every = int(env.get("EMA_EVERY", 1))
        ema = None
        small = lambda: [p for p in tr.model.parameters() if p.numel() < 10_000_000]
        prefetch = bool(env.get("PREFETCH")) and hasattr(tr.model, "prep") and tr.device.type == "cuda"
        side = torch.cuda.Stream() if prefetch else None

        def fetch(st):
            sq = cfg(st)[0]
            b = data.batch(args.batch * (args.seq // sq), sq)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                pr = [tr.model.prep(mb[:, :-1]) for mb in b.split(micro0 * (args.seq // sq))]
                ev = torch.cuda.Event()
                ev.record(side)
            return b, pr, ev

        def sync():
            """Wait for the device; this is also where the kernels' status words are read (a bounded wait that ran
            out inside a GEMM or a peer barrier means later kernels worked on incomplete data): raises then."""
            if tr.device.type == "cuda":
                torch.cuda.synchronize()
                device_status(tr)
        phase = {"data": 0.0, "enqueue": 0.0, "eval": 0.0, "ckpt": 0.0, "n": 0.0}
        sync()
        t0 = time.time()
        nxt = fetch(start) if prefetch else None
        loss = torch.zeros((), device=tr.device)
        try:
            for step in range(start, last + 1):
                seq = apply(cfg(step))
                diag.step(step)
                if step == start + 1:
                    diag.phase("first step enqueued")
                pn = env.get("PANIC")
                if pn:
                    pfrac, pw = (float(x) for x in pn.split(":"))
                    tr.model.panic = pw if step > (1 - pfrac) * args.steps else 0
                if prefetch:
                    xy_b, preps, ev = nxt
                    torch.cuda.current_stream().wait_event(ev)
                    for pr_ in preps:
                        for v in pr_.values():
                            if torch.is_tensor(v):
                                v.record_stream(torch.cuda.current_stream())
                    if step < last:
                        nxt = fetch(step + 1)
                    loss = tr.step(xy_b, step - 1, preps)
                else:
                    td = time.time()
                    xy_b = data.batch(args.batch * (args.seq // seq), seq)
                    ts = time.time()
                    npreps, lr_mul_ = None, 1.0
                    if fish_full >= 0 and step >= fish_full and hasattr(getattr(data, "corpus", None), "full"):
                        data.corpus.full = True              # last phase: every step runs the whole set of its kind
                    ex_ = getattr(data, "extra", None)
                    mc_ = getattr(tr.model, "cfg", None)
                    if rb is None and ex_ is not None and (
                            "kind" in ex_ or any(k.startswith("prep_") for k in ex_) or ("rem" in ex_ and max(getattr(mc_, "remind_w", 0), getattr(mc_, "remind_use_w", 0)) > 0)):
                        rm_ = getattr(data, "remind", None)
                        synth_ = bool(rm_ is not None and rm_.synth_at(data.loader.n_done - 1))
                        npreps = needle_preps(tr.model, xy_b, ex_, tr.cfg.micro or len(xy_b), synth_)
                        if ramp and rm_ is not None and not synth_:
                            # after the synthetic stage the step on TEXT batches grows from 0 to full over `ramp`
                            # text batches (synthetic batches keep the full step); the count is not checkpointed
                            text_seen += 1
                            lr_mul_ = min(1.0, text_seen / ramp)
                        if "kind" in ex_:
                            tr.card = int(ex_["kind"][0, 0])        # OptConfig.card_by_kind: one card per kind of text
                    ex0_ = getattr(data, "extra", None)
                    if rb is not None and ex0_ is not None and "kind" in ex0_:
                        tr.card = int(ex0_["kind"][0, 0])
                    loss = rb.step(xy_b, step - 1, kind=tr.card or 0) if rb is not None else tr.step(xy_b, step - 1, npreps, lr_mul_)
                    phase["data"] += ts - td
                    phase["enqueue"] += time.time() - ts
                    phase["n"] += 1
                if nan_at and step == nan_at:                       # host-made failure for the guard tests
                    loss = loss * float("nan")
                nan.check(loss)
                if loss_log is not None or cmp_ref is not None:     # one host read per step: a test mode, not a run mode
                    lv = float(loss)
                    if loss_log is not None:
                        loss_log.write(json.dumps({"step": step, "loss": lv}) + "\n")
                        loss_log.flush()
                    if cmp_ref is not None and step in cmp_ref:
                        cmp_n, cmp_max = cmp_n + 1, max(cmp_max, abs(lv - cmp_ref[step]))
                if dog:
                    dog.beat()
                if ema_start and step >= ema_start * args.steps and step % ema_every == 0:
                    with torch.no_grad():
                        ps = small()
                        if ema is None:
                            ema = [p.detach().float().clone() for p in ps]
                        else:
                            torch._foreach_lerp_(ema, [p.detach().float() for p in ps], 1 - ema_beta ** ema_every)
                if step % args.eval_every == 0 or step == last:
                    sync()
                    train_time += time.time() - t0
                    nan.flush()
                    cur = None
                    if ema is not None:
                        with torch.no_grad():
                            ps = small()
                            cur = [p.detach().clone() for p in ps]
                            for p, e in zip(ps, ema):
                                p.copy_(e)
                    te = time.time()
                    vl = float(val_loss(tr.model, data.val, args.seq, n=int(env.get("VAL_BATCHES", 20))))
                    phase["eval"] += time.time() - te
                    if cur is not None:
                        with torch.no_grad():
                            for p, c0 in zip(ps, cur):
                                p.copy_(c0)
                    spikes.check(step, float(loss))
                    extra = "".join(f"  {k} {float(v):.2f}" for k, v in getattr(tr.model, "stats", {}).items()
                                    if torch.is_tensor(v) and v.numel() == 1)
                    extra += "".join(f"  {k} [{' '.join(f'{x:.2f}' for x in v.tolist())}]"       # per-layer statistics
                                     for k, v in getattr(tr.model, "stats", {}).items()
                                     if torch.is_tensor(v) and v.dim() == 1 and 1 < v.numel() <= 64 and k.endswith("_l"))
                    sets = run_evals()
                    hoop = getattr(tr.model, "hoop", None)
                    if hoop is not None and "uroboros_eaten" in tr.model.stats:
                        # the heavy layers' budget steps down one level once enough words are "eaten"
                        st_ = tr.model.stats
                        seen_ = torch.stack([st_["uroboros_eaten"].float(), st_["uroboros_corr"].float()])
                        if parallel is not None and hasattr(parallel, "mean_vector"):
                            seen_ = parallel.mean_vector(seen_.clone())      # every rank must take the same decision:
                        nb = hoop.next_budget(tr.model.hoop_budget, seen_[0], tr.model.cfg.uroboros_levels,   # the budget
                                              corr=seen_[1])                                                # sets shapes
                        if nb != tr.model.hoop_budget:
                            print(f"hoop: budget {tr.model.hoop_budget} -> {nb} (eaten {float(seen_[0]):.2f})",
                                  file=out, flush=True)
                            tr.model.hoop_budget = nb
                    rm = getattr(data, "remind", None)
                    # with several ranks every rank scores (the forward has collectives) and the curriculum moves on the
                    # summed counts, so that all ranks stay on the same level (levels set batch shapes)
                    if rm is not None and data.extra is not None and "rem" in data.extra and (
                            parallel is not None or data.extra["rem"].any()):
                        hits, n_ans = needle_hits(tr.model, xy_b, torch.from_numpy(data.extra["rem"]).to(tr.device) > 0,
                                                  data.extra.get("rem_y"))
                        if parallel is not None and hasattr(parallel, "mean_vector"):
                            tot_ = parallel.mean_vector(torch.tensor([hits, n_ans], device=tr.device)) * parallel.W
                            hits, n_ans = float(tot_[0]), float(tot_[1])
                        if n_ans > 0:
                            sets["needles"] = hits / n_ans
                            msg = rm.observe(data.loader.n_done - 1, hits, n_ans)
                            if msg:
                                print(msg, file=out, flush=True)
                    extra += "".join(f"  {k} {v:.3f}" for k, v in sets.items())
                    log.append({"step": step, "time": train_time, "val": vl, **({"sets": sets} if sets else {})})
                    print(f"{name}[{args.stage}]  step {step:5d}  val {vl:.3f}  bpb {vl / bpu / math.log(2):.4f}  "
                          f"train {float(loss):.3f}{extra}  {train_time / 60:.1f} min", file=out, flush=True)
                    if env.get("DIAG") == "1":                  # host-side phase times since the last report
                        n_ = max(phase["n"], 1)
                        mem = f", device {torch.cuda.max_memory_allocated() / 2 ** 30:.1f} GiB peak" if tr.device.type == "cuda" else ""
                        print(f"[diag] per step: data wait {1e3 * phase['data'] / n_:.2f} ms, step enqueue "
                              f"{1e3 * phase['enqueue'] / n_:.2f} ms; eval {phase['eval']:.2f} s, checkpoint "
                              f"{phase['ckpt']:.2f} s (snapshot only: the write is in the background){mem}", file=out, flush=True)
                        phase = dict.fromkeys(phase, 0.0)
                    sync()
                    t0 = time.time()
                if ck is not None and ck_every and (step % ck_every == 0 or (step == last and env.get("NO_FINAL_CKPT") != "1")):
                    nan.flush()                                  # never save a state that already went non-finite
                    sync()                                       # nor one made after a device wait ran out
                    if parallel is not None:
                        parallel.before_checkpoint()             # rows kept by other ranks come home first
                    tc = time.time()
                    ck.save(tr, step, log, data.state_dict())
                    phase["ckpt"] += time.time() - tc
        finally:
            diag.close()
            if dog:
                dog.close()
            if ck is not None:
                ck.wait()
            if loss_log is not None:
                loss_log.close()
        if cmp_ref is not None:
            ok = cmp_n > 0 and cmp_max <= cmp_tol
            print(f"[train] RESUME_TEST {'PASS' if ok else 'FAIL'}: steps {start}..{last}, {cmp_n} compared, "
                  f"max |d loss| {cmp_max:.3e} (tolerance {cmp_tol:g})", file=out, flush=True)
        if env.get("DUMP_TOK"):
            dump_token_losses(tr.model, data.val, args.seq, env["DUMP_TOK"])
        os.makedirs("results", exist_ok=True)
        json.dump({"log": log}, open(f"results/{name}_{args.stage}.json", "w"))
        logs[name] = log
        del tr
    return logs


@torch.no_grad()
def recall_by_distance(model, store, seq, remind, spec, window, rows=8):
    """Needle accuracy on held-out text with exactly d words between facts and questions, for each d of `spec`
    ("a,b,c"; empty: half the window, the window, twice the window and the farthest that fits the row).  Fixed
    validation windows, every row gets a needle.  -> {"recall_d<d>": accuracy}"""
    room = seq + 1 - 2 * remind.L
    ds = [int(v) for v in spec.split(",") if v] or [window // 2, window, 2 * window, room]
    ds = sorted({d for d in ds if 0 <= d <= room})
    g = torch.Generator(device=store.device).manual_seed(1)
    start = torch.randint(0, len(store.t) - seq - 1, (rows,), device=store.device, generator=g)
    base = store.t[start[:, None] + torch.arange(seq + 1, device=store.device)].cpu().numpy()
    out = {}
    for d in ds:
        xy, ex = remind(base, p=1.0, exact=d)
        xy_t = torch.from_numpy(np.ascontiguousarray(xy)).long().to(store.device)
        hits, n_ans = needle_hits(model, xy_t, torch.from_numpy(ex["rem"]).to(store.device) > 0, ex.get("rem_y"))
        out[f"recall_d{d}"] = hits / max(n_ans, 1.0)
    return out


def needle_preps(model, xy, extra, micro, synth=False):
    """One `prep` dict per micro-batch that carries what the data pipeline knows about the batch as device tensors:
    the needle masks under "remind" (the model's loss reads them) and, with a per-kind corpus, "kind" and "fish".  Where the model has induction locks they are switched off at the question
    positions: the lock "last earlier occurrence of this word -> the word after it" would hand over the answer
    without any memory (memarch_jax/memarch_jax/data.py:333-341 of the reference)."""
    ex = {k: torch.from_numpy(np.ascontiguousarray(v)).to(xy.device, non_blocking=True) for k, v in extra.items()}
    out = []
    for i0 in range(0, len(xy), micro):
        sl = {k: v[i0:i0 + micro] for k, v in ex.items()}
        ready = {k[5:]: v for k, v in sl.items() if k.startswith("prep_")}
        if ready:
            pr = ready                                   # prepared on the loader's thread
        else:
            pr = model.prep(xy[i0:i0 + micro, :-1]) if hasattr(model, "ind_a") and hasattr(model, "prep") else {}
        needles = {k: v for k, v in sl.items() if k.startswith("rem")}
        if needles:
            if "ind_on" in pr:
                pr["ind_on"] = pr["ind_on"] & ~(sl["rem"] > 0)[..., None]
            pr["remind"] = dict(needles, synth=synth)
        for k in ("kind", "fish"):                       # layer pool: the step's kind of text and combination of layers
            if k in sl:
                pr[k] = sl[k]
        out.append(pr)
    return out


@torch.no_grad()
def needle_hits(model, xy, rem, rem_y=None):
    """(hits, answers) on the marked question positions of a training batch: an answer counts when the value gets more
    than half of the probability (it is then certainly the arg-max).  One extra forward without gradient.  `rem_y`:
    the true values where the text shows a blank."""
    was = model.training
    model.eval()
    out, _ = model(xy[:, :-1])
    y = xy[:, 1:]
    if rem_y is not None:
        y = torch.where(rem, torch.as_tensor(rem_y).to(y), y)
    if hasattr(model, "_ce_tok"):
        ce = model._ce_tok(out[0], y).float().view_as(y)
    else:
        V = out.shape[-1]
        ce = torch.nn.functional.cross_entropy(out.float().view(-1, V), y.reshape(-1), reduction="none").view_as(y)
    model.train(was)
    return float((ce[rem] < math.log(2.0)).sum()), float(rem.sum())


@torch.no_grad()
def dump_token_losses(model, store, seq, path, n=20, batch=8):
    """Per-token CE on the validation windows (same windows as `val_loss`), saved as one flat tensor."""
    was = model.training
    model.eval()
    g = torch.Generator(device=store.device).manual_seed(0)
    ces = []
    for _ in range(n):
        start = torch.randint(0, len(store.t) - seq - 1, (batch,), device=store.device, generator=g)
        xy = store.t[start[:, None] + torch.arange(seq + 1, device=store.device)].long()
        out, _ = model(xy[:, :-1])
        if hasattr(model, "_ce_tok"):
            ces.append(model._ce_tok(out[0], xy[:, 1:]).float().flatten())
        else:
            V = out.shape[-1]
            ces.append(torch.nn.functional.cross_entropy(out.float().view(-1, V), xy[:, 1:].reshape(-1), reduction="none"))
    model.train(was)
    torch.save(torch.cat(ces).cpu(), path)
