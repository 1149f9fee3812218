"""Step profiler and host-synchronisation audit.

`profile_steps`: warm steps, then `torch.profiler` over a few steps; prints the top kernels and the device time per
step bucketed by kernel family (own tcgen05 GEMMs / library GEMMs / attention / optimizer / own row kernels /
collectives / copies / other), the view the reference gets from profile_step.py:22-51.
`part_times`: forward, memory pass and re-reading timed separately with CUDA events (prof_long.py:24-49).
`sync_audit`: runs steps with `torch.cuda.set_sync_debug_mode("warn")` and reports every place where the host waited
for the device (sync_audit.py:1-27); the training step of stages A/B/X must report none.
"""
from __future__ import annotations

import os
import sys
import warnings

import torch

BUCKETS = (
    ("own tcgen05 gemm", ("gemm_tc",)),
    ("library gemm", ("gemm", "cutlass", "cublas", "nvjet", "sm90_xmma", "sm100_xmma", "xmma")),
    ("attention", ("attn", "flash", "fmha", "sdpa", "cudnn")),
    ("optimizer", ("instinct",)),
    ("collectives", ("nccl", "peer_", "allreduce", "multimem")),
    ("own row kernels", ("rmsnorm", "relu2", "swiglu", "rope", "ce_rows", "resid_add", "gather_rows", "gather_sum",
                         "row_dot", "anchor_select", "moe_slots", "lock_find")),
    ("copies", ("memcpy", "memset", "copy_", "CatArrayBatchedCopy", "direct_copy")),
)


def bucket_of(name):
    low = name.lower()
    for b, keys in BUCKETS:
        if any(k.lower() in low for k in keys):
            return b
    return "other"


def _setup(args, device):
    from ..data.synth import MarkovCorpus, TokenStore
    from ..train.loop import make_trainer
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    vocab = int(os.environ.get("VOCAB", 50304))
    tr = make_trainer(args.models[0], args.stage, args, device)
    toks = MarkovCorpus(vocab=min(vocab, int(os.environ.get("PHR_V", vocab))), seed=0).stream(max(1_000_000, 4 * args.batch * args.seq), text_len=2048, seed=1)
    return tr, TokenStore(toks, seed=1, device=tr.device)


def profile_steps(args, device=None, steps=5, top=45, out=None):
    out = out or sys.stdout
    from torch.profiler import ProfilerActivity, profile
    tr, store = _setup(args, device)
    for s in range(args.warmup):
        tr.step(store.batch(args.batch, args.seq), s)
    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if tr.device.type == "cuda" else [])
    with profile(activities=acts) as prof:
        for s in range(steps):
            tr.step(store.batch(args.batch, args.seq), args.warmup + s)
        if tr.device.type == "cuda":
            torch.cuda.synchronize()
    key = "self_cuda_time_total" if tr.device.type == "cuda" else "self_cpu_time_total"
    print(prof.key_averages().table(sort_by=key, row_limit=top), file=out)
    sums = {}
    for e in prof.key_averages():
        t = getattr(e, "self_device_time_total", None)
        if t is None:
            t = getattr(e, "self_cuda_time_total", 0.0)
        if tr.device.type != "cuda":
            t = e.self_cpu_time_total
        if t:
            b = bucket_of(e.key)
            sums[b] = sums.get(b, 0.0) + t / 1e3 / steps
    total = sum(sums.values())
    print(f"device time per step by kernel family (ms), total {total:.1f}:", file=out)
    for b, v in sorted(sums.items(), key=lambda kv: -kv[1]):
        print(f"  {b:18s} {v:8.2f}  {100 * v / max(total, 1e-9):5.1f}%", file=out)
    return sums


def part_times(model, xy, n=5):
    """ms of (full forward, memory pass, re-reading) measured separately; {} entries absent when the part is off."""
    dev = xy.device
    cuda = dev.type == "cuda"

    def timed(fn):
        import time
        fn()
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        return (time.perf_counter() - t0) * 1e3 / n
    out = {}
    with torch.no_grad():
        out["forward"] = timed(lambda: model(xy[:, :-1]))
        if hasattr(model, "_memory_pass") and not model.cfg.no_mem:
            h = model.emb(xy[:, :-1]).float()
            out["memory_pass"] = timed(lambda: model._memory_pass(h, model.cfg.seg))
            if hasattr(model, "reread") and not model.cfg.no_reread:
                _, snaps, _ = model._memory_pass(h, model.cfg.seg)
                out["reread"] = timed(lambda: model._reread_pass(h, xy[:, :-1], snaps, model.cfg.seg))
    return out


def sync_audit(args, device=None, steps=3, out=None):
    out = out or sys.stdout
    tr, store = _setup(args, device)
    for s in range(max(args.warmup, 3)):
        tr.step(store.batch(args.batch, args.seq), s)
    if tr.device.type != "cuda":
        print("sync-audit: needs a CUDA device (host synchronisation is a device concept)", file=out)
        return []
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("warn")
    found = []
    try:
        with warnings.catch_warnings(record=True) as w:
            warnings.simplefilter("always")
            for s in range(steps):
                tr.step(store.batch(args.batch, args.seq), 100 + s)
            found = [f"{x.filename}:{x.lineno}: {x.message}" for x in w if "synchroniz" in str(x.message).lower()]
    finally:
        torch.cuda.set_sync_debug_mode("default")
    print(f"sync-audit: {len(found)} host synchronisation(s) in {steps} steps", file=out)
    for f in sorted(set(found)):
        print("  " + f, file=out)
    return found


class LayerDiag:
    """Per-heavy-layer forward / backward device time (the reference's DIAG_LAYER, full2.py:46-112).  The reference
    synchronises between sub-phases, which breaks overlap by design; here CUDA events are recorded on the stream by
    module hooks and read once at `report()`, so the step itself is not disturbed.

        diag = LayerDiag(model); run steps; print(diag.report()); diag.close()
    """

    def __init__(self, model, layers=None):
        self.layers = list(layers if layers is not None else getattr(model, "heavy", []))
        self.ev = {i: {"f": [], "b": []} for i in range(len(self.layers))}
        self.handles = []
        self.cuda = next(model.parameters()).is_cuda
        for i, m in enumerate(self.layers):
            self.handles.append(m.register_forward_pre_hook(self._mark(i, "f", 0)))
            self.handles.append(m.register_forward_hook(self._mark(i, "f", 1)))
            self.handles.append(m.register_full_backward_pre_hook(self._mark(i, "b", 0)))
            self.handles.append(m.register_full_backward_hook(self._mark(i, "b", 1)))

    def _now(self):
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            return e
        import time
        return time.perf_counter()

    def _mark(self, i, which, end):
        def hook(*_):
            lst = self.ev[i][which]
            if end:
                if lst and len(lst[-1]) == 1:
                    lst[-1].append(self._now())
            else:
                lst.append([self._now()])
        return hook

    def report(self):
        if self.cuda:
            torch.cuda.synchronize()
        rows = []
        for i in range(len(self.layers)):
            r = {"layer": i}
            for which, name in (("f", "fwd_ms"), ("b", "bwd_ms")):
                pairs = [p for p in self.ev[i][which] if len(p) == 2]
                if pairs:
                    ms = [(a.elapsed_time(b) if self.cuda else (b - a) * 1e3) for a, b in pairs]
                    r[name] = sum(ms) / len(ms)
            rows.append(r)
        return rows

    def close(self):
        for h in self.handles:
            h.remove()
