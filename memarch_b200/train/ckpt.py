"""Checkpoint / resume.

File format is the reference's `latest.pt` (fastloop.py:713-766): `{step, log, banks, model, opt, corpus}` where
`banks` lists the frozen expert ids of every bank layer (re-applied *before* the weights are loaded, because the
layout decides which tensors exist), `model` is the CPU state_dict, `opt` the optimizer blob (every tensor /
list-of-tensors / scalar attribute) and `corpus` the data position.  Two additions: `run_id`, a hash of the model
name and shape-defining settings that refuses a foreign checkpoint (train_tpu.py:371-392), and `rng`.

Writing never blocks the step longer than the device->pinned-host copy: `Checkpointer.save` snapshots into reusable
pinned buffers on a side stream, then a writer thread serialises to `latest.pt.tmp`, fsyncs and `os.replace`s it, so a
kill at any moment leaves either the previous or the new complete file (ckpt.py:134-192 of the reference's JAX port
has the same snapshot-then-write split).  `keep > 0` also keeps `step_<n>.pt` hard links of the last `keep` saves.

Several ranks: a rank's state is not the whole state (it holds its own experts, their momentum and its own data
position), so every rank writes its own file `latest.rank<r>of<W>.pt` (the single-rank file keeps the reference's name
and layout) and rank 0 adds `latest.json` = {step, world}.  On resume every rank loads its own file and the ranks
agree on the step (one tiny all-reduce) before anything is restored; files of another world size are refused.
"""
from __future__ import annotations

import hashlib
import json
import os
import threading

import torch


def run_id(name, model_cfg=None, extra=None):
    """Short hash naming a run: checkpoints of another model / width / vocabulary are refused on resume."""
    import dataclasses
    blob = {"name": name, "extra": extra}
    if model_cfg is not None:
        c = dataclasses.asdict(model_cfg) if dataclasses.is_dataclass(model_cfg) else dict(model_cfg)
        blob["cfg"] = {k: c[k] for k in sorted(c) if k in ("d", "vocab", "heads", "light_a", "light_b", "heavy", "final",
                                                           "n_exp", "moe", "bank", "moe_act", "window", "seg")}
    return hashlib.sha1(json.dumps(blob, sort_keys=True, default=str).encode()).hexdigest()[:12]


def bank_layout(model):
    return [list(b.Fz) for b in getattr(model, "heavy", []) if hasattr(b, "Fz")]


def _opt_blob(opt):
    if hasattr(opt, "plist"):                         # Instinct: attribute blob (reference layout)
        return opt.state_dict()
    return {"torch_optim": opt.state_dict()}


def _opt_restore(opt, blob):
    if "torch_optim" in blob:
        opt.load_state_dict(blob["torch_optim"])
    else:
        opt.load_state_dict(blob)


class _PinnedSnapshot:
    """Reusable pinned host buffers keyed by name; `take` copies device tensors into them on a side stream."""

    def __init__(self):
        self.buf = {}
        self.stream = None

    def _host(self, key, t):
        b = self.buf.get(key)
        if b is None or b.shape != t.shape or b.dtype != t.dtype:
            b = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=t.is_cuda)
            self.buf[key] = b
        return b

    def take(self, tree, prefix=""):
        if torch.is_tensor(tree):
            h = self._host(prefix, tree)
            h.copy_(tree.detach(), non_blocking=True)
            return h
        if isinstance(tree, dict):
            return {k: self.take(v, f"{prefix}/{k}") for k, v in tree.items()}
        if isinstance(tree, (list, tuple)):
            return [self.take(v, f"{prefix}/{i}") for i, v in enumerate(tree)]
        return tree


class FileStore:
    """Second home of the checkpoints (another disk or a mounted bucket): `step_XXXXXXXX.pt` plus a small
    `step_XXXXXXXX.json` tag with the run id, both written as `.tmp` and renamed, the tag last, so that a copy is
    either complete and tagged or ignored.  Copies of another run are never taken and never deleted
    (memarch_jax/memarch_jax/train_tpu.py:464-673, 686)."""

    def __init__(self, root, rid=None, keep=2):
        self.root, self.rid, self.keep = root, rid, keep
        os.makedirs(root, exist_ok=True)

    def _tag(self, step):
        return os.path.join(self.root, f"step_{int(step):08d}.json")

    def _blob(self, step):
        return os.path.join(self.root, f"step_{int(step):08d}.pt")

    def steps(self, mine=True):
        """Steps with a complete copy, oldest first; `mine` keeps the copies of this run only."""
        out = []
        for f in sorted(os.listdir(self.root)):
            if f.startswith("step_") and f.endswith(".json"):
                try:
                    tag = json.load(open(os.path.join(self.root, f)))
                except (OSError, ValueError):
                    continue
                if os.path.exists(self._blob(tag["step"])) and (not mine or self.rid is None or tag.get("run_id") == self.rid):
                    out.append(int(tag["step"]))
        return out

    def put(self, path, step):
        import shutil
        tmp = self._blob(step) + ".tmp"
        shutil.copyfile(path, tmp)
        with open(tmp, "rb") as f:
            os.fsync(f.fileno())
        os.replace(tmp, self._blob(step))
        with open(self._tag(step) + ".tmp", "w") as f:
            json.dump({"step": int(step), "run_id": self.rid, "bytes": os.path.getsize(self._blob(step))}, f)
        os.replace(self._tag(step) + ".tmp", self._tag(step))
        if self.keep > 0:
            for old in self.steps()[:-self.keep]:
                os.remove(self._tag(old))                       # tag first: a half-deleted copy is not a copy
                os.remove(self._blob(old))

    def fetch_latest(self, path):
        """Copy this run's newest complete checkpoint to `path`; returns its step or None."""
        import shutil
        have = self.steps()
        if not have:
            return None
        shutil.copyfile(self._blob(have[-1]), path + ".tmp")
        os.replace(path + ".tmp", path)
        return have[-1]


class Checkpointer:
    def __init__(self, directory, rid=None, keep=0, background=True, mirror=None, mirror_keep=2, rank=0, world=1):
        self.dir, self.rid, self.keep, self.background = directory, rid, keep, background
        self.rank, self.world = int(rank), int(world)
        os.makedirs(directory, exist_ok=True)
        if mirror and self.world > 1:
            mirror = os.path.join(mirror, f"rank{self.rank}of{self.world}")     # one mirrored series per rank
        self.store = FileStore(mirror, rid, mirror_keep) if mirror else None
        self.snap = _PinnedSnapshot()
        self.thread = None
        self.error = None

    @property
    def path(self):
        if self.world > 1:
            return os.path.join(self.dir, f"latest.rank{self.rank}of{self.world}.pt")
        return os.path.join(self.dir, "latest.pt")

    @property
    def manifest(self):
        return os.path.join(self.dir, "latest.json")

    # ---------------------------------------------------------------------------------------------- save
    def _device_state(self, trainer):
        opt = trainer.opt
        if hasattr(opt, "plist"):
            o = {k: v for k, v in vars(opt).items() if k not in opt._SKIP and
                 (torch.is_tensor(v) or (isinstance(v, list) and all(t is None or torch.is_tensor(t) for t in v)) or
                  isinstance(v, (int, float, bool, str)) or v is None)}
            o["_lr"] = [g["lr"] for g in opt.param_groups]      # one rate per parameter group, as the reference stores it
        else:
            o = {"torch_optim": opt.state_dict()}
        return {"model": dict(trainer.model.state_dict()), "opt": o}

    def save(self, trainer, step, log=(), corpus_state=None, extra=None):
        """Snapshot now, write in the background.  Returns after the device->host copies are enqueued and the previous
        write (if still running) has finished; the writer waits for the copies before serialising."""
        self.wait()
        dev_state = self._device_state(trainer)
        cuda = trainer.device.type == "cuda"
        if cuda:
            if self.snap.stream is None:
                self.snap.stream = torch.cuda.Stream()
            self.snap.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.snap.stream):
                host = self.snap.take(dev_state)
                done = torch.cuda.Event()
                done.record(self.snap.stream)
            torch.cuda.current_stream().wait_stream(self.snap.stream)   # weights must not change under the copy
        else:
            host, done = self.snap.take(dev_state), None         # own buffers: the previous write has finished (wait above)
        st = {"step": int(step), "log": list(log), "banks": bank_layout(trainer.model), "model": host["model"],
              "opt": host["opt"], "corpus": corpus_state, "run_id": self.rid, "extra": extra,
              "rng": {"cpu": torch.get_rng_state()}, "rank": self.rank, "world": self.world}

        def write():
            try:
                if done is not None:
                    done.synchronize()
                tmp = self.path + ".tmp"
                with open(tmp, "wb") as f:
                    torch.save(st, f)
                    f.flush()
                    os.fsync(f.fileno())
                os.replace(tmp, self.path)
                if self.world > 1 and self.rank == 0:
                    with open(self.manifest + ".tmp", "w") as f:
                        json.dump({"step": int(step), "world": self.world, "run_id": self.rid}, f)
                    os.replace(self.manifest + ".tmp", self.manifest)
                if self.keep > 0:
                    hist = os.path.join(self.dir, f"step_{int(step):08d}" + (f".rank{self.rank}of{self.world}" if self.world > 1 else "") + ".pt")
                    if os.path.exists(hist):
                        os.remove(hist)
                    os.link(self.path, hist)
                    tail = (f".rank{self.rank}of{self.world}.pt" if self.world > 1 else ".pt")
                    old = sorted(f for f in os.listdir(self.dir) if f.startswith("step_") and f.endswith(tail)
                                 and (self.world > 1 or ".rank" not in f))
                    for f in old[:-self.keep]:
                        os.remove(os.path.join(self.dir, f))
                if self.store is not None:
                    self.store.put(self.path, step)
            except BaseException as e:   # noqa: BLE001 - re-raised on the training thread by wait()
                self.error = e

        if self.background:
            self.thread = threading.Thread(target=write, daemon=False)
            self.thread.start()
        else:
            write()
            self.wait()

    def wait(self):
        if self.thread is not None:
            self.thread.join()
            self.thread = None
        if self.error is not None:
            e, self.error = self.error, None
            raise RuntimeError("checkpoint write failed") from e

    # ---------------------------------------------------------------------------------------------- load
    def load(self, trainer, corpus=None, strict_run=True):
        """Resume from `latest.pt` if present.  Returns (next step, log); (first step, []) when there is nothing."""
        if not os.path.exists(self.path) and self.store is not None:
            self.store.fetch_latest(self.path)                   # local disk lost: take this run's newest mirrored copy
        st = torch.load(self.path, map_location="cpu", weights_only=False) if os.path.exists(self.path) else None
        if self.world > 1:
            # all ranks resume from the same step or none does: a rank whose file is missing or older (killed between
            # two ranks' writes) must not pair with ranks that are a save ahead
            import torch.distributed as dist
            mine = int(st["step"]) if st is not None else -1
            if st is not None and int(st.get("world", self.world)) != self.world:
                raise RuntimeError(f"checkpoint {self.path} was written by {st.get('world')} ranks, this run has {self.world}")
            dev = trainer.device if trainer.device.type == "cuda" else torch.device("cpu")
            lo, hi = torch.tensor([mine], device=dev), torch.tensor([mine], device=dev)
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            if int(lo) != int(hi):
                raise RuntimeError(f"ranks disagree on the checkpoint step (between {int(lo)} and {int(hi)}; -1 = no file): "
                                   f"remove the newer files or restore the missing ones in {self.dir}")
        if st is None:
            return 1, []
        if strict_run and self.rid is not None and st.get("run_id") not in (None, self.rid):
            raise RuntimeError(f"checkpoint {self.path} belongs to run {st.get('run_id')}, this run is {self.rid}")
        restore(trainer, st, corpus)
        return st["step"] + 1, st.get("log", [])


def restore(trainer, st, corpus=None):
    """Apply a loaded checkpoint dict: bank layout first, then weights, optimizer, data position."""
    banks = [b for b in getattr(trainer.model, "heavy", []) if hasattr(b, "Fz")]
    changes = []
    for b, fz in zip(banks, st.get("banks", [])):
        if fz and sorted(fz) != sorted(b.Fz):
            fz = set(fz)
            changes += b.rebank([e in fz for e in range(b.E)])
    if changes:
        trainer._apply_rebank(changes)
    trainer.model.load_state_dict(st["model"])
    if st.get("opt") is not None and hasattr(trainer, "opt"):
        _opt_restore(trainer.opt, st["opt"])
    if st.get("corpus") is not None and corpus is not None:
        corpus.load_state_dict(st["corpus"])
    if st.get("rng"):
        torch.set_rng_state(st["rng"]["cpu"])
