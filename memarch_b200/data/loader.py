"""Resumable weighted-mix shard corpus and a pinned-memory host loader with exact resume state.

Shard layout follows the reference (data/loader.py:1-193): `<root>/<source>/<name>.u32.zst` holds uint32 tokens of
whole documents, each ending in the end-of-text id; beside it optional `<name>.drop.npy` / `<name>.cdrop.npy`
(document numbers to skip: dedup and benchmark decontamination), `<name>.score.npy` (code quality 0-5 -> repeats:
>= 3.0 three times, 2.5-3.0 once, below that one document in four) and `<name>.json` (manifest with `eos`).
Uncompressed shards `<name>.u32.npy` / `<name>.u32` are accepted as well, so the loader works where the
`zstandard` module is not installed.

Sources are mixed deterministically by token share (the source furthest below its target share goes next), documents
are concatenated into windows of `seq + 1` tokens, and the position (epoch, shard, document, offset per source; tokens
taken per source; the leftover buffer) round-trips through `state_dict()` so a killed run continues from the same
token.  With several ranks each takes shards `i % world == rank`.

`HostLoader` (the reference's JAX port keeps one in data.py:257-316) runs the corpus on a worker thread, stages each
batch in pinned memory and tags it with the corpus state *after* that batch, so a checkpoint taken at step k resumes
with the batch of step k + 1 even though the thread has read ahead.  Worker exceptions surface on the consumer.
"""
from __future__ import annotations

import json
import os
import queue
import threading

import numpy as np

SHARD_EXTS = (".u32.zst", ".u32.npy", ".u32")
MASK_EXTS = (".drop.npy", ".cdrop.npy", ".score.npy")


def _shard_names(root, src):
    names = set()
    for f in os.listdir(os.path.join(root, src)):
        for e in SHARD_EXTS:
            if f.endswith(e):
                names.add(f[:-len(e)])
    return sorted(names)


def _read_tokens(base):
    if os.path.exists(base + ".u32.zst"):
        try:
            import zstandard
        except ImportError as e:                                    # noqa: F841
            raise RuntimeError(f"{base}.u32.zst needs the zstandard module; store the shard as .u32.npy instead")
        return np.frombuffer(zstandard.ZstdDecompressor().decompress(open(base + ".u32.zst", "rb").read()), dtype=np.uint32)
    if os.path.exists(base + ".u32.npy"):
        return np.load(base + ".u32.npy", mmap_mode="r").astype(np.uint32, copy=False)
    return np.fromfile(base + ".u32", dtype=np.uint32)


def heldout_tail(lens, tok):
    """How many trailing documents of a shard are held out: enough for `tok` tokens, at most a tenth of the shard,
    at least one (memarch_jax/memarch_jax/train_tpu.py:316-330)."""
    n, k, acc = len(lens), 0, 0
    while k < max(1, n // 10) and acc < tok:
        acc += int(lens[n - 1 - k])
        k += 1
    return k


def shard_documents(base, eos, rng, held=None):
    """Documents of one shard after masks and quality repeats, shuffled so that repeats do not sit together.
    `held` = ("train" | "eval", tokens): the held-out tail of the shard is removed (train) or is all that is left,
    every document once (eval)."""
    arr = _read_tokens(base)
    ends = np.flatnonzero(arr == eos) + 1
    starts = np.concatenate([[0], ends[:-1]])
    keep = np.ones(len(ends), dtype=bool)
    if held is not None and len(ends):
        k = heldout_tail(ends - starts, held[1])
        if held[0] == "eval":
            keep[:len(ends) - k] = False
        else:
            keep[len(ends) - k:] = False
    for ext in MASK_EXTS[:2]:
        if os.path.exists(base + ext):
            idx = np.load(base + ext).astype(np.int64)
            keep[idx[idx < len(keep)]] = False
    reps = np.ones(len(ends), dtype=np.int64)
    if os.path.exists(base + ".score.npy") and not (held is not None and held[0] == "eval"):
        s = np.load(base + ".score.npy").astype(np.float32)[:len(ends)]
        reps[:len(s)] = np.where(s >= 3.0, 3, np.where(s >= 2.5, 1, (rng.random(len(s)) < 0.25).astype(np.int64)))
    out = []
    for i in np.flatnonzero(keep & (reps > 0)):
        out.extend([np.asarray(arr[starts[i]:ends[i]])] * int(reps[i]))
    order = rng.permutation(len(out))
    return [out[j] for j in order]


class _Source:
    """One named source: shard order per epoch from (seed, epoch), documents per shard from (seed, epoch, shard)."""

    def __init__(self, root, src, seed, rank, world, eos, heldout_tok=0, split="train"):
        self.dir, self.eos, self.seed = os.path.join(root, src), eos, seed
        names = _shard_names(root, src)
        # held-out text = the tail of the source's last shard (by name, before the split over ranks): training never
        # sees it, the "eval" split reads nothing else (every rank the same documents: evaluation is replicated)
        self.held = (names[-1], split, int(heldout_tok)) if heldout_tok and names else None
        if self.held and split == "eval":
            names, rank, world = names[-1:], 0, 1
        self.names = [n for i, n in enumerate(names) if i % world == rank]
        if not self.names:
            raise ValueError(f"{src}: no shards for rank {rank} of {world}")
        self.epoch = self.si = self.di = self.off = 0
        self.docs, self.ahead = None, None
        self._reorder()

    def _reorder(self):
        self.order = np.random.default_rng((self.seed, self.epoch)).permutation(len(self.names))

    def _load(self, epoch, si):
        name = self.names[np.random.default_rng((self.seed, epoch)).permutation(len(self.names))[si % len(self.names)]]
        held = (self.held[1], self.held[2]) if self.held and name == self.held[0] else None
        return shard_documents(os.path.join(self.dir, name), self.eos, np.random.default_rng((self.seed, epoch, si)), held)

    def _prefetch(self):
        nxt = self.si + 1
        if nxt >= len(self.order):
            self.ahead = None
            return
        box, epoch = {}, self.epoch

        def work():
            try:
                box["docs"] = self._load(epoch, nxt)
            except BaseException as e:   # noqa: BLE001 - re-raised by the consumer
                box["err"] = e
        t = threading.Thread(target=work, daemon=True)
        t.start()
        self.ahead = (epoch, nxt, t, box)

    def _take_ahead(self):
        if self.ahead is not None and self.ahead[:2] == (self.epoch, self.si):
            _, _, t, box = self.ahead
            t.join()
            if "err" in box:
                raise box["err"]
            return box["docs"]
        return self._load(self.epoch, self.si)

    def next_piece(self, n):
        """Next <= n tokens: a huge document (a whole repository) comes out in parts, so that one document of
        hundreds of thousands of tokens does not distort the shares."""
        if self.docs is None:
            self.docs = self._load(self.epoch, self.si)
            self._prefetch()
        while self.di >= len(self.docs):
            self.si, self.di, self.off = self.si + 1, 0, 0
            if self.si >= len(self.order):
                self.epoch, self.si = self.epoch + 1, 0
                self._reorder()
            self.docs = self._take_ahead()
            self._prefetch()
        d = self.docs[self.di]
        piece = d[self.off:self.off + n]
        self.off += len(piece)
        if self.off >= len(d):
            self.di, self.off = self.di + 1, 0
        return piece

    def state(self):
        return {"epoch": self.epoch, "si": self.si, "di": self.di, "off": self.off}

    def restore(self, st):
        self.epoch, self.si, self.di, self.off = st["epoch"], st["si"], st["di"], st.get("off", 0)
        self._reorder()
        self.docs, self.ahead = None, None


class ShardCorpus:
    def __init__(self, weights, root, seq=8192, seed=0, rank=0, world=1, eos=None, heldout_tok=0, split="train"):
        self.srcs = list(weights)
        if eos is None:
            first = _shard_names(root, self.srcs[0])[0]
            eos = json.load(open(os.path.join(root, self.srcs[0], first + ".json")))["eos"]
        self.eos = int(eos)
        tot = float(sum(weights.values()))
        self.p = np.array([weights[s] / tot for s in self.srcs])
        self.sources = [_Source(root, s, seed + 1000 * k, rank, world, self.eos, heldout_tok, split)
                        for k, s in enumerate(self.srcs)]
        self.seq, self.n_docs = seq, 0
        self.buf = np.zeros(0, dtype=np.uint32)
        self.taken = np.zeros(len(self.srcs))

    def _pick(self):
        return int(np.argmax(self.p * (self.taken.sum() + 1) - self.taken))

    def batch(self, B):
        """(B, seq + 1) int64 windows."""
        need = B * (self.seq + 1)
        parts, have = [self.buf], len(self.buf)
        while have < need:
            k = self._pick()
            d = self.sources[k].next_piece(self.seq + 1)
            self.taken[k] += len(d)
            self.n_docs += 1
            parts.append(d)
            have += len(d)
        flat = np.concatenate(parts)
        self.buf = flat[need:]
        return flat[:need].astype(np.int64).reshape(B, self.seq + 1)

    def state_dict(self):
        return {"sources": [s.state() for s in self.sources], "taken": self.taken.tolist(), "buf": self.buf.tolist(),
                "n_docs": self.n_docs}

    def load_state_dict(self, st):
        for s, ss in zip(self.sources, st["sources"]):
            s.restore(ss)
        self.taken = np.array(st["taken"], dtype=np.float64)
        self.buf = np.array(st["buf"], dtype=np.uint32)
        self.n_docs = st["n_docs"]

    def mix(self):
        t = self.taken.sum() or 1
        return {s: round(float(x / t), 4) for s, x in zip(self.srcs, self.taken)}


def write_shard(root, src, name, docs, eos, drop=None, cdrop=None, score=None, compress=False):
    """Write one shard in the layout above (used by the tests and by the synthetic-corpus command)."""
    d = os.path.join(root, src)
    os.makedirs(d, exist_ok=True)
    flat = np.concatenate([np.concatenate([np.asarray(x, dtype=np.uint32), [np.uint32(eos)]]) for x in docs]).astype(np.uint32)
    if compress:
        import zstandard
        open(os.path.join(d, name + ".u32.zst"), "wb").write(zstandard.ZstdCompressor().compress(flat.tobytes()))
    else:
        np.save(os.path.join(d, name + ".u32.npy"), flat)
    json.dump({"eos": int(eos), "docs": len(docs), "tokens": int(len(flat))}, open(os.path.join(d, name + ".json"), "w"))
    for ext, v in ((".drop.npy", drop), (".cdrop.npy", cdrop), (".score.npy", score)):
        if v is not None:
            np.save(os.path.join(d, name + ext), np.asarray(v))


class HostLoader:
    """Worker thread -> bounded queue of (pinned batch, corpus state after it).  `next()` returns the batch on
    `device` (async copy from pinned memory) and remembers that batch's state for `state_dict()`."""

    def __init__(self, corpus, B, device="cpu", depth=2, pin=None, xform=None, first=0):
        """`xform(xy, n) -> (xy, extra)` rewrites batch number n on the worker thread (needle injection); the batch
        number is part of the loader's state, so a resumed run rewrites the same batches the same way, and the
        `extra` of the batch handed out last is kept in `self.extra`."""
        import torch
        self.corpus, self.B, self.device = corpus, B, torch.device(device)
        self.xform, self.n_next, self.n_done, self.extra = xform, int(first), int(first), None
        self.pin = (self.device.type == "cuda") if pin is None else pin
        self.q = queue.Queue(maxsize=depth)
        self.state = corpus.state_dict()
        self._stop = threading.Event()
        self.bytes_per_batch = B * (corpus.seq + 1) * 8
        self.t = threading.Thread(target=self._work, daemon=True)
        self.t.start()

    def _work(self):
        import torch
        try:
            while not self._stop.is_set():
                xy, extra = self.corpus.batch(self.B), None
                if self.xform is not None:
                    xy, extra = self.xform(xy, self.n_next)
                    xy = np.ascontiguousarray(xy, dtype=np.int64)
                if hasattr(self.corpus, "extra"):            # per-kind corpus: the kind and layer combination of the step
                    kx = self.corpus.extra()
                    if kx:                                   # (synthetic rows may have changed the number of rows)
                        extra = dict(extra or {}, **{k: np.repeat(v[:1], len(xy), 0) for k, v in kx.items()})
                self.n_next += 1
                x = torch.from_numpy(xy)
                if self.pin:
                    x = x.pin_memory()
                item = (x, self.corpus.state_dict(), extra, self.n_next)
                while not self._stop.is_set():
                    try:
                        self.q.put(item, timeout=0.2)
                        break
                    except queue.Full:
                        continue
        except BaseException as e:   # noqa: BLE001 - forwarded to the consumer
            self.q.put(e)

    def next(self):
        item = self.q.get()
        if isinstance(item, BaseException):
            raise RuntimeError("corpus worker failed") from item
        x, self.state, self.extra, self.n_done = item
        return x.to(self.device, non_blocking=True)

    def state_dict(self):
        return dict(self.state, loader_n=self.n_done)

    def close(self):
        self._stop.set()
        try:
            while True:
                self.q.get_nowait()
        except queue.Empty:
            pass
        self.t.join(timeout=2)
