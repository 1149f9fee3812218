"""Corpus preparation on token shards: tokenise -> near-duplicate removal (MinHash) -> benchmark decontamination
(13-gram matches) -> code-quality score; the masks it writes are the ones `data/loader.py` honours.

Behaviour follows the reference's `data/` tools (tokenize_hf.py, minhash.py, dedup_cluster.py, decontam.py,
contam_report.py, score_code.py, postproc.py); everything works on token ids, texts are never decoded again; storage
is a local directory tree `<root>/<source>/<shard>.*` (the reference's bucket transport is out of scope here).

  signatures      one-permutation MinHash over 5-token shingles, 112 bins = 14 bands x 8 rows (threshold ~0.8 Jaccard),
                  empty bins densified from the next non-empty one; one uint64 per band, 0 = no shingle at all
  dedup           band collisions across ALL sources -> connected components -> keep one copy per cluster (source
                  priority first, then first seen) -> `<shard>.drop.npy`
  bench index     hashes of every 13 consecutive tokens of the benchmark items
  match / dirty   sparse (document, gram) pairs per shard; a document is dirty for an item if it covers
                  >= max(min(0.5 x item grams, 40), 5) distinct grams of it -> `<shard>.cdrop.npy`
  CodeScorer      linear model on sqrt unigram / hashed-bigram frequencies + log length -> `<shard>.score.npy`
"""
from __future__ import annotations

import glob
import json
import os

import numpy as np

from .loader import _read_tokens, _shard_names, write_shard

M1, M2 = np.uint64(0x9E3779B97F4A7C15), np.uint64(0xBF58476D1CE4E5B9)
EMPTY = np.uint64(0xFFFFFFFF)


def _roll_hash(a, n, mul=M1):
    a = a.astype(np.uint64)
    h = np.zeros(len(a) - n + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        for k in range(n):
            h = h * mul + a[k:len(a) - n + 1 + k]
    return h


def doc_bounds(arr, eos):
    ends = np.flatnonzero(arr == eos)
    return np.concatenate([[0], ends[:-1] + 1]), ends            # [start, end) without the end-of-text token


# ------------------------------------------------------------------------------------------------ MinHash
def signatures(arr, eos, shingle=5, bins=112, bands=14):
    """(documents, bands) uint64 band hashes of one shard."""
    rows = bins // bands
    starts, ends = doc_bounds(arr, eos)
    out = np.zeros((len(ends), bands), dtype=np.uint64)
    if len(arr) < shingle or not len(ends):
        return out
    h = _roll_hash(arr, shingle)
    with np.errstate(over="ignore"):
        h ^= h >> np.uint64(31)
        h *= M2
        h ^= h >> np.uint64(29)
    p = np.arange(len(h))
    d = np.searchsorted(ends, p)                                   # document in which the shingle starts
    ok = (d < len(ends)) & (p + shingle - 1 < ends[np.minimum(d, len(ends) - 1)])   # does not touch end-of-text
    h, d = h[ok], d[ok]
    sig = np.full((len(ends), bins), EMPTY, dtype=np.uint64)
    if len(h):
        cell = d * bins + (h % np.uint64(bins)).astype(np.int64)
        val = h >> np.uint64(32)
        order = np.lexsort((val, cell))
        cell, val = cell[order], val[order]
        first = np.concatenate([[True], cell[1:] != cell[:-1]])   # minimum of every (document, bin)
        sig.reshape(-1)[cell[first]] = val[first]
    filled = sig != EMPTY
    has_any = filled.any(1)
    # densify: an empty bin takes the next non-empty bin to its right (circular) plus an offset for the distance
    idx = np.arange(2 * bins)
    nxt = np.where(np.concatenate([filled, filled], 1), idx, 4 * bins)
    nxt = np.minimum.accumulate(nxt[:, ::-1], axis=1)[:, ::-1][:, :bins]
    src = np.where(nxt < 2 * bins, nxt % bins, 0)
    dens = np.take_along_axis(sig, src, 1) + (nxt - idx[:bins]).astype(np.uint64) * np.uint64(1 << 32)
    sig = np.where(filled, sig, dens).reshape(len(ends), bands, rows)
    with np.errstate(over="ignore"):
        bh = np.full((len(ends), bands), np.uint64(1469598103934665603), dtype=np.uint64)
        for r in range(rows):
            bh = (bh ^ sig[:, :, r]) * M2
        bh += np.arange(bands, dtype=np.uint64) * M1               # bands never match one another
    bh[bh == 0] = 1
    bh[~has_any] = 0
    return bh


def dedup(sig_files, priority=(), min_bands=1):
    """sig_files: list of `<root>/<source>/<shard>.mh.npy`.  Writes `<shard>.drop.npy` beside each and returns
    {source: (documents, dropped)}."""
    from scipy.sparse import coo_matrix
    from scipy.sparse.csgraph import connected_components
    srcs = [os.path.basename(os.path.dirname(f)) for f in sig_files]
    pri = [priority.index(s) if s in priority else len(priority) for s in srcs]
    mm = [np.load(f, mmap_mode="r") for f in sig_files]
    sizes = np.array([len(m) for m in mm], dtype=np.int64)
    off = np.concatenate([[0], np.cumsum(sizes)])
    total = int(off[-1])
    rank = np.repeat(np.array(pri, dtype=np.int64), sizes) * max(total, 1) + np.arange(total)
    eu, ev = [], []
    for b in range(mm[0].shape[1] if mm else 0):
        h = np.concatenate([np.asarray(m[:, b]) for m in mm])
        g = np.flatnonzero(h)
        o = np.argsort(h[g], kind="stable")
        hs, g = h[g][o], g[o]
        same = np.flatnonzero(hs[1:] == hs[:-1])
        eu.append(g[same])
        ev.append(g[same + 1])                                     # a chain inside a group of equal hashes connects it
    u = np.concatenate(eu) if eu else np.zeros(0, np.int64)
    v = np.concatenate(ev) if ev else np.zeros(0, np.int64)
    if min_bands > 1 and len(u):
        key = np.minimum(u, v) * total + np.maximum(u, v)
        k, c = np.unique(key, return_counts=True)
        k = k[c >= min_bands]
        u, v = k // total, k % total
    drop = np.zeros(0, np.int64)
    if len(u):
        nodes, inv = np.unique(np.concatenate([u, v]), return_inverse=True)
        n = len(nodes)
        gr = coo_matrix((np.ones(len(u), dtype=np.int8), (inv[:len(u)], inv[len(u):])), shape=(n, n))
        nc, lab = connected_components(gr, directed=False)
        r = rank[nodes]
        best = np.full(nc, np.iinfo(np.int64).max)
        np.minimum.at(best, lab, r)
        drop = np.sort(nodes[r != best[lab]])
    fi = np.searchsorted(off, drop, side="right") - 1
    report = {}
    for i, f in enumerate(sig_files):
        d = (drop[fi == i] - off[i]).astype(np.uint32)
        np.save(f.replace(".mh.npy", ".drop.npy"), d)
        t = report.setdefault(srcs[i], [0, 0])
        t[0] += int(sizes[i])
        t[1] += len(d)
    return {k: tuple(v) for k, v in report.items()}


# ------------------------------------------------------------------------------------------------ decontamination
def build_bench_index(items, n=13, names=None, item_src=None):
    """items: list of token-id arrays (one per benchmark question/solution).  Returns the index dict:
    h (sorted unique gram hashes), item (item of every gram), item_grams (distinct grams per item)."""
    hs, it = [], []
    for k, ids in enumerate(items):
        ids = np.asarray(ids, dtype=np.uint32)
        if len(ids) >= n:
            g = _roll_hash(ids, n)
            hs.append(g)
            it.append(np.full(len(g), k, dtype=np.uint32))
    h = np.concatenate(hs) if hs else np.zeros(0, np.uint64)
    item = np.concatenate(it) if it else np.zeros(0, np.uint32)
    h, i = np.unique(h, return_index=True)
    item = item[i]
    return {"h": h, "item": item, "item_grams": np.bincount(item, minlength=len(items)).astype(np.uint32), "n": n,
            "item_src": np.asarray(item_src if item_src is not None else np.zeros(len(items)), dtype=np.uint8),
            "names": np.asarray(names if names is not None else ["bench"])}


def match_bench(arr, eos, index, chunk=16_000_000):
    """(doc, gram, n_docs): every 13-gram of the shard that is a benchmark gram, as sparse pairs."""
    n, bh = int(index["n"]), index["h"]
    ends = np.flatnonzero(arr == eos)
    docs, gs = [], []
    for s in range(0, max(len(arr) - n + 1, 0), chunk):           # overlapping chunks: no gram lost on a boundary
        h = _roll_hash(arr[s:s + chunk + n - 1], n)
        j = np.searchsorted(bh, h)
        j[j == len(bh)] = 0
        ok = bh[j] == h if len(bh) else np.zeros(len(h), bool)
        pos = np.flatnonzero(ok)
        docs.append(np.searchsorted(ends, s + pos).astype(np.uint32))
        gs.append(j[pos].astype(np.uint32))
    cat = lambda xs: np.concatenate(xs) if xs else np.zeros(0, np.uint32)
    return cat(docs), cat(gs), len(ends)


def dirty_docs(doc, gram, index, frac=0.5, cap=40, minimum=5):
    """Documents that really contain a benchmark item (boilerplate lines give 1-2 matches per item and do not pass)."""
    if len(doc) == 0:
        return np.zeros(0, np.uint32), np.zeros(0, np.uint32)
    key = np.unique(doc.astype(np.uint64) << np.uint64(32) | gram.astype(np.uint64))
    d = (key >> np.uint64(32)).astype(np.uint32)
    it = index["item"][(key & np.uint64(0xFFFFFFFF)).astype(np.int64)]
    pk, cnt = np.unique(d.astype(np.uint64) << np.uint64(32) | it.astype(np.uint64), return_counts=True)
    pd, pi = (pk >> np.uint64(32)).astype(np.uint32), (pk & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    need = np.maximum(np.minimum(frac * index["item_grams"][pi], cap), minimum)
    ok = cnt >= need
    return pd[ok], pi[ok]


# ------------------------------------------------------------------------------------------------ code quality
class CodeScorer:
    """score = sqrt(unigram freq) . cu + sqrt(hashed-bigram freq) . cb + cl log(n)/10 + b0, a 0-5 quality estimate."""

    def __init__(self, V, H=1 << 16, coef=None, intercept=0.0):
        self.V, self.H = V, H
        self.coef = np.zeros(V + H + 1, dtype=np.float32) if coef is None else np.asarray(coef, dtype=np.float32)
        self.intercept = float(intercept)

    def features(self, d):
        n = max(len(d), 1)
        u, cu = np.unique(np.minimum(d, self.V - 1), return_counts=True)
        bh = (d[:-1].astype(np.int64) * 1_000_003 + d[1:]) % self.H
        bu, bc = np.unique(bh, return_counts=True)
        return (u, np.sqrt(cu / n)), (bu + self.V, np.sqrt(bc / n)), np.log(n) / 10

    def score_doc(self, d):
        (u, fu), (b, fb), ln = self.features(np.asarray(d))
        return float(fu @ self.coef[u] + fb @ self.coef[b] + self.coef[-1] * ln + self.intercept)

    def score_shard(self, arr, eos):
        starts, ends = doc_bounds(arr, eos)
        return np.asarray([self.score_doc(arr[s:e]) for s, e in zip(starts, ends)], dtype=np.float16)

    def fit(self, docs, labels, l2=1.0, iters=200, lr=0.5):
        """Ridge regression by gradient descent on the sparse features (labels 0-5)."""
        feats = [self.features(np.asarray(d)) for d in docs]
        y = np.asarray(labels, dtype=np.float32)
        self.intercept = float(y.mean())
        for _ in range(iters):
            grad = l2 * self.coef / len(docs)
            gb = 0.0
            for ((u, fu), (b, fb), ln), t in zip(feats, y):
                r = fu @ self.coef[u] + fb @ self.coef[b] + self.coef[-1] * ln + self.intercept - t
                np.add.at(grad, u, r * fu / len(docs))
                np.add.at(grad, b, r * fb / len(docs))
                grad[-1] += r * ln / len(docs)
                gb += r / len(docs)
            self.coef -= lr * grad
            self.intercept -= lr * gb
        return self

    def save(self, path):
        np.savez(path, V=self.V, H=self.H, coef=self.coef, intercept=self.intercept)

    @classmethod
    def load(cls, path):
        m = np.load(path)
        return cls(int(m["V"]), int(m["H"]), m["coef"], float(m["intercept"]))


# ------------------------------------------------------------------------------------------------ stages
def tokenize_texts(texts, encode, eos, root, source, shard_tokens=50_000_000, compress=False):
    """Encode an iterable of texts with `encode(str) -> ids` and write shards of about `shard_tokens` tokens."""
    docs, n, k = [], 0, 0
    for t in texts:
        ids = np.asarray(encode(t), dtype=np.uint32)
        docs.append(ids)
        n += len(ids) + 1
        if n >= shard_tokens:
            write_shard(root, source, f"shard_{k:05d}", docs, eos, compress=compress)
            docs, n, k = [], 0, k + 1
    if docs:
        write_shard(root, source, f"shard_{k:05d}", docs, eos, compress=compress)
        k += 1
    return k


def postprocess(root, sources=None, bench_index=None, scorer=None, code_sources=("stack_v3",)):
    """One pass per shard: `.mh.npy`, `.contam.npz` and (code sources) `.score.npy`; what exists is skipped, so a
    restart continues where it stopped."""
    done = []
    for src in sources or sorted(d for d in os.listdir(root) if os.path.isdir(os.path.join(root, d))):
        for name in _shard_names(root, src):
            base = os.path.join(root, src, name)
            eos = json.load(open(base + ".json"))["eos"]
            arr = None
            load = lambda: np.asarray(_read_tokens(base))
            if not os.path.exists(base + ".mh.npy"):
                arr = load() if arr is None else arr
                np.save(base + ".mh.npy", signatures(arr, eos))
                done.append(base + ".mh.npy")
            if bench_index is not None and not os.path.exists(base + ".contam.npz"):
                arr = load() if arr is None else arr
                d, g, n = match_bench(arr, eos, bench_index)
                np.savez(base + ".contam.npz", doc=d, gram=g, n_docs=n)
                done.append(base + ".contam.npz")
            if scorer is not None and src in code_sources and not os.path.exists(base + ".score.npy"):
                arr = load() if arr is None else arr
                np.save(base + ".score.npy", scorer.score_shard(arr, eos))
                done.append(base + ".score.npy")
    return done


def finalize(root, bench_index=None, priority=()):
    """After `postprocess` ran for every shard: cluster duplicates across sources and settle contamination."""
    rep = {"dedup": dedup(sorted(glob.glob(os.path.join(root, "*", "*.mh.npy"))), priority)}
    if bench_index is not None:
        per = {}
        for f in sorted(glob.glob(os.path.join(root, "*", "*.contam.npz"))):
            z = np.load(f)
            pd, _ = dirty_docs(z["doc"], z["gram"], bench_index)
            drop = np.unique(pd)
            np.save(f.replace(".contam.npz", ".cdrop.npy"), drop)
            t = per.setdefault(os.path.basename(os.path.dirname(f)), [0, 0])
            t[0] += int(z["n_docs"])
            t[1] += len(drop)
        rep["contamination"] = {k: tuple(v) for k, v in per.items()}
    return rep
