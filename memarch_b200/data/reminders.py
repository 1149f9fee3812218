"""Recall needles written into real text, with a success-driven distance curriculum, and the per-kind corpus of the
layer-pool ("fishki") experiments.

Behaviour follows the reference's host-side data tools (memarch_jax/memarch_jax/data.py:344-774 `Reminders`,
200-255 `KindCorpus`):

* a row gets, with probability p, a block of facts `[M k1 v1 .. kn vn M]` and, at least `dist` words later, a block of
  questions `[M kq1 vq1 .. M]` over the same keys in a shuffled order; keys are distinct tokens of a 512-token range,
  values come from a 64-token range, `M` is a marker token; shapes never change (the needle overwrites text);
* `rem` (B, T) marks the positions of x that hold a question key: the target there is the value;
* randomness depends on (seed, content of the row) only, so the same batch gets the same needles after a resume;
* p may follow a schedule (p0 for `warm` batches, then linear over `decay` batches to p);
* with a distance ladder the needle distance is drawn from the current level's range; a level is passed when the
  accuracy over the last >= `win` needle answers reaches `thr`, and the next level starts `lag` batches later
  (more than the prefetch depth, so the choice is deterministic); the last level mixes all distances;
* `exact` (evaluation) puts exactly that many words between the two blocks;
* `synth` batches are filler plus one needle (the pure recall task);
* `near`: a share of the needles at distance 0..near_max, inside the attention window;
* `per_row` / `far_log`: several marker-free needles per row of text with log-uniform far distances;
* `same_fmt`: one needle per row in the marker-free format of the synthetic episodes, `[k v]*n` ... `[k v]*n`, with
  every other occurrence of a needle token scrubbed from the row;
* `blank`: the true values are returned in `rem_y` (B, T); with `same_fmt` and in the episodes the value after each
  question key is also replaced by the marker in the text: "the answers are seen only after the test";
* `pack`: the `synth` batches are the short-row episodes of `data.episodes.Episodes` with their own curriculum, and
  `mix=(shares, length)` keeps a decaying share of synthetic batches after the stage: phase k of `length` batches has
  the share `shares[k]`, the last share stays for good (which batches are synthetic depends on the number only);
* `__call__(..., pack=(pairs, fill))` (evaluation): rows densely laid out with episodes of exactly that shape.
"""
from __future__ import annotations

import zlib

import numpy as np

from .episodes import Episodes

N_KEYS, N_VALS = 512, 64
GOLDEN = 0.6180339887498949                          # batch number -> evenly spread point of [0, 1)


class Reminders:
    def __init__(self, p, T, n=16, dist=2048, tok0=1000, seed=0, V=None, p0=None, warm=0, decay=0, ladder=None,
                 thr=0.9, win=800, lag=5, dmin=0, synth=0, doc_eos=None, near=0.0, near_max=0, blank=False,
                 per_row=1, far_log=None, same_fmt=False, pack=None, mix=None):
        """`pack`: None, True or a dict of `Episodes` options."""
        self.p, self.T, self.n, self.dist, self.seed = float(p), int(T), int(n), int(dist), int(seed)
        self.p0 = None if p0 is None else float(p0)
        self.warm, self.decay = int(warm), int(decay)
        self.ladder = sorted(int(v) for v in ladder) if ladder else None
        self.thr, self.win, self.lag, self.dmin = float(thr), int(win), int(lag), int(dmin)
        self.synth, self.V = int(synth), V
        self.doc_eos = None if doc_eos is None or int(doc_eos) < 0 else int(doc_eos)
        self.near, self.near_max = float(near), int(near_max)
        self.per_row, self.far_log = int(per_row), (None if far_log is None else float(far_log))
        self.blank, self.same_fmt = bool(blank), bool(same_fmt)
        self.n_keys, self.n_vals = N_KEYS, N_VALS
        self.mix_shares, self.mix_len = (list(mix[0]), int(mix[1])) if mix else (None, 250)
        self.k0, self.v0, self.mark = tok0, tok0 + N_KEYS, tok0 + N_KEYS + N_VALS
        self.L = 2 * self.n + 2                      # one block: marker, n (key, value) pairs, marker
        self.changes = [(0, 0)]                      # (first batch, level)
        self.hits = self.answers = 0.0
        if V is not None and self.mark >= V:
            raise ValueError(f"needle tokens {tok0}..{self.mark} do not fit a vocabulary of {V}")
        if self.n > N_KEYS:
            raise ValueError("more pairs than distinct keys")
        if 2 * self.L + self.dist > self.T + 1:
            raise ValueError(f"T={T} too short for two blocks of {self.L} and a distance of {dist}")
        if self.ladder and self.ladder[-1] > self.T + 1 - 2 * self.L:
            raise ValueError(f"ladder {self.ladder} exceeds the row")
        self.pack = Episodes(self, **(pack if isinstance(pack, dict) else {})) if pack else None

    # ------------------------------------------------------------------------------------------------ schedule
    def p_at(self, i):
        if self.p0 is None:
            return self.p
        if i < self.warm:
            return self.p0
        return self.p0 + (self.p - self.p0) * min(1.0, (i - self.warm) / max(self.decay, 1))

    def synth_at(self, i):
        if i is None:
            return False
        if i < self.synth:
            return True
        if not self.mix_shares:
            return False
        phase = min((i - self.synth) // max(self.mix_len, 1), len(self.mix_shares) - 1)
        return (i * GOLDEN) % 1.0 < self.mix_shares[phase]

    def level_at(self, i):
        k = 0
        for first, level in self.changes:
            if first <= i:
                k = level
        return k

    def range_at(self, i):
        k = self.level_at(i)
        if k == len(self.ladder) - 1:                # last level: every distance, short ones are not forgotten
            return self.dmin, self.ladder[-1]
        return (self.ladder[k - 1] if k else self.dmin), self.ladder[k]

    def observe(self, i, hits, n_ans):
        """After step i: needle accuracy of the training batch -> maybe a level change; returns a log line or None."""
        if self.pack is not None and self.synth_at(i):
            return self.pack.observe(i, hits, n_ans)
        if not self.ladder:
            return None
        self.hits += hits
        self.answers += n_ans
        k = self.changes[-1][1]
        if self.answers < self.win or k >= len(self.ladder) - 1:
            return None
        acc = self.hits / self.answers
        self.hits = self.answers = 0.0
        if acc < self.thr:
            return None
        self.changes.append((i + self.lag, k + 1))
        lo, hi = self.range_at(i + self.lag)
        return f"reminders: level {k} -> {k + 1} (accuracy {acc:.3f}), from batch {i + self.lag} distance {lo}..{hi}"

    def state(self):
        st = {"changes": [list(c) for c in self.changes], "acc_h": self.hits, "acc_n": self.answers}
        if self.pack is not None:
            st.update(self.pack.state())
        return st

    def load(self, st):
        self.changes = [tuple(c) for c in st["changes"]]
        self.hits, self.answers = st["acc_h"], st["acc_n"]
        if self.pack is not None:
            self.pack.load(st)

    # ------------------------------------------------------------------------------------------------ rows
    def _filler(self, rng, n):
        """Random words outside the needle tokens."""
        V = self.V or (self.mark + 20001)
        span = self.mark + 1 - self.k0
        f = rng.integers(0, V - span, n)
        f = np.where(f >= self.k0, f + span, f).astype(np.int32)
        if self.doc_eos is not None:
            f[f == self.doc_eos] = 0
        return f

    def _needle(self, row, rng, exact=None, level_range=None):
        n, L, T1 = self.n, self.L, len(row)
        keys = self.k0 + rng.permutation(N_KEYS)[:n]
        vals = self.v0 + rng.integers(0, N_VALS, n)
        if exact is None and level_range is not None:
            exact = int(rng.integers(level_range[0], level_range[1] + 1))
        if exact is None:
            s = int(rng.integers(0, T1 - 2 * L - self.dist + 1))
            q = int(rng.integers(s + L + self.dist, T1 - L + 1))
        else:
            if not 0 <= exact <= T1 - 2 * L:
                raise ValueError(f"distance {exact} does not fit a row of {T1}")
            s = int(rng.integers(0, T1 - 2 * L - exact + 1))
            q = s + L + exact
        facts = np.stack([keys, vals], 1).reshape(-1)
        order = rng.permutation(n)
        asks = np.stack([keys[order], vals[order]], 1).reshape(-1)
        if self.same_fmt:                            # needle tokens are ordinary words of real text: 5-7 % of a row
            stray = (row >= self.k0) & (row <= self.mark)   # would look like facts, so none stays outside the needle
            if stray.any():
                row[stray] = self._filler(rng, int(stray.sum()))
            row[s:s + 2 * n], row[q:q + 2 * n] = facts, asks
            first = q
        else:
            row[s] = row[s + L - 1] = row[q] = row[q + L - 1] = self.mark
            row[s + 1:s + L - 1], row[q + 1:q + L - 1] = facts, asks
            first = q + 1
        if self.doc_eos is not None:                 # a document boundary between facts and questions would hide them
            seg = row[s:q + L]
            hit = seg == self.doc_eos
            if hit.any():
                seg[hit] = self._filler(rng, int(hit.sum()))
        return first + 2 * np.arange(n)              # positions of the question keys in x (y there is the value)

    def _several(self, row, rng):
        """Several needles in one row of text, without markers: facts `[k v]*n`, questions `[k v]*n` in another order.
        All keys of the row are distinct, blocks do not overlap (a needle may lie inside another, as in a
        conversation), and the needle tokens occur nowhere else in the row.  Distance: with probability `far_log`
        (default 1 - near) log-uniform between `dist` and the end of the row, otherwise 0..near_max."""
        n, T1 = self.n, len(row)
        Lb = 2 * n
        stray = (row >= self.k0) & (row <= self.mark)
        if stray.any():
            row[stray] = self._filler(rng, int(stray.sum()))
        R = max(1, min(self.per_row, N_KEYS // n))
        all_keys = self.k0 + rng.permutation(N_KEYS)[:R * n]
        taken = np.zeros(T1, bool)
        dmax = T1 - 2 * Lb
        far = self.far_log if self.far_log is not None else 1.0 - self.near
        lo = max(1, min(self.dist, dmax))
        found = []
        for r in range(R):
            for _ in range(32):                                       # a few tries to find free room
                if rng.random() < far:
                    d = min(max(int(np.exp(rng.uniform(np.log(lo), np.log(dmax + 1)))), lo), dmax)
                else:
                    d = int(rng.integers(0, min(self.near_max, dmax) + 1))
                s = int(rng.integers(0, dmax - d + 1))
                q = s + Lb + d
                if taken[s:s + Lb].any() or taken[q:q + Lb].any():
                    continue
                keys = all_keys[r * n:(r + 1) * n]
                vals = self.v0 + rng.integers(0, N_VALS, n)
                order = rng.permutation(n)
                row[s:s + Lb] = np.stack([keys, vals], 1).reshape(-1)
                row[q:q + Lb] = np.stack([keys[order], vals[order]], 1).reshape(-1)
                taken[s:s + Lb] = taken[q:q + Lb] = True
                if self.doc_eos is not None:
                    seg = row[s:q + Lb]
                    cut = seg == self.doc_eos
                    if cut.any():
                        seg[cut] = self._filler(rng, int(cut.sum()))
                found.append(q + 2 * np.arange(n))
                break
        return np.sort(np.concatenate(found)) if found else np.zeros(0, np.int64)

    def __call__(self, xy, p=None, exact=None, n=None, synth=None, pack=None):
        """xy (B, T+1) tokens -> (xy with needles, {"rem": (B, T) int8}).  `n` = number of the training batch."""
        if synth is None:
            synth = self.synth_at(n)
        level_range = None
        if n is not None and p is None:
            p = self.p_at(n)
            level_range = self.range_at(n) if self.ladder else None
        p = self.p if p is None else p
        if synth and self.pack is not None and n is not None and pack is None:
            return self.pack.batch(xy.shape, n)
        dense = (self.pack or Episodes(self)) if synth and pack is not None else None
        xy = np.array(xy, copy=True)
        B, T1 = xy.shape
        rem = np.zeros((B, T1 - 1), np.int8)
        rem_y = np.zeros((B, T1 - 1), np.int32) if self.blank else None
        for b in range(B):
            rng = np.random.default_rng([self.seed, zlib.crc32(xy[b].tobytes())])
            pq, hide = None, self.same_fmt
            if dense is not None:
                xy[b] = self._filler(rng, T1)
                pq, hide = dense.fill_row(xy[b], rng, *pack), True
            elif synth:
                xy[b] = self._filler(rng, T1)
                pq = self._needle(xy[b], rng, exact, level_range)
            elif rng.random() < p:
                ex = exact
                several = self.per_row > 1 or self.far_log is not None          # draws its own near / far distances
                if ex is None and not several and self.near > 0 and self.near_max > 0 and rng.random() < self.near:
                    ex = int(rng.integers(0, min(self.near_max, T1 - 2 * self.L) + 1))
                if ex is None and level_range is None and several:
                    pq = self._several(xy[b], rng)
                else:
                    pq = self._needle(xy[b], rng, ex, None if ex is not None else level_range)
            if pq is not None:
                rem[b, pq] = 1
                if self.blank:
                    rem_y[b, pq] = xy[b, pq + 1]
                    if hide:
                        xy[b, pq + 1] = self.mark
        out = {"rem": rem}
        if self.blank:
            out["rem_y"] = rem_y
        return xy, out

    @staticmethod
    def score(logits_argmax, xy, rem):
        """(hits, answers) of a batch: predictions at the marked positions against the values that follow."""
        rem = np.asarray(rem) > 0
        y = np.asarray(xy)[:, 1:]
        return float((np.asarray(logits_argmax)[rem] == y[rem]).sum()), float(rem.sum())


class KindCorpus:
    """Every batch of a step comes from one kind of text.  `kinds`: {kind: {source: weight}}; `pools`: the layer sets
    per kind (`models.fishki.pools`).  The kind of a step is the one furthest behind its share (depends on the step
    number only, so all processes agree); the combination of `c` layers is drawn from the kind's pool by
    (seed, step); `full=True` uses the whole pool in its order.  `extra()` -> {"kind": (B,1), "fish": (B,c)}."""

    def __init__(self, kinds, pools, c, root, seq=8192, seed=0, rank=0, world=1, eos=None, doc_seed=None):
        from .loader import ShardCorpus
        self.names = list(kinds)
        w = np.array([sum(kinds[k].values()) for k in self.names], np.float64)
        self.p = w / w.sum()
        base = seed if doc_seed is None else doc_seed             # other documents, same schedule of kinds
        self.subs = [ShardCorpus(kinds[k], root, seq=seq, seed=base + 7919 * i, rank=rank, world=world, eos=eos)
                     for i, k in enumerate(self.names)]
        self.eos, self.seq = self.subs[0].eos, seq
        self.pools, self.c, self.seed = pools, int(c), seed
        self.full = False
        self.n = 0
        self.count = np.zeros(len(self.names))
        self._extra = None

    def _kind(self):
        return int(np.argmax(self.p * (self.n + 1) - self.count))

    def batch(self, B):
        k = self._kind()
        xy = self.subs[k].batch(B)
        if self.full:
            order = list(self.pools[k])
        else:
            rng = np.random.default_rng([self.seed, 31337, self.n])
            order = [int(i) for i in rng.choice(self.pools[k], self.c, replace=False)]
        self._extra = {"kind": np.full((B, 1), k, np.int32), "fish": np.tile(np.asarray(order, np.int32), (B, 1))}
        self.count[k] += 1
        self.n += 1
        return xy

    def extra(self):
        return self._extra

    def state_dict(self):
        return {"subs": [s.state_dict() for s in self.subs], "count": self.count.tolist(), "n": self.n}

    def load_state_dict(self, st):
        if st.get("subs") is not None:                            # None: new documents from the start, same schedule
            for s, ss in zip(self.subs, st["subs"]):
                s.load_state_dict(ss)
        self.count = np.array(st["count"], np.float64)
        self.n = int(st["n"])

    def mix(self):
        t = self.count.sum() or 1
        return {k: round(float(x / t), 4) for k, x in zip(self.names, self.count)}
