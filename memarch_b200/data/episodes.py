"""Stage one of the recall curriculum: short synthetic rows that hold nothing but a recall episode.

An episode is `pairs` (key, value) facts, `fill` random words, then the same keys in another order, each followed by its
value: `[k v]*pairs  filler  [k v]*pairs`.  The facts stand at the very start of the row, where attention sees only a
few words, so the link "value <- its key" is learned quickly; the same task in the middle of a long row takes many
times longer (memarch_jax/memarch_jax/data.py:550-596 of the reference).

* The curriculum is a table of (pairs, fill) steps: for every fill length 16, 32, 64, ... (or, with `frac`, the given
  fractions of the model's attention window `win_ref`, which makes one table serve models of different sizes) the
  pair counts 4, 8 and n.  A step is passed when the accuracy over the last >= `win` answers reaches `thr`; the next
  step starts `lag` batches later, beyond the prefetch depth, so producer and consumer agree.  The last step draws the
  fill length of each batch from all lengths (optionally `far_frac` of the batches beyond `far_win` words, where only
  the long-range read can answer).
* The row length follows the step (4 * pairs + fill, rounded up to `round_to`), and the number of rows is chosen so
  that a batch holds as many words as a normal one, a multiple of `rows_mult` (one row per device at least).  Without
  `tail` the rounding lengthens the fill; with `tail` the fill stays nominal and the padding goes after the questions.
* `blank`: the value after each question key is replaced by the marker, the true value is returned in `rem_y`.
  `strict`: the row's fact values are returned in `rem_vals` (-1 beyond `pairs`).
* `fill_row` lays episodes densely into one long row (evaluation at a fixed (pairs, fill)); with `gap` marker words
  between episodes a question sees only its own episode inside the window.  Keys do not repeat within a row.

Everything is a function of (seed, batch number) or (seed, row content): a resumed run gets the same batches.
"""
from __future__ import annotations

import numpy as np

FILLS = tuple(16 << i for i in range(13))            # 16 .. 65536


class Episodes:
    def __init__(self, host, gap=0, round_to=1, rows_mult=1, frac=None, win_ref=None, tail=False, strict=False,
                 far_frac=None, far_win=2048, rank=0):
        """`host` is the `Reminders` object whose tokens, filler, seed, pair count and thresholds are used."""
        self.h = host
        self.gap, self.round_to, self.rows_mult = int(gap), max(1, int(round_to)), max(1, int(rows_mult))
        self.tail, self.strict = bool(tail), bool(strict)
        self.rank = int(rank)                           # data-parallel rank: same shapes on every rank, other rows
        self.far_frac, self.far_win = (None if far_frac is None else float(far_frac)), int(far_win)
        n, T = host.n, host.T
        if frac:
            if not win_ref:
                raise ValueError("a ladder in fractions of the window needs win_ref")
            fills = sorted({max(16, int(round(float(f) * win_ref))) for f in frac})
        else:
            fills = list(FILLS)
        self.fills = [f for f in fills if 4 * n + f <= T + 1]
        if not self.fills:
            raise ValueError(f"T={T} too short for an episode of {n} pairs and 16 words of filler")
        self.steps, seen = [], set()
        for f in self.fills:
            for pairs in sorted({min(4, n), min(8, n), n}):
                nominal = f
                if frac and self.round_to > 1 and not self.tail:         # to the NEAREST multiple, not upwards
                    r = self.round_to
                    nominal = max(r, int(round((4 * pairs + f - 1) / r)) * r) + 1 - 4 * pairs
                real = self.real_fill(pairs, nominal)
                if frac and (pairs, real) in seen:                       # the same true distance is no new step
                    continue
                seen.add((pairs, real))
                self.steps.append((pairs, nominal))
        self.changes = [(0, 0)]
        self.hits = self.answers = 0.0

    # ------------------------------------------------------------------------------------------------ curriculum
    def row_len(self, pairs, f):
        return -(-(4 * pairs + f - 1) // self.round_to) * self.round_to

    def real_fill(self, pairs, f):
        """Words between facts and questions once the row length is rounded."""
        return f if self.tail else self.row_len(pairs, f) + 1 - 4 * pairs

    def step_at(self, i):
        k = 0
        for first, step in self.changes:
            if first <= i:
                k = step
        return k

    def _last_fill(self, rng, pairs):
        fs = [f for p, f in self.steps if p == pairs] or self.fills
        if self.far_frac is None:
            return fs[int(rng.integers(0, len(fs)))]
        far = [f for f in fs if self.real_fill(pairs, f) + 2 > self.far_win]
        near = [f for f in fs if f not in far]
        pool = (far if rng.random() < self.far_frac else near) if far and near else fs
        return pool[int(rng.integers(0, len(pool)))]

    def _draw(self, i):
        """(generator of batch i, pairs, nominal fill): the one place that decides what batch i looks like."""
        k = self.step_at(i)
        pairs, f = self.steps[k]
        rng = np.random.default_rng([self.h.seed, 7919, i])
        if k == len(self.steps) - 1:
            f = self._last_fill(rng, pairs)
        return rng, pairs, f

    def shape_at(self, i):
        """(pairs, true fill) of batch i, for accuracy logs split by distance."""
        _, pairs, f = self._draw(i)
        return pairs, self.real_fill(pairs, f)

    def observe(self, i, hits, n_ans):
        self.hits += hits
        self.answers += n_ans
        k = self.changes[-1][1]
        if self.answers < self.h.win or k >= len(self.steps) - 1:
            return None
        acc = self.hits / self.answers
        self.hits = self.answers = 0.0
        if acc < self.h.thr:
            return None
        first = i + self.h.lag
        self.changes.append((first, k + 1))
        pairs, f = self.steps[k + 1]
        last = " (last: all lengths mixed)" if k + 1 == len(self.steps) - 1 else ""
        return f"episodes: step {k} -> {k + 1} (accuracy {acc:.3f}), from batch {first} pairs {pairs} filler {f}{last}"

    def state(self):
        return {"pchanges": [list(c) for c in self.changes], "pacc_h": self.hits, "pacc_n": self.answers}

    def load(self, st):
        if "pchanges" in st:
            self.changes = [tuple(c) for c in st["pchanges"]]
            self.hits, self.answers = st["pacc_h"], st["pacc_n"]

    # ------------------------------------------------------------------------------------------------ batches
    def _facts(self, rng, pairs):
        h = self.h
        keys = h.k0 + rng.permutation(h.n_keys)[:pairs]
        vals = h.v0 + rng.integers(0, h.n_vals, pairs)
        return keys, vals, rng.permutation(pairs)

    def batch(self, shape, i):
        """Batch i of the stage: (xy (R, Ts+1) int32, extras).  `shape` is the (B, T+1) of a normal batch."""
        h = self.h
        B, T1 = shape
        rng, pairs, f = self._draw(i)
        if self.rank:                                   # the shape is decided above, identically on every rank
            rng = np.random.default_rng([h.seed, 7919, i, self.rank])
        Ts = self.row_len(pairs, f)
        if not self.tail:
            f = Ts + 1 - 4 * pairs
        R = max(self.rows_mult, (B * (T1 - 1) // Ts) // self.rows_mult * self.rows_mult)
        xy = np.empty((R, Ts + 1), np.int32)
        if self.tail:                                   # what follows the questions carries no loss: filler
            xy[:] = h._filler(rng, R * (Ts + 1)).reshape(R, Ts + 1)
        q0 = 2 * pairs + f
        ans = q0 + 2 * np.arange(pairs)
        rem = np.zeros((R, Ts), np.int8)
        rem[:, ans] = 1
        vals_of = np.full((R, h.n), -1, np.int32)
        rem_y = np.zeros((R, Ts), np.int32)
        for r in range(R):
            keys, vals, order = self._facts(rng, pairs)
            xy[r, :2 * pairs] = np.stack([keys, vals], 1).reshape(-1)
            xy[r, 2 * pairs:q0] = h._filler(rng, f)
            xy[r, q0:q0 + 2 * pairs] = np.stack([keys[order], vals[order]], 1).reshape(-1)
            vals_of[r, :pairs] = vals
            if h.blank:
                rem_y[r, ans] = vals[order]
                xy[r, ans + 1] = h.mark
        extra = {"rem": rem}
        if self.strict:
            extra["rem_vals"] = vals_of
        if h.blank:
            extra["rem_y"] = rem_y
        return xy, extra

    def fill_row(self, row, rng, pairs, f):
        """Overwrite `row` (already filler) with as many episodes as fit, flush to the end of the row; returns the
        positions of the question keys."""
        h, g = self.h, self.gap
        T1, Le = len(row), 4 * pairs + f
        ne = min((T1 + g) // (Le + g), h.n_keys // pairs)            # no key twice in a row
        start = T1 - (ne * Le + (ne - 1) * g)
        if g:
            row[:start] = h.mark
        perms = [rng.permutation(h.n_keys) for _ in range(-(-ne * pairs // h.n_keys))]
        keys = (h.k0 + np.concatenate(perms))[:ne * pairs].reshape(ne, pairs)
        vals = h.v0 + rng.integers(0, h.n_vals, (ne, pairs))
        found = []
        for e in range(ne):
            b0 = start + e * (Le + g)
            if g and e:
                row[b0 - g:b0] = h.mark
            order = rng.permutation(pairs)
            row[b0:b0 + 2 * pairs] = np.stack([keys[e], vals[e]], 1).reshape(-1)
            q0 = b0 + 2 * pairs + f
            row[q0:q0 + 2 * pairs] = np.stack([keys[e][order], vals[e][order]], 1).reshape(-1)
            found.append(q0 + 2 * np.arange(pairs))
        return np.concatenate(found)
