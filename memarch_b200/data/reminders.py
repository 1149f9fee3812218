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


def _interleave(a, b):
    """[a0 b0 a1 b1 ...]"""
    return np.stack([a, b], 1).reshape(-1)


class Ladder:
    """Success-driven levels: `observe` adds up hits and answers; once at least `win` answers are in, an accuracy of
    `thr` or more opens the next level `lag` batches later (beyond the prefetch depth, so the producer thread and the
    training loop agree on which batch is the first of the new level)."""

    def __init__(self, n_levels, thr, win, lag):
        self.n_levels, self.thr, self.win, self.lag = n_levels, thr, win, lag
        self.changes = [(0, 0)]                      # (first batch, level)
        self.hits = self.answers = 0.0

    def at(self, i):
        level = 0
        for first, lv in self.changes:
            if first <= i:
                level = lv
        return level

    def observe(self, i, hits, n_ans):
        """-> (accuracy, new level, its first batch) when a level is passed, else None."""
        self.hits += hits
        self.answers += n_ans
        cur = self.changes[-1][1]
        if self.answers < self.win or cur >= self.n_levels - 1:
            return None
        acc, self.hits, self.answers = self.hits / self.answers, 0.0, 0.0
        if acc < self.thr:
            return None
        self.changes.append((i + self.lag, cur + 1))
        return acc, cur + 1, i + self.lag


class Reminders:
    def __init__(self, p, T, n=16, dist=2048, tok0=1000, seed=0, V=None, p0=None, warm=0, decay=0, ladder=None,
                 thr=0.9, win=800, lag=5, dmin=0, synth=0, doc_eos=None, near=0.0, near_max=0, blank=False,
                 per_row=1, far_log=None, same_fmt=False, pack=None, mix=None):
        """`pack`: None, True or a dict of `Episodes` options."""
        # what a needle looks like
        self.T, self.n, self.dist, self.seed, self.V = int(T), int(n), int(dist), int(seed), V
        self.n_keys, self.n_vals = N_KEYS, N_VALS
        self.k0, self.v0, self.mark = tok0, tok0 + N_KEYS, tok0 + N_KEYS + N_VALS
        self.L = 2 * self.n + 2                      # one block with markers: M, n (key, value) pairs, M
        self.blank, self.same_fmt = bool(blank), bool(same_fmt)
        eos = -1 if doc_eos is None else int(doc_eos)
        self.doc_eos = eos if eos >= 0 else None
        # how often and how far
        self.p, self.p0, self.warm, self.decay = float(p), (None if p0 is None else float(p0)), int(warm), int(decay)
        self.dmin, self.near, self.near_max = int(dmin), float(near), int(near_max)
        self.per_row, self.far_log = int(per_row), (None if far_log is None else float(far_log))
        self.rungs = sorted(int(v) for v in ladder) if ladder else None
        self.thr, self.win, self.lag = float(thr), int(win), int(lag)
        self._ladder = Ladder(len(self.rungs) if self.rungs else 1, self.thr, self.win, self.lag)
        # the synthetic stage
        self.synth = int(synth)
        self.mix_shares, self.mix_len = (list(mix[0]), int(mix[1])) if mix else (None, 250)
        room = self.T + 1 - 2 * self.L
        if V is not None and self.mark >= V:
            raise ValueError(f"needle tokens {tok0}..{self.mark} do not fit a vocabulary of {V}")
        if self.n > N_KEYS:
            raise ValueError("more pairs than distinct keys")
        if self.dist > room:
            raise ValueError(f"T={T} too short for two blocks of {self.L} and a distance of {dist}")
        if self.rungs and self.rungs[-1] > room:
            raise ValueError(f"ladder {self.rungs} exceeds the row")
        self.pack = Episodes(self, **(pack if isinstance(pack, dict) else {})) if pack else None

    # the ladder's bookkeeping under the names checkpoints and callers use
    ladder = property(lambda self: self.rungs)
    changes = property(lambda self: self._ladder.changes)

    # ------------------------------------------------------------------------------------------------ schedule
    def p_at(self, i):
        """Share of rows with a needle at batch i: p0 during the warm-up, then linearly to p over `decay` batches."""
        if self.p0 is None:
            return self.p
        t = min(1.0, max(0, i - self.warm) / max(self.decay, 1)) if i >= self.warm else 0.0
        return self.p0 + (self.p - self.p0) * t

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
        return self._ladder.at(i)

    def range_at(self, i):
        """Distances of batch i: the level's own band; the last level mixes all distances (short ones are not forgotten)."""
        lv, top = self.level_at(i), len(self.rungs) - 1
        low = self.dmin if lv in (0, top) else self.rungs[lv - 1]
        return low, self.rungs[lv]

    def observe(self, i, hits, n_ans):
        """After step i: needle accuracy of the training batch -> maybe a level change; returns a log line or None."""
        if self.pack is not None and self.synth_at(i):
            return self.pack.observe(i, hits, n_ans)
        if not self.rungs:
            return None
        passed = self._ladder.observe(i, hits, n_ans)
        if passed is None:
            return None
        acc, lv, first = passed
        lo, hi = self.range_at(first)
        return f"reminders: level {lv - 1} -> {lv} (accuracy {acc:.3f}), from batch {first} distance {lo}..{hi}"

    def state(self):
        st = {"changes": [list(c) for c in self._ladder.changes], "acc_h": self._ladder.hits, "acc_n": self._ladder.answers}
        if self.pack is not None:
            st.update(self.pack.state())
        return st

    def load(self, st):
        self._ladder.changes = [tuple(c) for c in st["changes"]]
        self._ladder.hits, self._ladder.answers = st["acc_h"], st["acc_n"]
        if self.pack is not None:
            self.pack.load(st)

    # ------------------------------------------------------------------------------------------------ tokens
    def _filler(self, rng, n):
        """Random words outside the needle tokens (and never the end-of-document token)."""
        span = self.mark + 1 - self.k0
        words = rng.integers(0, (self.V or (self.mark + 20001)) - span, n)
        words = np.where(words >= self.k0, words + span, words).astype(np.int32)
        if self.doc_eos is not None:
            words[words == self.doc_eos] = 0
        return words

    def _scrub(self, part, rng, which):
        """Replace the flagged words of `part` by filler (draws only when something is flagged)."""
        if which.any():
            part[which] = self._filler(rng, int(which.sum()))

    def _no_stray_needle_words(self, row, rng):
        # needle tokens are ordinary words of real text (5-7 % of a row): outside the needle they would look like facts
        self._scrub(row, rng, (row >= self.k0) & (row <= self.mark))

    def _one_document(self, row, rng, lo, hi):
        # a document boundary between facts and questions would hide the facts from a reader that stops at boundaries
        if self.doc_eos is not None:
            part = row[lo:hi]
            self._scrub(part, rng, part == self.doc_eos)

    # ------------------------------------------------------------------------------------------------ needles
    def _needle(self, row, rng, exact=None, level_range=None):
        """One needle into `row`; returns the positions of the question keys in x (y there is the value)."""
        n, L, T1 = self.n, self.L, len(row)
        keys = self.k0 + rng.permutation(N_KEYS)[:n]
        vals = self.v0 + rng.integers(0, N_VALS, n)
        if exact is None and level_range is not None:
            exact = int(rng.integers(level_range[0], level_range[1] + 1))
        if exact is not None:
            if not 0 <= exact <= T1 - 2 * L:
                raise ValueError(f"distance {exact} does not fit a row of {T1}")
            s = int(rng.integers(0, T1 - 2 * L - exact + 1))
            q = s + L + exact
        else:                                        # anywhere, at least `dist` words apart
            s = int(rng.integers(0, T1 - 2 * L - self.dist + 1))
            q = int(rng.integers(s + L + self.dist, T1 - L + 1))
        asked = rng.permutation(n)
        facts, asks = _interleave(keys, vals), _interleave(keys[asked], vals[asked])
        if self.same_fmt:                            # the marker-free format of the synthetic episodes
            self._no_stray_needle_words(row, rng)
            first = q
            for at, block in ((s, facts), (q, asks)):
                row[at:at + 2 * n] = block
        else:
            first = q + 1
            for at, block in ((s, facts), (q, asks)):
                row[at] = row[at + L - 1] = self.mark
                row[at + 1:at + L - 1] = block
        self._one_document(row, rng, s, q + L)
        return first + 2 * np.arange(n)

    def _several(self, row, rng):
        """Several needles in one row of text, without markers: facts `[k v]*n`, questions `[k v]*n` in another order.
        All keys of the row are distinct, blocks do not overlap (a needle may lie inside another, as in a
        conversation), and the needle tokens occur nowhere else in the row.  Distance: with probability `far_log`
        (default 1 - near) log-uniform between `dist` and the end of the row, otherwise 0..near_max."""
        n, T1, width = self.n, len(row), 2 * self.n
        self._no_stray_needle_words(row, rng)
        count = max(1, min(self.per_row, N_KEYS // n))
        key_pool = self.k0 + rng.permutation(N_KEYS)[:count * n]
        busy = np.zeros(T1, bool)
        longest = T1 - 2 * width
        p_far = self.far_log if self.far_log is not None else 1.0 - self.near
        shortest_far = max(1, min(self.dist, longest))
        questions = []
        for j in range(count):
            for _ in range(32):                      # a few tries to find free room
                if rng.random() < p_far:
                    d = int(np.exp(rng.uniform(np.log(shortest_far), np.log(longest + 1))))
                    d = min(max(d, shortest_far), longest)
                else:
                    d = int(rng.integers(0, min(self.near_max, longest) + 1))
                s = int(rng.integers(0, longest - d + 1))
                q = s + width + d
                if busy[s:s + width].any() or busy[q:q + width].any():
                    continue
                keys = key_pool[j * n:(j + 1) * n]
                vals = self.v0 + rng.integers(0, N_VALS, n)
                asked = rng.permutation(n)
                row[s:s + width], row[q:q + width] = _interleave(keys, vals), _interleave(keys[asked], vals[asked])
                busy[s:s + width] = busy[q:q + width] = True
                self._one_document(row, rng, s, q + width)
                questions.append(q + 2 * np.arange(n))
                break
        return np.sort(np.concatenate(questions)) if questions else np.zeros(0, np.int64)

    def _text_row(self, row, rng, p, exact, level_range):
        """A row of real text: with probability p it gets a needle (or several).  -> question positions or None."""
        if not rng.random() < p:
            return None
        many = self.per_row > 1 or self.far_log is not None            # that form draws its own near / far distances
        if exact is None and not many and self.near > 0 and self.near_max > 0 and rng.random() < self.near:
            exact = int(rng.integers(0, min(self.near_max, len(row) - 2 * self.L) + 1))
        if exact is None and level_range is None and many:
            return self._several(row, rng)
        return self._needle(row, rng, exact, None if exact is not None else level_range)

    def __call__(self, xy, p=None, exact=None, n=None, synth=None, pack=None):
        """xy (B, T+1) tokens -> (xy with needles, {"rem": (B, T) int8}).  `n` = number of the training batch."""
        synth = self.synth_at(n) if synth is None else synth
        level_range = None
        if n is not None and p is None:              # a training batch: its share and its level come from its number
            p = self.p_at(n)
            level_range = self.range_at(n) if self.rungs else None
        elif p is None:
            p = self.p
        if synth and self.pack is not None and n is not None and pack is None:
            return self.pack.batch(xy.shape, n)
        dense = (self.pack or Episodes(self)) if synth and pack is not None else None
        xy = np.array(xy, copy=True)
        rows, T1 = xy.shape
        rem = np.zeros((rows, T1 - 1), np.int8)
        rem_y = np.zeros((rows, T1 - 1), np.int32) if self.blank else None
        for r in range(rows):
            row = xy[r]
            rng = np.random.default_rng([self.seed, zlib.crc32(row.tobytes())])      # same row -> same needle
            hide = self.same_fmt
            if synth:
                row[:] = self._filler(rng, T1)
                if dense is not None:
                    asked, hide = dense.fill_row(row, rng, *pack), True
                else:
                    asked = self._needle(row, rng, exact, level_range)
            else:
                asked = self._text_row(row, rng, p, exact, level_range)
            if asked is None:
                continue
            rem[r, asked] = 1
            if self.blank:                           # the answers go to the target; the text shows them only with markers
                rem_y[r, asked] = row[asked + 1]
                if hide:
                    row[asked + 1] = self.mark
        return xy, ({"rem": rem, "rem_y": rem_y} if self.blank else {"rem": rem})

    @staticmethod
    def score(logits_argmax, xy, rem):
        """(hits, answers) of a batch: predictions at the marked positions against the values that follow."""
        asked = np.asarray(rem) > 0
        right = np.asarray(logits_argmax)[asked] == np.asarray(xy)[:, 1:][asked]
        return float(right.sum()), float(asked.sum())


class KindCorpus:
    """Every batch of a step comes from one kind of text.  `kinds`: {kind: {source: weight}}; `pools`: the layer sets
    per kind (`models.fishki.pools`).  The kind of a step is the one furthest behind its share (depends on the step
    number only, so all processes agree); the combination of `c` layers is drawn from the kind's pool by
    (seed, step); `full=True` uses the whole pool in its order.  `extra()` -> {"kind": (B,1), "fish": (B,c)}."""

    def __init__(self, kinds, pools, c, root, seq=8192, seed=0, rank=0, world=1, eos=None, doc_seed=None):
        from .loader import ShardCorpus
        self.names = list(kinds)
        weight = np.asarray([sum(kinds[name].values()) for name in self.names], np.float64)
        self.share = weight / weight.sum()
        docs = seed if doc_seed is None else doc_seed             # other documents, same schedule of kinds
        self.subs = [ShardCorpus(kinds[name], root, seq=seq, seed=docs + 7919 * j, rank=rank, world=world, eos=eos)
                     for j, name in enumerate(self.names)]
        self.eos, self.seq = self.subs[0].eos, seq
        self.pools, self.c, self.seed = pools, int(c), seed
        self.full, self.n = False, 0
        self.count = np.zeros(len(self.names))
        self._extra = None

    def _layers(self, kind):
        if self.full:
            return list(self.pools[kind])
        rng = np.random.default_rng([self.seed, 31337, self.n])
        return [int(v) for v in rng.choice(self.pools[kind], self.c, replace=False)]

    def batch(self, B):
        kind = int(np.argmax(self.share * (self.n + 1) - self.count))             # the kind furthest behind its share
        xy = self.subs[kind].batch(B)
        layers = np.asarray(self._layers(kind), np.int32)
        self._extra = {"kind": np.full((B, 1), kind, np.int32), "fish": np.tile(layers, (B, 1))}
        self.count[kind] += 1
        self.n += 1
        return xy

    def extra(self):
        return self._extra

    def state_dict(self):
        return {"subs": [sub.state_dict() for sub in self.subs], "count": self.count.tolist(), "n": self.n}

    def load_state_dict(self, st):
        if st.get("subs") is not None:                            # None: new documents from the start, same schedule
            for sub, saved in zip(self.subs, st["subs"]):
                sub.load_state_dict(saved)
        self.count, self.n = np.array(st["count"], np.float64), int(st["n"])

    def mix(self):
        total = self.count.sum() or 1
        return {name: round(float(c / total), 4) for name, c in zip(self.names, self.count)}
