"""Recall needles in real text (schedule, ladder curriculum, determinism), the per-kind corpus, and the
single-process stand-in for torch.distributed."""
import json
import os

import numpy as np
import pytest
import torch

from memarch_b200.data.reminders import N_KEYS, N_VALS, KindCorpus, Reminders


def rows(B, T1, seed=0, V=30000):
    return np.random.default_rng(seed).integers(0, V, (B, T1)).astype(np.int32)


def check_needle(r, x, rem_row):
    """The marked positions hold question keys, the following tokens their values, and the same (key, value) pairs
    stand in a facts block earlier in the row.  Returns the number of words between the two blocks."""
    pos = np.flatnonzero(rem_row)
    assert len(pos) == r.n
    q = pos[0] - 1
    assert x[q] == r.mark and x[q + r.L - 1] == r.mark
    asked = {int(x[p]): int(x[p + 1]) for p in pos}
    assert len(asked) == r.n and all(r.k0 <= k < r.k0 + N_KEYS and r.v0 <= v < r.v0 + N_VALS for k, v in asked.items())
    starts = [s for s in np.flatnonzero(x[:q] == r.mark) if s + r.L - 1 < q + 1 and x[s + r.L - 1] == r.mark]
    facts = None
    for s in starts:
        kv = x[s + 1:s + r.L - 1].reshape(-1, 2)
        if {int(k): int(v) for k, v in kv} == asked:
            facts = s
    assert facts is not None
    return q - (facts + r.L)


def test_needles_are_well_formed_deterministic_and_scheduled():
    r = Reminders(0.5, T=512, n=4, dist=64, seed=1, V=30000, p0=1.0, warm=3, decay=4)
    assert [r.p_at(i) for i in (0, 2, 3, 5, 7, 100)] == [1.0, 1.0, 1.0, 0.75, 0.5, 0.5]
    xy = rows(16, 513)
    out, ex = r(xy, n=0)                                    # p = 1: every row gets a needle
    assert out.shape == xy.shape and ex["rem"].shape == (16, 512) and ex["rem"].sum() == 16 * 4
    for b in range(16):
        assert check_needle(r, out[b], ex["rem"][b]) >= 64
    out2, ex2 = r(xy, n=0)                                  # same content, same needles
    assert np.array_equal(out, out2) and np.array_equal(ex["rem"], ex2["rem"])
    assert not np.array_equal(xy, out) and np.array_equal(xy, rows(16, 513))       # the input is not modified
    big = rows(400, 513, seed=5)
    _, e = r(big, n=100)                                    # p = 0.5
    share = (e["rem"].sum(1) > 0).mean()
    assert 0.4 < share < 0.6
    _, e = r(big, p=0.0)
    assert e["rem"].sum() == 0


def test_exact_distance_synthetic_rows_and_document_boundaries():
    r = Reminders(1.0, T=256, n=3, dist=16, seed=2, V=5000, tok0=1000, synth=2, doc_eos=7)
    xy = rows(8, 257, V=5000)
    xy[:, ::5] = 7                                          # many document boundaries
    for d in (0, 10, 200):
        out, e = r(xy, p=1.0, exact=d)
        for b in range(8):
            assert check_needle(r, out[b], e["rem"][b]) == d
            pos = np.flatnonzero(e["rem"][b])
            s = pos[0] - 1 - d - r.L
            assert not (out[b, s:pos[0] - 1 + r.L] == 7).any()          # none between the facts and the questions
    out, e = r(xy, n=0)                                     # a synthetic batch: filler + needle
    assert e["rem"].sum() == 8 * 3
    body = out[e["rem"].sum(1) > 0]
    inside = (body >= r.k0) & (body <= r.mark)
    assert inside.sum() == 8 * 2 * r.L                      # needle tokens appear in the two blocks only
    out3, _ = r(xy, n=2)                                    # past the synthetic phase: text is kept
    assert (out3 == xy).mean() > 0.8
    with pytest.raises(ValueError):
        Reminders(1.0, T=32, n=8, dist=64)
    with pytest.raises(ValueError):
        Reminders(1.0, T=256, n=3, dist=16, V=1200)


def test_ladder_levels_follow_success_with_a_lag_and_survive_resume():
    r = Reminders(1.0, T=1024, n=4, dist=16, ladder=[32, 128, 512], thr=0.9, win=100, lag=5, dmin=4, seed=0)
    assert r.range_at(0) == (4, 32)
    xy = rows(6, 1025)
    out, e = r(xy, n=0)
    assert all(4 <= check_needle(r, out[b], e["rem"][b]) <= 32 for b in range(6))
    assert r.observe(0, 50, 60) is None                     # not enough answers yet
    assert r.observe(1, 30, 60) is None                     # 80/120 < 0.9: window restarts
    assert r.observe(2, 60, 60) is None
    msg = r.observe(3, 58, 60)                              # 118/120
    assert msg and "level 0 -> 1" in msg
    assert r.level_at(7) == 0 and r.level_at(8) == 1 and r.range_at(8) == (32, 128)
    out, e = r(xy, n=8)
    assert all(32 <= check_needle(r, out[b], e["rem"][b]) <= 128 for b in range(6))
    st = json.loads(json.dumps(r.state()))
    r2 = Reminders(1.0, T=1024, n=4, dist=16, ladder=[32, 128, 512], thr=0.9, win=100, lag=5, dmin=4, seed=0)
    r2.load(st)
    assert r2.level_at(8) == 1
    assert r2.observe(9, 100, 100) and r2.range_at(14) == (4, 512)        # last level: all distances
    assert r2.observe(20, 100, 100) is None                               # nothing above the last level
    near = Reminders(1.0, T=1024, n=4, dist=256, near=1.0, near_max=8)
    out, e = near(xy)
    assert all(check_needle(near, out[b], e["rem"][b]) <= 8 for b in range(6))
    hits, n_ans = Reminders.score(out[:, 1:], out, e["rem"])              # a perfect predictor
    assert hits == n_ans == 24
    hidden = Reminders(1.0, T=1024, n=4, dist=256, blank=True, same_fmt=True)
    plain = Reminders(1.0, T=1024, n=4, dist=256, same_fmt=True)
    oh, eh = hidden(xy)
    op, ep = plain(xy)
    assert np.array_equal(eh["rem"], ep["rem"])
    m = ep["rem"] > 0
    assert (oh[:, 1:][m] == hidden.mark).all() and np.array_equal(eh["rem_y"][m], op[:, 1:][m])   # answers only in rem_y
    assert (eh["rem_y"][~m] == 0).all() and np.array_equal(np.where(m, 0, oh[:, 1:]), np.where(m, 0, op[:, 1:]))
    assert not (op == plain.mark).any()                                   # the marker-free format
    seen = Reminders(1.0, T=1024, n=4, dist=256, blank=True)              # with markers the answers stay in the text
    os_, es = seen(xy)
    ms = es["rem"] > 0
    assert np.array_equal(es["rem_y"][ms], os_[:, 1:][ms]) and (os_[:, 1:][ms] != seen.mark).all()


def test_kind_corpus_schedule_pools_and_resume(tmp_path):
    from memarch_b200.data.loader import write_shard
    from memarch_b200.models.fishki import pools
    rng = np.random.default_rng(0)
    for src, lo in (("web", 0), ("code", 400), ("math", 800)):
        for s in range(2):
            write_shard(str(tmp_path), src, f"s{s}", [rng.integers(lo, lo + 300, size=rng.integers(20, 120))
                                                      for _ in range(30)], 999)
    kinds = {"prose": {"web": 3.0}, "formal": {"code": 1.0, "math": 1.0}}
    sets = pools(2, 8, 5)
    kc = KindCorpus(kinds, sets, c=3, root=str(tmp_path), seq=48, seed=4)
    seen = []
    for _ in range(20):
        xy = kc.batch(4)
        ex = kc.extra()
        k = int(ex["kind"][0, 0])
        seen.append(k)
        assert xy.shape == (4, 49) and ex["kind"].shape == (4, 1) and ex["fish"].shape == (4, 3)
        assert (ex["kind"] == k).all() and (ex["fish"] == ex["fish"][0]).all()
        assert set(ex["fish"][0].tolist()) <= set(sets[k]) and len(set(ex["fish"][0].tolist())) == 3
        lo_tok = xy[xy != 999]
        assert (lo_tok < 300).all() if k == 0 else (lo_tok >= 400).all()       # the whole batch is of one kind
    assert kc.mix() == {"prose": 0.6, "formal": 0.4}
    st = json.loads(json.dumps(kc.state_dict()))
    want = [(kc.batch(4), kc.extra()["fish"].copy()) for _ in range(6)]
    kc2 = KindCorpus(kinds, sets, c=3, root=str(tmp_path), seq=48, seed=4)
    kc2.load_state_dict(st)
    for xy, fish in want:
        assert np.array_equal(kc2.batch(4), xy) and np.array_equal(kc2.extra()["fish"], fish)
    kc2.full = True
    kc2.batch(2)
    assert kc2.extra()["fish"][0].tolist() == list(sets[int(kc2.extra()["kind"][0, 0])])


def test_fake_world_runs_the_multi_rank_paths_in_one_process():
    import torch.distributed as dist
    from memarch_b200.parallel.fake import fake_world
    before = dist.all_reduce
    assert not dist.is_initialized()
    with fake_world() as g:
        assert dist.is_initialized() and dist.get_world_size() == 1 and dist.get_rank() == 0 and g.size() == 1
        t = torch.arange(6.0)
        assert dist.all_reduce(t) is None and dist.all_reduce(t, async_op=True).wait()
        assert torch.equal(t, torch.arange(6.0))
        out = [torch.zeros(6)]
        dist.all_gather(out, t)
        assert torch.equal(out[0], t)
        big = torch.zeros(6)
        dist.all_gather_into_tensor(big, t)
        dist.broadcast(big, 0)
        assert torch.equal(big, t)
        rs = torch.zeros(6)
        dist.reduce_scatter_tensor(rs, t)
        a2a = torch.zeros(6)
        dist.all_to_all_single(a2a, t)
        assert torch.equal(rs, t) and torch.equal(a2a, t)
        dist.barrier()
        dist.all_reduce(t, async_op=True).get_future().wait()
        # the engine's NCCL-mode gradient path, world of one
        from memarch_b200.parallel import ParallelEngine
        eng = ParallelEngine(0, 1, fused=False)
        assert eng.W == 1
    assert dist.all_reduce is before and not dist.is_initialized()


def test_heldout_tail_is_disjoint_from_training_and_is_the_eval_split(tmp_path):
    from memarch_b200.data.loader import ShardCorpus, heldout_tail, write_shard
    assert heldout_tail(np.array([10] * 50), 25) == 3 and heldout_tail(np.array([10] * 50), 10 ** 9) == 5
    assert heldout_tail(np.array([10] * 4), 0) == 0 and heldout_tail(np.array([7, 7, 7]), 5) == 1
    rng = np.random.default_rng(0)
    uid = 1000                                               # every document starts with its own id
    docs_of = {}
    for s in range(3):
        dd = []
        for _ in range(40):
            dd.append(np.concatenate([[uid], rng.integers(0, 900, size=rng.integers(5, 30))]))
            uid += 1
        docs_of[s] = dd
        write_shard(str(tmp_path), "web", f"s{s}", dd, 999, score=rng.uniform(2.6, 4.0, size=40) if s == 2 else None)
    tail_ids = {int(d[0]) for d in docs_of[2][-4:]}          # a tenth of the last shard
    ev = ShardCorpus({"web": 1.0}, str(tmp_path), seq=31, heldout_tok=10 ** 9, split="eval")
    flat = ev.batch(2).reshape(-1)
    ids = [int(t) for t in flat if t >= 1000]
    assert set(ids) <= tail_ids and len(set(ids)) >= 2
    first_epoch = ids[:4]
    assert len(set(first_epoch)) == len(first_epoch)         # no quality repeats in evaluation
    tr = ShardCorpus({"web": 1.0}, str(tmp_path), seq=31, heldout_tok=10 ** 9)
    seen = set()
    for _ in range(80):
        seen |= {int(t) for t in tr.batch(4).reshape(-1) if t >= 1000}
    assert not (seen & tail_ids) and len(seen) == 120 - 4    # everything but the tail is trained on
    both = ShardCorpus({"web": 1.0}, str(tmp_path), seq=31)
    seen = set()
    for _ in range(80):
        seen |= {int(t) for t in both.batch(4).reshape(-1) if t >= 1000}
    assert tail_ids <= seen                                  # without the switch nothing is held out


def test_several_marker_free_needles_per_row():
    r = Reminders(1.0, T=2048, n=4, dist=64, per_row=3, near=0.3, near_max=16, seed=3, V=30000)
    xy = rows(12, 2049, seed=9)
    xy[:, 100:110] = r.k0 + 5                                       # stray needle tokens in the text
    out, e = r(xy)
    total = 0
    for b in range(12):
        pos = np.flatnonzero(e["rem"][b])
        assert len(pos) % 4 == 0 and 4 <= len(pos) <= 12
        total += len(pos)
        keys = out[b, pos]
        assert len(set(keys.tolist())) == len(keys)                  # all keys of the row differ
        in_range = (out[b] >= r.k0) & (out[b] <= r.mark)
        assert in_range.sum() == 4 * len(pos) and not (out[b] == r.mark).any()      # facts + questions only, no markers
        for p_ in pos:                                               # every question has its fact earlier in the row
            k, v = out[b, p_], out[b, p_ + 1]
            earlier = np.flatnonzero(out[b, :p_] == k)
            assert len(earlier) == 1 and out[b, earlier[0] + 1] == v
    assert total >= 12 * 8                                           # most rows get two or three needles
    out2, e2 = r(xy)
    assert np.array_equal(out, out2) and np.array_equal(e["rem"], e2["rem"])
    one = Reminders(1.0, T=2048, n=4, dist=64, far_log=1.0, seed=3)
    o1, e1 = one(xy)
    for b in range(12):
        pos = np.flatnonzero(e1["rem"][b])
        assert len(pos) == 4
        first_fact = min(int(np.flatnonzero(o1[b, :p_] == o1[b, p_])[0]) for p_ in pos)
        assert pos[0] - (first_fact + 8) >= 64                       # far needles keep the minimum distance


def test_episode_stage_curriculum_and_rows():
    r = Reminders(1.0, T=1024, n=16, dist=64, seed=5, V=30000, synth=40, thr=0.9, win=50, lag=3, blank=True,
                  pack=dict(round_to=64, rows_mult=2, strict=True), mix=([0.75, 0.25], 10))
    ep = r.pack
    assert ep.steps[:4] == [(4, 16), (8, 16), (16, 16), (4, 32)] and ep.steps[-1][0] == 16
    assert all(4 * 16 + f <= 1025 for _, f in ep.steps)
    shape = (4, 1025)
    xy, ex = r(np.zeros(shape, np.int32), n=0)
    pairs, fill = ep.shape_at(0)
    assert (pairs, fill) == (4, 64 + 1 - 16) and xy.shape == (4 * 1024 // 64, 65) and xy.shape[0] % 2 == 0
    assert set(ex) == {"rem", "rem_vals", "rem_y"} and ex["rem"].shape == (64, 64)
    for row, rem, vals, y in zip(xy, ex["rem"], ex["rem_vals"], ex["rem_y"]):
        facts = dict(zip(row[0:2 * pairs:2], row[1:2 * pairs:2]))
        q = np.nonzero(rem)[0]
        assert len(q) == pairs and len(facts) == pairs and q[0] == 2 * pairs + fill
        assert [facts[k] for k in row[q]] == list(y[q]) and (row[q + 1] == r.mark).all()          # hidden answers
        assert list(vals[:pairs]) == list(row[1:2 * pairs:2]) and (vals[pairs:] == -1).all()
        mid = row[2 * pairs:2 * pairs + fill]
        assert ((mid < r.k0) | (mid > r.mark)).all()
    again, _ = r(np.ones(shape, np.int32), n=0)
    assert np.array_equal(xy, again)                                      # a function of the batch number only
    # the curriculum moves on success, `lag` batches later, and survives a checkpoint
    assert r.observe(0, 10, 60) is None                                   # accuracy too low: the window restarts
    msg = r.observe(1, 60, 60)
    assert "step 0 -> 1" in msg and ep.step_at(3) == 0 and ep.step_at(4) == 1
    assert r(np.zeros(shape, np.int32), n=4)[0].shape[1] == 64 + 1 and ep.shape_at(4)[0] == 8
    r2 = Reminders(1.0, T=1024, n=16, dist=64, seed=5, V=30000, synth=40, thr=0.9, win=50, lag=3, blank=True,
                   pack=dict(round_to=64, rows_mult=2, strict=True))
    r2.load(r.state())
    assert r2.pack.changes == ep.changes and np.array_equal(r2(np.zeros(shape, np.int32), n=4)[0],
                                                            r(np.zeros(shape, np.int32), n=4)[0])
    # last step: the fill of every batch is drawn from all lengths
    ep.changes.append((20, len(ep.steps) - 1))
    assert len({ep.shape_at(i)[1] for i in range(20, 40)}) > 2
    # after the stage a decaying share of the batches stays synthetic
    share = lambda lo, hi: np.mean([r.synth_at(i) for i in range(lo, hi)])
    assert share(0, 40) == 1.0 and share(40, 50) > share(50, 60) > 0 and abs(share(1000, 1400) - 0.25) < 0.03
    assert not Reminders(1.0, T=1024, n=16, dist=64, synth=40).synth_at(40)
    # with `tail` the fill stays nominal and the padding follows the questions
    t = Reminders(1.0, T=1024, n=16, dist=64, seed=5, V=30000, synth=40, pack=dict(round_to=64, tail=True))
    xt, et = t(np.zeros(shape, np.int32), n=0)
    assert t.pack.shape_at(0) == (4, 16) and xt.shape[1] == 65 and np.nonzero(et["rem"][0])[0][0] == 8 + 16
    with pytest.raises(ValueError):
        Reminders(1.0, T=1024, n=16, dist=64, pack=dict(frac=[0.5]))
    # data-parallel ranks: the same shapes (also on the last step, where the fill is drawn per batch), other rows
    mk = lambda rank: Reminders(1.0, T=1024, n=16, dist=64, seed=5, V=30000, synth=40, pack=dict(round_to=64, rank=rank))
    r0, r1 = mk(0), mk(1)
    for rr in (r0, r1):
        rr.pack.changes.append((0, len(rr.pack.steps) - 1))
    for i in range(6):
        a, b = r0(np.zeros(shape, np.int32), n=i)[0], r1(np.zeros(shape, np.int32), n=i)[0]
        assert a.shape == b.shape and not np.array_equal(a, b)


def test_dense_episode_rows_for_evaluation():
    r = Reminders(1.0, T=2048, n=8, dist=64, seed=2, V=30000, pack=dict(gap=3))
    xy = np.random.default_rng(0).integers(0, 900, (3, 2049)).astype(np.int32)
    out, ex = r(xy, synth=True, pack=(4, 32))
    for row, rem in zip(out, ex["rem"]):
        q = np.nonzero(rem)[0]
        assert len(q) == 4 * ((2049 + 3) // (48 + 3))
        keys = row[q]
        assert len(set(keys)) == len(keys)                                 # no key twice in a row
        for e0 in q[::4]:                                                  # every episode: facts, 32 words, questions
            b0 = e0 - 32 - 8
            facts = dict(zip(row[b0:b0 + 8:2], row[b0 + 1:b0 + 8:2]))
            assert [facts[k] for k in row[e0:e0 + 8:2]] == list(row[e0 + 1:e0 + 8:2])
            if b0 >= 3:
                assert (row[b0 - 3:b0] == r.mark).all()


def _reference_data():
    import importlib.util
    root = os.environ.get("MEMARCH_REF_DIR", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                                          "baseline", "_ref"))
    path = os.path.join(root, "memarch_jax", "memarch_jax", "data.py")
    if not os.path.exists(path):
        pytest.skip("reference tree not present")
    spec = importlib.util.spec_from_file_location("reference_data", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("kw,attrs", [
    ({}, {}),
    ({"ladder": [32, 128, 512], "dmin": 4}, {}),
    ({"synth": 3, "doc_eos": 7}, {}),
    ({"near": 0.5, "near_max": 8, "p0": 1.0, "warm": 2, "decay": 4}, {}),
    ({"blank": True}, {}),
    ({"blank": True}, {"same_fmt": True}),
    ({"blank": True, "near": 0.3, "near_max": 16}, {"same_fmt": True, "per_row": 3}),
    ({}, {"far_log": 1.0}),
    ({"synth": 6, "pack": True}, {}),
    ({"synth": 6, "pack": True, "blank": True, "strict": True, "pack_round": 64, "pack_mult": 2}, {}),
    ({"synth": 6, "pack": True, "tail": True, "pack_round": 128}, {}),
    ({"synth": 6, "pack": True, "pack_round": 64, "pack_frac": [0.05, 0.1, 0.25, 0.5, 1.0], "win_ref": 512}, {}),
    ({"synth": 6, "pack": True}, {"far_frac": 0.7, "far_win": 100, "mix_fracs": [0.9, 0.5], "mix_len": 3}),
])
def test_same_batches_as_the_reference(kw, attrs):
    """Needles, masks, schedules and curriculum steps equal the reference's host-side injector bit for bit."""
    ref = _reference_data()
    a = ref.Reminders(0.7, 1024, n=8, dist=64, seed=3, V=30000, thr=0.5, win=20, lag=2, **kw)
    for k, v in attrs.items():
        setattr(a, k, v)
    ours = {k: v for k, v in kw.items() if k not in ("pack", "strict", "tail", "pack_round", "pack_mult", "pack_frac",
                                                     "win_ref")}
    if kw.get("pack"):
        ours["pack"] = dict(strict=kw.get("strict", False), tail=kw.get("tail", False), round_to=kw.get("pack_round", 1),
                            rows_mult=kw.get("pack_mult", 1), frac=kw.get("pack_frac"), win_ref=kw.get("win_ref"),
                            far_frac=attrs.get("far_frac"), far_win=attrs.get("far_win", 2048))
    if "mix_fracs" in attrs:
        ours["mix"] = (attrs["mix_fracs"], attrs["mix_len"])
    ours.update({k: v for k, v in attrs.items() if k in ("same_fmt", "per_row", "far_log")})
    b = Reminders(0.7, 1024, n=8, dist=64, seed=3, V=30000, thr=0.5, win=20, lag=2, **ours)
    if kw.get("pack"):
        assert b.pack.steps == a.plevels
    g = np.random.default_rng(1)
    for n in range(14):
        xy = g.integers(0, 5000, (4, 1025)).astype(np.int32)
        xa, ea = a(xy, n=n)
        xb, eb = b(xy, n=n)
        assert a.synth_at(n) == b.synth_at(n)
        assert xa.shape == xb.shape and np.array_equal(xa, xb), n
        assert set(ea) == set(eb) and all(np.array_equal(ea[k], eb[k]) for k in ea), n
        hits = float(ea["rem"].sum()) * (0.9 if n % 3 else 0.2)
        assert (a.observe(n, hits, float(ea["rem"].sum())) is None) == (b.observe(n, hits, float(eb["rem"].sum())) is None)
        if kw.get("pack") and a.synth_at(n):
            assert a.pack_fill_at(n) == b.pack.shape_at(n)
    sa, sb = a.state(), b.state()
    assert sa == sb
    xy = g.integers(0, 5000, (2, 1025)).astype(np.int32)
    for call in (dict(exact=100), dict(p=1.0), dict(synth=True, pack=(4, 40))):
        xa, ea = a(xy, **call)
        xb, eb = b(xy, **call)
        assert np.array_equal(xa, xb) and all(np.array_equal(ea[k], eb[k]) for k in ea), call
