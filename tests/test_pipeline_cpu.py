"""Corpus preparation: MinHash dedup, decontamination, code score, tokenizer pruning."""
import os

import numpy as np

from memarch_b200.data import pipeline as pl
from memarch_b200.data import tokprune
from memarch_b200.data.loader import ShardCorpus, write_shard

EOS = 9999


def test_minhash_dedup_keeps_the_priority_copy(tmp_path):
    rng = np.random.default_rng(0)
    docs_a = [rng.integers(0, 5000, size=300) for _ in range(20)]
    near = docs_a[3].copy()
    near[::50] = 7                                             # ~6 of 300 tokens changed: Jaccard of shingles ~0.8+
    docs_b = [rng.integers(0, 5000, size=300) for _ in range(10)] + [near, docs_a[7].copy(), np.array([1, 2])]
    write_shard(str(tmp_path), "wiki", "s0", docs_a, EOS)
    write_shard(str(tmp_path), "web", "s0", docs_b, EOS)
    done = pl.postprocess(str(tmp_path))
    assert len(done) == 2 and pl.postprocess(str(tmp_path)) == []          # restart does nothing
    sig = np.load(tmp_path / "web" / "s0.mh.npy")
    assert sig.shape == (13, 14) and (sig[12] == 0).all()      # a 2-token document has no shingle
    rep = pl.finalize(str(tmp_path), priority=("wiki", "web"))
    drop_web = np.load(tmp_path / "web" / "s0.drop.npy")
    assert 11 in drop_web                                      # exact copy of wiki doc 7 goes, the wiki copy stays
    assert len(np.load(tmp_path / "wiki" / "s0.drop.npy")) == 0
    assert rep["dedup"]["web"][1] >= 1
    c = ShardCorpus({"web": 1.0}, str(tmp_path), seq=64)       # the loader honours the mask
    seen = np.concatenate([c.batch(4).reshape(-1) for _ in range(10)])
    assert seen.size > 0


def test_decontamination_flags_real_copies_only(tmp_path):
    rng = np.random.default_rng(1)
    item = rng.integers(0, 5000, size=80)
    boiler = rng.integers(0, 5000, size=14)                    # a boilerplate line shared by item and corpus
    index = pl.build_bench_index([np.concatenate([item, boiler])], names=["toy"])
    clean = rng.integers(0, 5000, size=400)
    with_boiler = np.concatenate([rng.integers(0, 5000, size=100), boiler, rng.integers(0, 5000, size=100)])
    dirty = np.concatenate([rng.integers(0, 5000, size=50), item, rng.integers(0, 5000, size=50)])
    write_shard(str(tmp_path), "web", "s0", [clean, with_boiler, dirty], EOS)
    pl.postprocess(str(tmp_path), bench_index=index)
    z = np.load(tmp_path / "web" / "s0.contam.npz")
    assert set(np.unique(z["doc"])) == {1, 2}
    rep = pl.finalize(str(tmp_path), bench_index=index)
    assert np.load(tmp_path / "web" / "s0.cdrop.npy").tolist() == [2]
    assert rep["contamination"]["web"] == (3, 1)


def test_code_scorer_fit_and_score(tmp_path):
    rng = np.random.default_rng(2)
    good = [rng.integers(0, 50, size=200) for _ in range(30)]  # "good" repositories use the low token range
    bad = [rng.integers(50, 100, size=200) for _ in range(30)]
    sc = pl.CodeScorer(V=100, H=256).fit(good + bad, [4.0] * 30 + [1.0] * 30, iters=150)
    assert sc.score_doc(rng.integers(0, 50, size=200)) > 3.0 > 2.0 > sc.score_doc(rng.integers(50, 100, size=200))
    sc.save(tmp_path / "cq.npz")
    sc2 = pl.CodeScorer.load(tmp_path / "cq.npz")
    write_shard(str(tmp_path), "stack_v3", "s0", good[:3] + bad[:3], EOS)
    pl.postprocess(str(tmp_path), sources=["stack_v3"], scorer=sc2)
    s = np.load(tmp_path / "stack_v3" / "s0.score.npy")
    assert s.shape == (6,) and s[:3].min() > s[3:].max()


def test_tokenizer_pruning_round_trip():
    bt = sorted(tokprune.byte_tokens())
    assert len(bt) == 256
    vocab = {s: i for i, s in enumerate(bt)}
    merges = []

    def merge(a, b):
        merges.append(f"{a} {b}")
        vocab.setdefault(a + b, len(vocab))
    for a, b in (("t", "h"), ("th", "e"), ("a", "n"), ("an", "d"), ("x", "y"), ("xy", "z"), ("q", "q")):
        merge(a, b)
    tok = {"model": {"vocab": dict(vocab), "merges": merges}, "added_tokens": [{"id": len(vocab), "content": "<eot>"}]}
    V = len(vocab) + 1
    counts = {"en": np.zeros(V, dtype=np.int64), "code": np.zeros(V, dtype=np.int64)}
    counts["en"][vocab["the"]] = 100
    counts["en"][vocab["and"]] = 50
    counts["code"][vocab["xyz"]] = 1
    score = tokprune.weighted_scores(counts, {"en": 4, "code": 1}, V)
    pruned, old2new = tokprune.prune(tok, score, budget=256 + 4)
    kept = set(pruned["model"]["vocab"])
    assert {"the", "th", "and", "an"} <= kept and "xyz" not in kept and "qq" not in kept   # ancestors come along
    assert all(all(p in kept for p in m.split(" ")) and m.replace(" ", "") in kept for m in pruned["model"]["merges"])
    assert sorted(pruned["model"]["vocab"].values()) == list(range(len(kept)))
    assert pruned["added_tokens"][0]["id"] == len(kept) and old2new[len(vocab)] == len(kept)
    bad, n = tokprune.check(pruned, [list("theandxyz"), list("qqthe")])
    assert bad == 0 and n == 2 + 3 + 3                        # the, and, x, y, z | q, q, the
    c = tokprune.sample_counts({"a": [[1, 1, 2]], "b": [[0]]}, 4)
    assert c["a"].tolist() == [0, 2, 1, 0]
