"""CPU parity against the unmodified reference: same state_dict names and shapes, same loss and gradients from the
same weights and tokens, same Instinct trajectory.  The reference runs in a child process (`ref_oracle.py`) because
it reads its switches from the environment at import time.  Skipped when no reference tree is on disk."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("MEMARCH_REF_DIR", os.path.join(ROOT, "baseline", "_ref"))
pytestmark = pytest.mark.skipif(not os.path.exists(os.path.join(REF, "full2.py")), reason="reference tree not present")


def oracle(tmp_path, spec):
    out = str(tmp_path / "ref.pt")
    env = {k: v for k, v in os.environ.items() if k not in ("PYTHONPATH",)}
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "ref_oracle.py"), REF, out, json.dumps(spec)],
                       capture_output=True, text=True, env=env, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    return torch.load(out)


def artefacts(tmp_path, d, vocab, phr_v, k, n_succ=8, tokens=60_000, text_len=256):
    from memarch_b200.data import phrasebook
    from memarch_b200.data.synth import MarkovCorpus
    toks = MarkovCorpus(vocab=phr_v, n_succ=n_succ, seed=0).stream(tokens, text_len=text_len, seed=1)
    cnt = phrasebook.token_counts(toks, vocab)
    np.save(tmp_path / "token_counts.npy", cnt)
    ph = phrasebook.bigram_init(toks, d, phr_v)
    torch.save(ph, tmp_path / "bigram.pt")
    torch.save(phrasebook.phrase_table(toks, ph["head"], k, phr_v), tmp_path / "trigram.pt")
    torch.save(phrasebook.lock_trust(toks, vocab, cnt, T=128), tmp_path / "lock_trust.pt")
    return {"PHRASE_INIT": str(tmp_path / "bigram.pt"), "PHRASE3": str(tmp_path / "trigram.pt"), "SURP_PHRASE": "1",
            "INDUCT": "lock", "LOCK_TRUST": str(tmp_path / "lock_trust.pt"), "INDUCT_IN": "1", "INDUCT_MIX": "1",
            "TOKEN_COUNTS": str(tmp_path / "token_counts.npy"), "PHR_V": str(phr_v), "VOCAB": str(vocab)}, toks


def compare(d, m, rtol=2e-4):
    sd, ours = d["sd"], m.state_dict()
    assert sorted(sd) == sorted(ours)
    assert all(sd[k].shape == ours[k].shape and sd[k].dtype == ours[k].dtype for k in sd)
    m.load_state_dict(sd)
    m.train()
    xy = d["xy"]
    out, cost = m(xy[:, :-1])
    loss = m.train_loss(out, xy[:, 1:], True)
    assert abs(loss.item() - d["loss"].item()) < 2e-5 * max(1, abs(d["loss"].item()))
    assert abs(float(cost) - float(d["cost"])) < 1e-5
    (loss + 0.01 * cost.float()).backward()
    for n, p in m.named_parameters():
        g = d["grads"].get(n)
        assert (g is None) == (p.grad is None), n
        if g is None:
            continue
        scale = g.float().abs().max().item()
        if scale < 1e-7:                        # gate/importance scalars whose gradient is numerical dust in both
            assert p.grad.float().abs().max().item() < 1e-6, n
            continue
        tol = 2e-2 if g.dtype == torch.bfloat16 else rtol
        assert (p.grad.float() - g.float()).abs().max().item() <= tol * scale, n
    if d["tau"] is not None:
        assert abs(float(m.tau) - float(d["tau"])) < 1e-5
    for k in ("anchors", "moe_drop"):
        if not hasattr(m, "stats"):
            break
        if k in d["stats"] and k in m.stats:
            assert abs(float(m.stats[k]) - float(d["stats"][k])) < 1e-5, k


@pytest.mark.parametrize("name,env,T", [
    ("Fv2moeKs8", {}, 128),                                       # memory v2 + reread + bank MoE, SwiGLU experts
    ("Fv2moeKs8", {"MOE_ACT": "relu2", "NO_MEM": "1"}, 128),      # relu^2 experts, memory off
    ("Fv2s_nomem", {"ATTN_IMPL": "block"}, 160),                  # sliding window shorter than the text, ragged tail
    ("Fv2s", {"ATTN_IMPL": "block"}, 256),                        # dense heavy stack; memory demotes and prunes
    ("Fv3s", {"ATTN_IMPL": "block"}, 256),                        # volume memory (v3): pieces, merge on prune
    ("Fv2moeKs8", {"LIGHT_MOE": "8:2", "NO_MEM": "1"}, 64),       # light layers with their own small MoE
    ("Fv2moeKs8", {"HEAVY_ATTN": "1", "NO_MEM": "1"}, 64),        # anchors look back into the light states
    ("Fv2moeKs8", {"REREAD_SEP": "1", "REREAD_ANCH": "0.25", "ATTN_IMPL": "block"}, 160),                  # only the surprising words re-read; ragged last segment
])
def test_model_matches_reference(tmp_path, name, env, T):
    from memarch_b200.build import build
    d = oracle(tmp_path, {"what": "model", "name": name, "vocab": 512, "B": 2, "T": T, "env": env, "stable_sort": True})
    torch.manual_seed(0)
    compare(d, build(name, 512, env=env))


@pytest.mark.parametrize("name,T", [
    ("cards", 64), ("tail", 64), ("plan8", 64), ("planw8", 64), ("planwc8", 64), ("sketch8", 64),
    ("surp20", 64), ("surpc20", 64), ("surpq20", 128), ("surpcx20", 64), ("img_full", 64), ("transformer", 64),
])
def test_legacy_models_match_reference(tmp_path, name, T):
    """The earlier model generations: same names, same loss and gradients from the reference's weights."""
    from memarch_b200.build import build
    d = oracle(tmp_path, {"what": "model", "name": name, "vocab": 300, "B": 2, "T": T, "env": {"FAKE_IMAGES": "1"}})
    torch.manual_seed(0)
    m = build(name, 300)
    if name == "transformer":
        assert sorted(d["sd"]) == sorted(m.state_dict())
        return
    compare(d, m, rtol=5e-4)


def test_recipe_model_matches_reference(tmp_path):
    """The published switches: phrasebook init, phrase table, locks with trust, pointer mixture, fused CE."""
    from memarch_b200.build import build
    env, _ = artefacts(tmp_path, 256, 512, 500, 2048)
    env.update({"MOE_ACT": "relu2", "NO_MEM": "1", "WAVE_WARM": "1000000"})   # FUSED=ours is Triton in the reference: GPU only
    d = oracle(tmp_path, {"what": "model", "name": "Fv2moeKs8", "vocab": 512, "B": 2, "T": 128, "env": env})
    compare(d, build("Fv2moeKs8", 512, env=env), rtol=1e-3)


@pytest.mark.parametrize("kw", [
    {"norm": "hs", "scale": 0.12, "rel_every": 2},
    {"norm": "hs", "scale": 0.12, "m_bf16": True, "rel_every": 2},
    {},
])
def test_instinct_matches_reference(tmp_path, kw):
    from memarch_b200.config import OptConfig
    from memarch_b200.optim.instinct import Instinct
    shapes = [(64, 32), (4, 32, 48), (100, 16), (16,), ()]
    spec = {"what": "instinct", "shapes": shapes, "lr": 1e-2, "kw": kw, "steps": 5, "d": 32}
    d = oracle(tmp_path, spec)
    ps = [torch.nn.Parameter(w.clone()) for w in d["w0"]]
    opt = Instinct(ps, OptConfig(lr=1e-2, **kw))
    for step, (gs, sit) in enumerate(d["gs"]):
        opt.prepare(torch.tensor(3.0 - 0.1 * step), sit)
        for p, g in zip(ps, gs):
            p.grad = g.clone()
            opt.update(p)
            p.grad = None
        opt.finish()
        for p, w in zip(ps, d["ws"][step]):
            tol = 2e-2 if kw.get("m_bf16") else 1e-5        # bf16 momentum is stochastically rounded: different streams
            assert (p.detach() - w).abs().max().item() <= tol * max(w.abs().max().item(), 1e-3), (step, tuple(p.shape))
    if not kw.get("m_bf16"):
        assert torch.allclose(opt.gain, d["gain"], atol=1e-5)
        assert torch.allclose(opt.rel, d["rel"], atol=1e-5)


def test_loss_curve_matches_reference(tmp_path):
    """The tiny configuration of the benchmark list (d=256, 4 heads, 2+2 light, 2 heavy MoE layers of 4 SwiGLU experts,
    phrasebook + phrase table + locks, memory off, Instinct with homeostasis), trained from the reference's initial
    weights on the reference's batches: the two loss curves stay together.  The reference autocasts to bf16 on CPU,
    this build computes in fp32 there, hence a tolerance rather than equality."""
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.config import opt_from_env
    from memarch_b200.train import Trainer
    env, toks = artefacts(tmp_path, 256, 2048, 2000, 4096)
    np.save(tmp_path / "tokens.npy", toks.astype(np.int32))
    okw = {"norm": "hs", "scale": 0.12, "rel_every": 4}
    env.update({"NO_MEM": "1", "LIGHT": "2", "WAVE_WARM": "1000000", "WARMUP": "5", "OPT_KW": json.dumps(okw)})
    steps = 16
    d = oracle(tmp_path, {"what": "train", "name": "Fv2moeK4h2d256", "B": 4, "T": 128, "lr": 3e-3, "steps": steps,
                          "total_steps": 100, "tokens": str(tmp_path / "tokens.npy"), "env": env})
    m = build("Fv2moeK4h2d256", 2048, env=env)
    m.load_state_dict(d["sd"])
    tr = Trainer(m, TrainConfig(name="cfg0", stage="ABX", steps=100, batch=4, micro=4, seq=128, lr=3e-3, warmup=5),
                 opt_from_env(OptConfig(lr=3e-3), env), stage="ABX")
    ours = [float(tr.step(xy, s)) for s, xy in enumerate(d["batches"])]
    ref = d["losses"]
    print("loss curves (ours, reference):", [(round(a, 3), round(b, 3)) for a, b in zip(ours, ref)])
    assert abs(ours[0] - ref[0]) < 0.02
    assert ref[-1] < ref[0] - 0.3 and ours[-1] < ours[0] - 0.3            # both learn
    assert max(abs(a - b) for a, b in zip(ours, ref)) < 0.02, list(zip(ours, ref))


@pytest.mark.skipif(os.environ.get("MEMARCH_SLOW") != "1", reason="minutes of CPU time: set MEMARCH_SLOW=1")
def test_loss_curve_of_the_tiny_benchmark_configuration(tmp_path):
    """The tiny configuration of the benchmark list: d=256, 4 heads, 2+2 light layers (the registry model's window
    covers the whole 512-token text), 2 heavy layers of 4 SwiGLU experts, vocabulary 50257 with phrasebook, phrase table and locks, memory off, Instinct with
    homeostasis; sequence 512, batch 4, 50 steps on seed-0 Markov text (Zipf 1.1, 64 successors, Dirichlet 0.3, 10 %
    copies), from the reference's initial weights on the reference's batches."""
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.config import opt_from_env
    from memarch_b200.train import Trainer
    V = 50257
    env, toks = artefacts(tmp_path, 256, V, V, 65536, n_succ=64, tokens=400_000, text_len=512)
    np.save(tmp_path / "tokens.npy", toks.astype(np.int32))
    okw = {"norm": "hs", "scale": 0.12, "rel_every": 4}
    env.update({"NO_MEM": "1", "LIGHT": "2", "WAVE_WARM": "1000000", "WARMUP": "5", "OPT_KW": json.dumps(okw)})
    steps = 50
    d = oracle(tmp_path, {"what": "train", "name": "Fv2moeK4h2d256", "B": 4, "T": 512, "lr": 3e-3, "steps": steps,
                          "total_steps": 100, "tokens": str(tmp_path / "tokens.npy"), "env": env})
    m = build("Fv2moeK4h2d256", V, env=env)
    m.load_state_dict(d["sd"])
    tr = Trainer(m, TrainConfig(name="cfg0", stage="ABX", steps=100, batch=4, micro=4, seq=512, lr=3e-3, warmup=5),
                 opt_from_env(OptConfig(lr=3e-3), env), stage="ABX")
    ours = [float(tr.step(xy, s)) for s, xy in enumerate(d["batches"])]
    ref = d["losses"]
    print("loss curves (ours, reference):", [(round(a, 3), round(b, 3)) for a, b in zip(ours, ref)])
    assert abs(ours[0] - ref[0]) < 0.02
    assert ref[-1] < ref[0] - 0.3 and ours[-1] < ours[0] - 0.3
    assert max(abs(a - b) for a, b in zip(ours, ref)) < 0.01, list(zip(ours, ref))      # measured: 0.001


def test_tongue_tables_model_matches_reference(tmp_path):
    """The counted "tip of the tongue" tables built here, loaded by both code bases (TONGUE): same loss and gradients,
    the two learned strengths included."""
    from memarch_b200.build import build
    from memarch_b200.data import phrasebook
    env, toks = artefacts(tmp_path, 256, 512, 500, 2048)
    keys = torch.load(tmp_path / "trigram.pt")["keys"]
    tg = phrasebook.tongue_tables(toks, keys.numpy(), vocab=500, k_top=8)
    assert tg["bi_idx"].shape == (500, 8) and tg["tri_idx"].shape == (len(keys), 8) and float(tg["bi_val"].float().max()) > 0
    torch.save(tg, tmp_path / "tongue.pt")
    for k in ("INDUCT", "LOCK_TRUST", "INDUCT_IN", "INDUCT_MIX"):
        env.pop(k)
    env.update({"TONGUE": str(tmp_path / "tongue.pt"), "NO_MEM": "1", "WAVE_WARM": "1000000"})
    d = oracle(tmp_path, {"what": "model", "name": "Fv2moeKs8", "vocab": 512, "B": 2, "T": 128, "env": env})
    m = build("Fv2moeKs8", 512, env=env)
    assert hasattr(m, "tg_a")
    compare(d, m, rtol=1e-3)
    assert m.tg_a.grad is not None and m.tg_a.grad.abs().sum() > 0


def test_short_vocabulary_head_matches_reference(tmp_path):
    """Two-level output head (SHORT_V): frequent words + a "rare" bucket first, the full vocabulary only for a capped
    share of rare targets - loss and gradients against the reference."""
    from memarch_b200.build import build
    from memarch_b200.data.synth import MarkovCorpus
    from memarch_b200.data import phrasebook
    toks = MarkovCorpus(vocab=500, n_succ=8, seed=0).stream(60_000, text_len=256, seed=1)
    np.save(tmp_path / "token_counts.npy", phrasebook.token_counts(toks, 512))
    env = {"SHORT_V": "64", "TOKEN_COUNTS": str(tmp_path / "token_counts.npy"), "NO_MEM": "1", "VOCAB": "512",
           "WAVE_WARM": "1000000"}
    d = oracle(tmp_path, {"what": "model", "name": "Fv2moeKs8", "vocab": 512, "B": 2, "T": 128, "env": env})
    m = build("Fv2moeKs8", 512, env=env)
    assert m.short_v == 64
    compare(d, m, rtol=1e-3)


def test_wave_bookkeeping_follows_the_reference(tmp_path):
    """Bank MoE with the "stopped changing" wave switched on early (warm-up 2 steps, a wave every 3) over a 16-step run
    whose learning rate decays to a tenth, so the experts' movement falls below its peak share and they get marked as
    learned: from the reference's weights on the reference's batches every layer ends with the same `learned` experts
    and the same error / movement statistics."""
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.config import opt_from_env
    from memarch_b200.train import Trainer
    env, toks = artefacts(tmp_path, 256, 2048, 2000, 4096)
    np.save(tmp_path / "tokens.npy", toks.astype(np.int32))
    okw = {"norm": "hs", "scale": 0.12, "rel_every": 4}
    env.update({"NO_MEM": "1", "WAVE_WARM": "2", "WARMUP": "2", "OPT_KW": json.dumps(okw)})
    steps = 16
    d = oracle(tmp_path, {"what": "train", "name": "Fv2moeKs8", "B": 4, "T": 128, "lr": 3e-3, "steps": steps,
                          "total_steps": steps, "tokens": str(tmp_path / "tokens.npy"), "env": env, "wave_every": 3})
    m = build("Fv2moeKs8", 2048, env=env)
    m.load_state_dict(d["sd"])
    for b in m.heavy:
        b.wave_every = 3
    tr = Trainer(m, TrainConfig(name="waves", stage="ABX", steps=steps, batch=4, micro=4, seq=128, lr=3e-3, warmup=2),
                 opt_from_env(OptConfig(lr=3e-3), env), stage="ABX")
    ours = [float(tr.step(xy, s)) for s, xy in enumerate(d["batches"])]
    assert max(abs(a - b) for a, b in zip(ours, d["losses"])) < 0.03, list(zip(ours, d["losses"]))
    sd = m.state_dict()
    moved = 0
    for k, v in d["waves"].items():
        w = sd[k]
        if v.dtype == torch.bool:
            assert torch.equal(w, v), (k, w, v)
            moved += int(v.sum())
        else:
            assert torch.allclose(w.float(), v.float(), rtol=0.15, atol=1e-6), (k, w, v)      # the reference runs bf16 autocast
    assert moved > 0, "no expert was marked as learned: the test did not exercise the waves"


def test_three_word_and_draft_ahead_tables_match_reference(tmp_path):
    """The PHRASE4 and SKIP artefacts built here, loaded by both code bases: same loss and gradients (the tables feed
    the input of the model)."""
    from memarch_b200.build import build
    from memarch_b200.data import phrasebook
    env, toks = artefacts(tmp_path, 256, 512, 500, 2048)
    ph = torch.load(tmp_path / "bigram.pt")
    torch.save(phrasebook.context_table(toks, ph["head"], 1024, 3, 500), tmp_path / "quad.pt")
    torch.save(phrasebook.skip_table(toks, ph["head"], vocab=500), tmp_path / "skip.pt")
    env.update({"PHRASE4": str(tmp_path / "quad.pt"), "SKIP": str(tmp_path / "skip.pt"), "NO_MEM": "1", "WAVE_WARM": "1000000"})
    d = oracle(tmp_path, {"what": "model", "name": "Fv2moeKs8", "vocab": 512, "B": 2, "T": 128, "env": env})
    m = build("Fv2moeKs8", 512, env=env)
    assert hasattr(m, "phr4") and hasattr(m, "skip")
    compare(d, m, rtol=1e-3)


def test_dropless_moe_matches_the_reference_grouped_path(tmp_path):
    """MOE_GMM=1: the reference's dropless grouped-matmul dispatch against this build's dropless capacity form - same
    loss and gradients (nothing is dropped in either)."""
    from memarch_b200.build import build
    env = {"NO_MEM": "1", "WAVE_WARM": "1000000", "MOE_GMM": "1", "VOCAB": "512"}
    try:
        d = oracle(tmp_path, {"what": "model", "name": "Fv2moeKs8", "vocab": 512, "B": 2, "T": 128, "env": env})
    except AssertionError as e:                                  # the reference's grouped matmul may not exist on this CPU build
        pytest.skip("the reference's MOE_GMM path does not run here: " + str(e)[-200:])
    m = build("Fv2moeKs8", 512, env=env)
    assert m.heavy[0].dropless
    compare(d, m, rtol=1e-3)
    assert float(m.stats["moe_drop"]) == 0.0


@pytest.mark.parametrize("bank_q", ["", "int8", "int4"])
def test_frozen_bank_after_rebank_matches_reference(tmp_path, bank_q):
    """Experts 1, 4 and 6 of every bank layer move into the frozen bank (bf16, int8 or int4 storage) by the models' own
    `rebank`; the layer then runs learners and bank side by side: loss and gradients against the reference, the
    learners' weights keeping their gradients and the bank none."""
    from memarch_b200.build import build
    env = {"NO_MEM": "1", "WAVE_WARM": "1000000", "VOCAB": "512", "MOE_ACT": "relu2"}
    if bank_q:
        env["BANK_Q"] = bank_q
    freeze = [1, 4, 6]
    d = oracle(tmp_path, {"what": "model", "name": "Fv2moeKs8", "vocab": 512, "B": 2, "T": 128, "env": env, "freeze": freeze})
    m = build("Fv2moeKs8", 512, env=env)
    m.load_state_dict(d["sd"])
    for b in m.heavy:
        b.learned.zero_()
        b.learned[freeze] = True
    assert len(m.rebank(1000)) == 2 * len(m.heavy)               # (up, down) of every layer changed hands
    assert m.heavy[0].Fz == freeze and m.heavy[0].up.shape[0] == 5
    if bank_q:
        assert m.heavy[0].up_f.dtype == torch.int8
    m.train()
    xy = d["xy"]
    out, cost = m(xy[:, :-1])
    loss = m.train_loss(out, xy[:, 1:], True)
    assert abs(loss.item() - d["loss"].item()) < 2e-5 * max(1, abs(d["loss"].item())), (loss.item(), d["loss"].item())
    (loss + 0.01 * cost.float()).backward()
    checked = 0
    for n, p in m.named_parameters():
        g = d["grads"].get(n)
        assert (g is None) == (p.grad is None), n
        if g is not None and g.float().abs().max() > 1e-7:
            assert g.shape == p.grad.shape, n
            # the bank's bf16 weights (and bf16 scale arithmetic of the quantised forms) leave differences of bf16 size
            assert (p.grad.float() - g.float()).abs().max() <= 5e-3 * g.float().abs().max(), n
            checked += 1
    assert checked > 20


@pytest.mark.parametrize("kw", [{"m_dtype": "fp32"}, {"m_dtype": "fp32", "norm": "row", "cards": 3}])
def test_experience_optimizer_matches_reference(tmp_path, kw):
    """The first card optimizer (a momentum per card and weight, surprise-scaled steps) over 8 steps of alternating
    situations and rising / falling losses: same weights as the reference after every step, word table included."""
    from memarch_b200.optim.experience import ExperienceOpt
    shapes = [(24, 16), (10000, 4), (3, 8, 6), (16,)]
    d = oracle(tmp_path, {"what": "experience", "shapes": shapes, "lr": 1e-2, "kw": kw, "steps": 8, "d": 12})
    ps = [torch.nn.Parameter(w.clone()) for w in d["w0"]]
    opt = ExperienceOpt(ps, lr=1e-2, **kw)
    for step, (gs, sit, loss) in enumerate(d["feed"]):
        for p, g in zip(ps, gs):
            p.grad = g.clone()
        opt.step(torch.tensor(loss), sit)
        for p, w in zip(ps, d["ws"][step]):
            assert (p.detach() - w).abs().max().item() <= 1e-5 * max(w.abs().max().item(), 1e-3), (step, tuple(p.shape))
    assert opt.used == d["used"].tolist() and sum(opt.used) >= 2          # both kinds of batches got their own card
