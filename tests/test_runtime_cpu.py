"""Runtime pieces on CPU: shard corpus with exact resume, host loader, checkpoint round trip and kill test, guards,
train/speed loops, CLI."""
import io
import json
import os
import math
import signal
import subprocess
import sys
import time

import numpy as np
import pytest
import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def make_corpus(root, n_shards=3, docs=40, seed=0, eos=999):
    from memarch_b200.data.loader import write_shard
    rng = np.random.default_rng(seed)
    for src, lo in (("web", 0), ("code", 400)):
        for s in range(n_shards):
            dd = [rng.integers(lo, lo + 300, size=rng.integers(5, 200)) for _ in range(docs)]
            write_shard(root, src, f"s{s}", dd, eos,
                        drop=[1, 3] if s == 0 else None,
                        score=rng.uniform(1.5, 4.0, size=docs) if src == "code" else None)
    return {"web": 0.7, "code": 0.3}


def test_corpus_mix_and_exact_resume(tmp_path):
    from memarch_b200.data.loader import ShardCorpus
    w = make_corpus(str(tmp_path))
    c = ShardCorpus(w, str(tmp_path), seq=64, seed=3)
    for _ in range(7):
        c.batch(4)
    st = json.loads(json.dumps(c.state_dict()))              # must survive serialisation
    want = [c.batch(4) for _ in range(90)]                   # crosses shard and epoch boundaries
    assert abs(c.mix()["web"] - 0.7) < 0.02
    c2 = ShardCorpus(w, str(tmp_path), seq=64, seed=3)
    c2.load_state_dict(st)
    for a in want:
        assert np.array_equal(a, c2.batch(4))
    assert c.sources[0].epoch > 0                            # the test did wrap around


def test_corpus_masks_and_ranks(tmp_path):
    from memarch_b200.data.loader import ShardCorpus, shard_documents
    make_corpus(str(tmp_path))
    docs = shard_documents(os.path.join(str(tmp_path), "web", "s0"), 999, np.random.default_rng(0))
    assert len(docs) == 38                                   # two dropped by the dedup mask
    assert all(d[-1] == 999 for d in docs)
    a = ShardCorpus({"web": 1.0}, str(tmp_path), seq=32, rank=0, world=2)
    b = ShardCorpus({"web": 1.0}, str(tmp_path), seq=32, rank=1, world=2)
    assert set(a.sources[0].names).isdisjoint(b.sources[0].names)
    with pytest.raises(ValueError):
        ShardCorpus({"web": 1.0}, str(tmp_path), seq=32, rank=5, world=6)


def test_host_loader_state_is_the_consumed_batch(tmp_path):
    from memarch_b200.data.loader import HostLoader, ShardCorpus
    w = make_corpus(str(tmp_path))
    ld = HostLoader(ShardCorpus(w, str(tmp_path), seq=64, seed=1), B=2, depth=3)
    for _ in range(5):
        ld.next()
    time.sleep(0.2)                                          # let the worker read ahead
    st = ld.state_dict()
    nxt = ld.next()
    ld.close()
    c = ShardCorpus(w, str(tmp_path), seq=64, seed=1)
    c.load_state_dict(st)
    assert np.array_equal(c.batch(2), nxt.numpy())


def test_host_loader_forwards_worker_errors(tmp_path):
    from memarch_b200.data.loader import HostLoader

    class Broken:
        seq = 8

        def state_dict(self):
            return {}

        def batch(self, B):
            raise ValueError("shard unreadable")
    ld = HostLoader(Broken(), B=2)
    with pytest.raises(RuntimeError):
        ld.next()
    ld.close()


def tiny_trainer(seed=0, stage="ABX", **env):
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.train import Trainer
    torch.manual_seed(seed)
    e = {"NO_MEM": "1", "MOE_ACT": "relu2"}
    e.update(env)
    m = build("tiny", 256, env=e)
    return Trainer(m, TrainConfig(name="tiny", stage=stage, steps=50, batch=4, micro=4, seq=32, lr=1e-2, warmup=2),
                   OptConfig(lr=1e-2, norm="hs", scale=0.12, rel_every=2), stage=stage)


def batches(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 256, (4, 33), generator=g) for _ in range(n)]


def test_checkpoint_round_trip_continues_bit_exact(tmp_path):
    from memarch_b200.train.ckpt import Checkpointer
    xs = batches(8)
    a = tiny_trainer()
    for s in range(4):
        a.step(xs[s], s)
    ck = Checkpointer(str(tmp_path), rid="r1")
    ck.save(a, 4, log=[{"step": 4}], corpus_state={"k": 1})
    ck.wait()
    want = [float(a.step(xs[s], s)) for s in range(4, 8)]
    b = tiny_trainer(seed=7)                                 # different init: everything must come from the file
    nxt, log = Checkpointer(str(tmp_path), rid="r1").load(b)
    assert nxt == 5 and log == [{"step": 4}]
    got = [float(b.step(xs[s], s)) for s in range(4, 8)]
    assert got == want
    with pytest.raises(RuntimeError):
        Checkpointer(str(tmp_path), rid="other").load(tiny_trainer())
    st = torch.load(os.path.join(str(tmp_path), "latest.pt"), weights_only=False)
    assert set(st) >= {"step", "log", "banks", "model", "opt", "corpus"}
    assert {"m", "w", "gain", "keys", "used", "expect", "seen", "rel", "n_step", "_lr"} <= set(st["opt"])


def test_lagged_homeostasis_state_round_trips_through_a_checkpoint(tmp_path):
    """`hs_lag`: the previous step's second-axis mean squares (`cs`) are optimizer state; a resumed run continues
    bit-exact, and the blob keeps one learning rate per parameter group (a list, the reference's layout)."""
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.train import Trainer
    from memarch_b200.train.ckpt import Checkpointer

    def mk(seed):
        torch.manual_seed(seed)
        m = build("tiny", 256, env={"NO_MEM": "1", "MOE_ACT": "relu2"})
        return Trainer(m, TrainConfig(name="tiny", stage="ABX", steps=50, batch=4, micro=4, seq=32, lr=1e-2, warmup=2),
                       OptConfig(lr=1e-2, norm="hs", scale=0.12, rel_every=2, hs_lag=True), stage="ABX")
    xs = batches(7, seed=3)
    a = mk(0)
    for s in range(3):
        a.step(xs[s], s)
    assert any(c is not None and bool((c > 0).any()) for c in a.opt.cs)
    ck = Checkpointer(str(tmp_path), rid="lag")
    ck.save(a, 3)
    ck.wait()
    want = [float(a.step(xs[s], s)) for s in range(3, 7)]
    b = mk(5)
    Checkpointer(str(tmp_path), rid="lag").load(b)
    assert [float(b.step(xs[s], s)) for s in range(3, 7)] == want
    st = torch.load(os.path.join(str(tmp_path), "latest.pt"), weights_only=False)
    assert isinstance(st["opt"]["_lr"], list) and len(st["opt"]["_lr"]) == len(a.opt.param_groups)
    # a blob with a scalar rate (older files) still loads
    st["opt"]["_lr"] = float(st["opt"]["_lr"][0])
    b.opt.load_state_dict(st["opt"])
    assert b.opt.param_groups[0]["lr"] == st["opt"]["_lr"]


KILL_SCRIPT = r"""
import os, sys, time, torch
sys.path.insert(0, {root!r})
from memarch_b200.train.ckpt import Checkpointer
class M(torch.nn.Module):
    def __init__(self):
        super().__init__(); self.w = torch.nn.Parameter(torch.zeros(2_000_000))
class T:
    device = torch.device("cpu")
    def __init__(self): self.model = M(); self.opt = torch.optim.SGD(self.model.parameters(), lr=0.1)
t = T(); ck = Checkpointer({d!r}, background=True)
step = 0
while True:
    step += 1
    with torch.no_grad(): t.model.w.fill_(float(step))
    ck.save(t, step)
    print(step, flush=True)
"""


def test_kill_during_checkpoint_leaves_a_complete_file(tmp_path):
    """SIGKILL the writer at arbitrary moments: latest.pt is always loadable and internally consistent."""
    d = str(tmp_path)
    for trial in range(3):
        p = subprocess.Popen([sys.executable, "-c", KILL_SCRIPT.format(root=ROOT, d=d)], stdout=subprocess.PIPE, text=True)
        seen = 0
        t0 = time.time()
        while seen < 3 + trial and time.time() - t0 < 120:
            line = p.stdout.readline()
            if line.strip():
                seen = int(line)
        time.sleep(0.013 * (trial + 1))
        p.send_signal(signal.SIGKILL)
        p.wait()
        st = torch.load(os.path.join(d, "latest.pt"), weights_only=False)
        w = st["model"]["w"]
        assert st["step"] >= 1 and bool((w == float(st["step"])).all())


def test_nan_guard_and_spike_log():
    from memarch_b200.train.guards import NanGuard, NonFiniteLoss, SpikeLog
    g = NanGuard(every=4)
    for v in (1.0, 2.0, float("nan")):
        g.check(torch.tensor(v))
    with pytest.raises(NonFiniteLoss):
        g.check(torch.tensor(1.0))
    buf = io.StringIO()
    s = SpikeLog(spike=2.0, out=buf)
    for i, v in enumerate((3.0, 3.1, 2.9, 9.0, 3.0)):
        s.check(i, v)
    assert len(s.events) == 1 and s.events[0][0] == 3 and "spike" in buf.getvalue()


def test_rollback_guard_reverts_and_replays():
    from memarch_b200.train.guards import RollbackGuard
    xs = batches(6)
    tr = tiny_trainer()
    rb = RollbackGuard(tr, ratio=1.5, warm=2, lr_mul=0.5)
    for s in range(3):
        rb.step(xs[s], s)
    before_prev = [t.clone() for t in rb.snap_p]             # state before step 2 (the previous step)
    real = tr.step

    def spiky(xy, step, **kw):                               # host-made failure: this step reports a huge loss
        return real(xy, step, **kw) * 100.0
    tr.step = spiky
    rb.step(xs[3], 3)
    tr.step = real
    assert bool(rb.rep) and int(rb.n_hit) == 1
    for p, s in zip(tr.params, before_prev):
        assert torch.equal(p.data, s)                        # weights are back to the snapshot
    seen = {}

    def spy(xy, step, **kw):
        seen["xy"] = xy.clone()
        seen["mul"] = float(tr.opt.lr_mul_dev)
        return real(xy, step, **kw)
    tr.step = spy
    rb.step(xs[4], 4)
    assert torch.equal(seen["xy"], xs[2]) and seen["mul"] == 0.5   # replays the previous batch at half step
    assert not bool(rb.rep)
    rb.step(xs[5], 5)
    assert torch.equal(seen["xy"], xs[5]) and seen["mul"] == 1.0


def test_watchdog_dumps_stacks_without_killing():
    from memarch_b200.train.guards import Watchdog
    buf = io.StringIO()
    w = Watchdog(timeout=0.3, repeat=0.3, out=buf)
    for _ in range(5):
        w.beat()
        time.sleep(0.05)
    assert w.fired == 0
    time.sleep(1.2)
    w.close()
    assert w.fired >= 2 and "no progress" in buf.getvalue() and "thread" in buf.getvalue().lower()


class Args:
    def __init__(self, **kw):
        self.models, self.stages, self.stage = ["tiny"], ["ABX"], "ABX"
        self.steps, self.batch, self.micro, self.seq, self.lr = 12, 4, 4, 32, 1e-2
        self.read_cost, self.eval_every, self.tokens, self.warmup, self.n = 0.01, 6, 60_000, 1, 2
        self.__dict__.update(kw)


def test_train_loop_resumes_from_checkpoint(tmp_path, monkeypatch):
    from memarch_b200.train.loop import train
    monkeypatch.chdir(tmp_path)
    env = {"VOCAB": "256", "NO_MEM": "1", "CKPT_DIR": str(tmp_path / "ck"), "CKPT_EVERY": "6", "WATCHDOG": "0",
           "OPT_KW": json.dumps({"norm": "hs", "scale": 0.12}), "EMA_START": "0.5"}
    full = train(Args(), "cpu", env=env, out=io.StringIO())["tiny"]
    assert [e["step"] for e in full] == [6, 12] and full[-1]["val"] < 6.0
    assert os.path.exists(tmp_path / "results" / "tiny_ABX.json")
    # second run with the same directory: nothing left to do, log comes back from the file
    buf = io.StringIO()
    again = train(Args(), "cpu", env=env, out=buf)["tiny"]
    assert [e["step"] for e in again] == [6, 12]


def test_speed_and_cli(tmp_path, monkeypatch, capsys):
    from memarch_b200.cli import main
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("VOCAB", "256")
    monkeypatch.setenv("NO_MEM", "1")
    assert main(["speed", "--models", "tiny", "--batch", "2", "--seq", "32", "--n", "2", "--warmup", "1", "--device", "cpu"]) == 0
    out = capsys.readouterr().out
    assert "SPEED tiny ABX" in out and "ms/step" in out
    r = json.load(open(tmp_path / "results" / "speed.json"))
    assert r[0]["flops_per_step"] > 0


def test_injected_nan_stops_the_run_without_saving(tmp_path, monkeypatch):
    from memarch_b200.train.guards import NonFiniteLoss
    from memarch_b200.train.loop import train
    monkeypatch.chdir(tmp_path)
    env = {"VOCAB": "256", "NO_MEM": "1", "CKPT_DIR": str(tmp_path / "ck"), "CKPT_EVERY": "4", "WATCHDOG": "0",
           "TRAIN_NAN_AT": "6", "NAN_EVERY": "1"}
    with pytest.raises(NonFiniteLoss):
        train(Args(steps=12, eval_every=100), "cpu", env=env, out=io.StringIO())
    st = torch.load(tmp_path / "ck" / "latest.pt", weights_only=False)
    assert st["step"] == 4                                   # the last save is from before the failure


def test_learns_on_a_repeated_batch():
    """Smoke: the loss of a repeated batch drops by at least 0.05 and decreases on most steps."""
    tr = tiny_trainer()
    xy = batches(1)[0]
    losses = [float(tr.step(xy, s)) for s in range(9)]
    assert losses[0] - losses[-1] > 0.05
    assert sum(b < a for a, b in zip(losses, losses[1:])) >= 6, losses


@pytest.mark.parametrize("stage", ["A", "AS", "AX", "ABX"])
def test_trainer_stages_step_and_learn(stage):
    """Every optimizer arrangement of the trainer takes steps and lowers the loss of a repeated batch."""
    tr = tiny_trainer(stage=stage)
    xy = batches(1)[0]
    losses = [float(tr.step(xy, s)) for s in range(6)]
    assert all(l == l for l in losses) and losses[-1] < losses[0], (stage, losses)


def test_micro_batches_accumulate_to_the_full_batch_gradient():
    """Stage B steps the weights only on the last micro-batch, from the accumulated gradient: two micro-batches of 2
    move the weights the same way as one batch of 4 (not bit-equal: the anchor threshold and the expert capacity are
    per forward call)."""
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.train import Trainer
    xy = batches(1)[0]
    deltas = []
    for micro in (4, 2):
        torch.manual_seed(0)
        m = build("tiny", 256, env={"NO_MEM": "1", "MOE_ACT": "relu2"})
        w0 = m.light_a[0].qkv.weight.detach().clone()
        tr = Trainer(m, TrainConfig(name="tiny", stage="ABX", steps=50, batch=4, micro=micro, seq=32, lr=1e-2, warmup=2),
                     OptConfig(lr=1e-2, norm="hs", scale=0.12, rel_every=2), stage="ABX")
        tr.step(xy, 0)
        deltas.append((m.light_a[0].qkv.weight.detach() - w0).flatten())
    assert deltas[0].abs().sum() > 0 and deltas[1].abs().sum() > 0
    cos = torch.nn.functional.cosine_similarity(deltas[0], deltas[1], dim=0).item()
    assert cos > 0.9, cos


def test_two_run_resume_check_prints_pass_and_detects_a_difference(tmp_path, monkeypatch):
    """Run A stops early and leaves a checkpoint in the middle plus its per-step losses; run B resumes, repeats the
    steps after the checkpoint and compares them with A's log."""
    from memarch_b200.train.loop import train
    monkeypatch.chdir(tmp_path)
    base = {"VOCAB": "256", "NO_MEM": "1", "CKPT_DIR": str(tmp_path / "ck"), "CKPT_EVERY": "4", "WATCHDOG": "0",
            "OPT_KW": json.dumps({"norm": "hs", "scale": 0.12}), "STOP_AT": "7", "NO_FINAL_CKPT": "1"}
    a_log = str(tmp_path / "A.jsonl")
    train(Args(steps=12), "cpu", env=dict(base, LOSS_LOG=a_log), out=io.StringIO())
    rows = [json.loads(l) for l in open(a_log)]
    assert [r["step"] for r in rows] == list(range(1, 8))
    buf = io.StringIO()
    train(Args(steps=12), "cpu", env=dict(base, COMPARE=a_log, CMP_TOL="1e-5"), out=buf)
    assert "resuming at step 5" in buf.getvalue()
    assert "RESUME_TEST PASS: steps 5..7, 3 compared" in buf.getvalue()
    # a log that does not belong to this run fails the check
    bad = str(tmp_path / "bad.jsonl")
    with open(bad, "w") as f:
        for r in rows:
            f.write(json.dumps({"step": r["step"], "loss": r["loss"] + 0.5}) + "\n")
    buf = io.StringIO()
    train(Args(steps=12), "cpu", env=dict(base, COMPARE=bad, CMP_TOL="1e-5"), out=buf)
    assert "RESUME_TEST FAIL" in buf.getvalue()


def test_mirrored_checkpoints_survive_the_loss_of_the_local_directory(tmp_path, monkeypatch):
    import shutil
    from memarch_b200.train.ckpt import FileStore
    from memarch_b200.train.loop import train
    monkeypatch.chdir(tmp_path)
    env = {"VOCAB": "256", "NO_MEM": "1", "CKPT_DIR": str(tmp_path / "ck"), "CKPT_EVERY": "3", "WATCHDOG": "0",
           "CKPT_MIRROR": str(tmp_path / "mirror"), "OPT_KW": json.dumps({"norm": "hs", "scale": 0.12}),
           "STOP_AT": "9", "NO_FINAL_CKPT": "1"}
    train(Args(steps=12, eval_every=100), "cpu", env=env, out=io.StringIO())
    files = sorted(os.listdir(tmp_path / "mirror"))
    assert files == ["step_00000006.json", "step_00000006.pt", "step_00000009.json", "step_00000009.pt"]   # keeps two
    tag = json.load(open(tmp_path / "mirror" / "step_00000009.json"))
    assert tag["step"] == 9 and tag["run_id"] and tag["bytes"] == os.path.getsize(tmp_path / "mirror" / "step_00000009.pt")
    # a foreign run's newer copy and a half-written copy sit in the same store
    shutil.copyfile(tmp_path / "mirror" / "step_00000009.pt", tmp_path / "mirror" / "step_00000050.pt")
    json.dump({"step": 50, "run_id": "someone-else"}, open(tmp_path / "mirror" / "step_00000050.json", "w"))
    shutil.copyfile(tmp_path / "mirror" / "step_00000009.pt", tmp_path / "mirror" / "step_00000060.pt.tmp")
    st = FileStore(str(tmp_path / "mirror"), tag["run_id"])
    assert st.steps() == [6, 9] and st.steps(mine=False) == [6, 9, 50]
    shutil.rmtree(tmp_path / "ck")                                        # the local disk is gone
    buf = io.StringIO()
    train(Args(steps=12, eval_every=100), "cpu", env=dict(env, STOP_AT="12"), out=buf)
    assert "resuming at step 10" in buf.getvalue()
    assert os.path.exists(tmp_path / "mirror" / "step_00000050.pt")       # other runs' copies are never deleted
    assert FileStore(str(tmp_path / "mirror"), tag["run_id"]).steps() == [9, 12]


def test_named_eval_sets_and_eval_only(tmp_path, monkeypatch):
    from memarch_b200.train.loop import train
    monkeypatch.chdir(tmp_path)
    rng = np.random.default_rng(0)
    np.save(tmp_path / "a.npy", rng.integers(0, 256, 6000).astype(np.int32))
    np.save(tmp_path / "b.npy", np.tile(np.arange(8, dtype=np.int32), 800))           # trivially predictable text
    env = {"VOCAB": "256", "NO_MEM": "1", "CKPT_DIR": str(tmp_path / "ck"), "CKPT_EVERY": "6", "WATCHDOG": "0",
           "OPT_KW": json.dumps({"norm": "hs", "scale": 0.12}), "EVAL_BATCHES": "2", "DIAG": "1",
           "EVAL_SETS": json.dumps({"noise": str(tmp_path / "a.npy"), "cycle": str(tmp_path / "b.npy")})}
    buf = io.StringIO()
    log = train(Args(steps=6), "cpu", env=env, out=buf)["tiny"]
    assert set(log[-1]["sets"]) == {"noise", "cycle"} and "noise" in buf.getvalue() and "cycle" in buf.getvalue()
    assert "[diag] per step: data wait" in buf.getvalue()                             # host-side phase times
    buf = io.StringIO()
    again = train(Args(steps=6), "cpu", env=dict(env, EVAL_ONLY="1"), out=buf)["tiny"]
    assert again[-1]["eval_only"] and again[-1]["step"] == 6
    assert abs(again[-1]["noise"] - log[-1]["sets"]["noise"]) < 1e-5 and abs(again[-1]["cycle"] - log[-1]["sets"]["cycle"]) < 1e-5
    assert "eval at step 6" in buf.getvalue()


def test_needles_in_the_training_text_follow_the_loader_and_resume(tmp_path, monkeypatch):
    from memarch_b200.train.loop import make_data, train
    monkeypatch.chdir(tmp_path)
    w = make_corpus(str(tmp_path / "corpus"), docs=60)
    env = {"VOCAB": "2048", "NO_MEM": "1", "WATCHDOG": "0", "CORPUS": json.dumps(w), "CORPUS_ROOT": str(tmp_path / "corpus"),
           "REMIND_P": "1.0", "REMIND_N": "2", "REMIND_DIST": "4", "REMIND_TOK0": "1000", "REMIND_LADDER": "6,12",
           "REMIND_WIN": "4", "REMIND_THR": "0.0", "REMIND_LAG": "3",
           "OPT_KW": json.dumps({"norm": "hs", "scale": 0.12})}
    a = Args(seq=48, batch=4, micro=4, steps=6, eval_every=2)
    data = make_data(a, "cpu", env)
    seen = [data.batch(4, 48).clone() for _ in range(3)]
    mark = data.remind.mark
    assert all(int((b == mark).sum()) == 4 * 4 for b in seen)                  # two blocks of two markers per row
    assert data.extra["rem"].shape == (4, 48) and data.extra["rem"].sum() == 8
    st = json.loads(json.dumps(data.state_dict()))
    assert st["loader_n"] == 3 and "remind" in st
    nxt = data.batch(4, 48).clone()
    data.loader.close()
    data2 = make_data(a, "cpu", env)
    data2.load_state_dict(st)
    assert torch.equal(data2.batch(4, 48), nxt)                                # same text, same needles after resume
    data2.loader.close()
    buf = io.StringIO()
    log = train(a, "cpu", env=env, out=buf)["tiny"]
    assert "needles" in log[-1]["sets"] and 0.0 <= log[-1]["sets"]["needles"] <= 1.0
    assert "reminders: level 0 -> 1" in buf.getvalue()                          # threshold 0: the ladder moves on
    # recall at fixed distances on held-out text, at every evaluation
    log = train(Args(seq=48, batch=4, micro=4, steps=2, eval_every=2), "cpu", env=dict(env, REMIND_EVAL="4,20,400"),
                out=io.StringIO())["tiny"]
    assert {"recall_d4", "recall_d20"} <= set(log[-1]["sets"]) and "recall_d400" not in log[-1]["sets"]
    assert all(0.0 <= log[-1]["sets"][k] <= 1.0 for k in ("recall_d4", "recall_d20"))


def test_recipe_plan_and_step_count(tmp_path, capsys):
    from memarch_b200.cli import main, recipe_steps
    assert recipe_steps(448.0, 1500.0) == 3300 and recipe_steps(5000.0, 1500.0) == 500 and recipe_steps(153.6, 1500) == 9750
    assert main(["recipe", "--dry", "--out", str(tmp_path / "art")]) == 0
    out = capsys.readouterr().out
    assert "T Td2048L16" in out and "ours Fv2moeK8h8d2048" in out
    ours = out.split("ours Fv2moeK8h8d2048")[1]
    assert '"INDUCT": "lock"' in ours and '"NO_MEM": "1"' in ours and '"MOE_ACT": "relu2"' in ours
    dense = out.split("ours Fv2moeK8h8d2048")[0]
    assert "INDUCT" not in dense and '"OPT_KW"' in dense


def test_recipe_runs_both_models_end_to_end(tmp_path, monkeypatch, capsys):
    from memarch_b200 import cli
    monkeypatch.chdir(tmp_path)
    for k, v in {"D_MODEL": "256", "VOCAB": "512", "WATCHDOG": "0"}.items():
        monkeypatch.setenv(k, v)
    monkeypatch.setattr(cli, "RECIPE_MODELS", (("T", "tiny", False), ("ours", "tiny", True)))
    monkeypatch.setattr(cli, "recipe_steps", lambda ms, budget: 4)
    args = cli.parser().parse_args(["recipe", "--out", "art", "--tokens", "120000", "--batch", "2", "--seq", "64",
                                    "--device", "cpu"])
    args.micro = 2
    before = dict(os.environ)
    plan = cli.recipe(args)
    assert [(p["tag"], p["steps"], len(p["log"])) for p in plan] == [("T", 4, 1), ("ours", 4, 1)]
    assert dict(os.environ) == before                                  # the switches of a model do not leak
    out = capsys.readouterr().out
    assert "[recipe] T tiny" in out and "[recipe] ours tiny" in out
    assert "trust" in out.split("[recipe] T tiny")[1] and "trust" not in out.split("[recipe] T tiny")[0]   # locks: ours only
    assert os.path.exists(tmp_path / "art" / "env.json")


def test_muon_combo_follows_torch_muon():
    """Muon on hidden matrices + AdamW on the rest (the reference's OPT=muon race optimizer, fastloop.py:63-82):
    three steps against torch.optim.Muon(adjust_lr_fn="match_rms_adamw") + AdamW on the same gradients."""
    import torch
    from memarch_b200.optim.muon import MuonAdamW, orthogonalise
    torch.manual_seed(0)
    shapes = [(48, 32), (32, 64), (20000, 8), (16,)]
    mk = lambda: [torch.nn.Parameter(torch.randn(*s) * 0.1) for s in shapes]
    torch.manual_seed(1); a = mk()
    torch.manual_seed(1); b = mk()
    ours = MuonAdamW(a, lr=0.02, weight_decay=0.1, betas=(0.9, 0.95), mul=1.5)
    assert [tuple(p.shape) for p in ours.mats] == [(48, 32), (32, 64)]             # the word table and the vector go to AdamW
    ref_m = torch.optim.Muon(b[:2], lr=0.02 * 1.5, weight_decay=0.1, adjust_lr_fn="match_rms_adamw")
    ref_a = torch.optim.AdamW(b[2:], lr=0.02, betas=(0.9, 0.95), weight_decay=0.1)
    for step in range(3):
        g = torch.Generator().manual_seed(10 + step)
        for p, r in zip(a, b):
            p.grad = torch.randn(p.shape, generator=g)
            r.grad = p.grad.clone()
        ours.step(); ref_m.step(); ref_a.step()
    for p, r in zip(a, b):
        assert (p - r).abs().max() < 5e-3 * max(1.0, float(r.abs().max())), float((p - r).abs().max())   # torch iterates in bf16
    o = orthogonalise(torch.randn(24, 40))
    sv = torch.linalg.svdvals(o)
    assert sv.min() > 0.5 and sv.max() < 1.3                                       # singular values pushed towards 1
    sd = ours.state_dict()
    ours.load_state_dict(sd)


def test_err_step_and_gearbox_pace_the_step():
    """Step-length rules on |g| against its usual value: err_step divides by the sensitivity; the gearbox shifts one
    gear at a time and its speed moves by at most gb_acc per step (JAX Instinct, instinct.py:150-172, 753-772)."""
    import torch
    from memarch_b200.config import OptConfig
    from memarch_b200.optim.instinct import Instinct
    torch.manual_seed(0)
    sit = torch.randn(16)

    def run(cfg, scales):
        p = torch.nn.Parameter(torch.randn(32, 24) * 0.1)
        opt = Instinct([p], cfg)
        g0 = torch.randn(32, 24)
        facs = []
        for sc in scales:
            opt.prepare(torch.tensor(3.0), sit)
            p.grad = g0 * sc
            opt.update(p)
            p.grad = None
            opt.finish()
            facs.append(float(opt.df[0]))
        return facs, opt

    calm = [1.0] * 12
    f, _ = run(OptConfig(lr=1e-3, damp=3.0, err_step=True), calm + [4.0, 1.0])
    assert all(abs(x - 1.0) < 1e-5 for x in f[1:12])            # usual |g|: the step is what it was
    assert abs(f[12] - 0.25) < 1e-3                               # 4x the sensitivity: a quarter of the step
    assert abs(f[13] - 1.0) < 0.2                                 # the surge entered the usual norm capped: back to ~1
    f, _ = run(OptConfig(lr=1e-3, damp=3.0, err_step=True, err_cap=2.0), calm + [0.1])
    assert abs(f[12] - 2.0) < 1e-5                                # capped

    f, opt = run(OptConfig(lr=1e-3, damp=3.0, gearbox=True), calm + [3.0, 3.0, 3.0, 1.0])
    assert 1.0 <= f[0] <= 1.05 + 1e-6
    top = max(f[:12])
    assert 1.0 < top <= 1.25 + 1e-6                               # calm driving shifts up towards the top gear
    steps = [abs(b - a) for a, b in zip(f, f[1:])]
    assert max(steps) <= 0.05 + 1e-6                              # the speed never jumps
    assert f[14] < f[11] and int(opt.gear[0]) < 3                 # three surges: geared down, slowing
    sd = opt.state_dict()
    assert "gear" in sd and "speed" in sd


def test_training_loop_raises_when_a_device_wait_has_run_out(monkeypatch):
    """The loop reads the kernels' status words wherever it synchronises with the host anyway; a non-zero word (a
    bounded device wait gave up) must stop the run with an exception, not pass as silently wrong weights.  The device
    is faked: a status reader that returns a code, and an engine whose check raises as `SymmetricHeap.check` does."""
    import types
    import torch
    from memarch_b200.ops import _ext
    from memarch_b200.train import loop

    class FakeC:
        def __init__(self, st):
            self.st = st

        def gemm_status(self, dev):
            return self.st

    class Engine:
        def check(self):
            raise RuntimeError("peer wait timed out (status 5): a rank did not reach the barrier within 4000.0 ms")

    tr = types.SimpleNamespace(device=torch.device("cuda", 0), parallel=None)
    monkeypatch.setattr(_ext, "available", lambda: True)
    monkeypatch.setattr(_ext, "C", lambda: FakeC(0))
    loop.device_status(tr)                                        # clean words: nothing happens
    monkeypatch.setattr(_ext, "C", lambda: FakeC(3))
    with pytest.raises(RuntimeError, match="bounded wait"):
        loop.device_status(tr)
    monkeypatch.setattr(_ext, "C", lambda: FakeC(0))
    tr.parallel = Engine()
    with pytest.raises(RuntimeError, match="peer wait timed out"):
        loop.device_status(tr)
    tr_cpu = types.SimpleNamespace(device=torch.device("cpu"), parallel=Engine())
    loop.device_status(tr_cpu)                                    # CPU runs have no status words


def test_named_weight_switches_of_the_optimizer():
    """gnorm (gradient scale does not matter), wd_norm (norm weights decay), norm_anchor (norm weights of the light
    blocks rest at 1), lr_mul (step multiplier by name prefix) - switches of the reference's JAX Instinct
    (instinct.py:65-131, 393-401)."""
    import torch
    from memarch_b200.config import OptConfig
    from memarch_b200.optim.instinct import Instinct
    sit = torch.ones(8)

    def run(cfg, names, gscale=1.0, steps=1, grad_fn=None):
        torch.manual_seed(0)
        ps = [torch.nn.Parameter(torch.randn(16, 12)), torch.nn.Parameter(torch.ones(12) * 1.5),
              torch.nn.Parameter(torch.ones(12) * 1.5)]
        opt = Instinct(ps, cfg, names=names)
        g = torch.Generator().manual_seed(1)
        for s in range(steps):
            opt.prepare(torch.tensor(3.0), sit)
            for p in ps:
                gr = torch.randn(p.shape, generator=g) * gscale if grad_fn is None else grad_fn(p)
                opt.update(p, gr)
            opt.finish()
        return [p.detach().clone() for p in ps]

    names = ["light_a.0.qkv.weight", "light_a.0.n1.weight", "norm.weight"]
    base = OptConfig(lr=1e-2, norm="hs", weight_decay=0.1)
    # gnorm: a thousand times larger gradients give the same momentum direction and the same first step anyway
    # (Instinct normalises the update), but the momentum itself is scale-free only with gnorm
    import dataclasses
    a = run(dataclasses.replace(base, gnorm=True), names, 1.0)
    b = run(dataclasses.replace(base, gnorm=True), names, 1000.0)
    assert all(torch.allclose(x, y, atol=1e-6) for x, y in zip(a, b))
    # lr_mul: the matrix under "light_a." moves half as far, the rest as before
    w0 = run(base, names, steps=0)
    full = run(base, names)
    half = run(dataclasses.replace(base, lr_mul=(("light_a.0.qkv", 0.5),)), names)
    # decay is part of the step: compare the distance from the start
    d_full, d_half = (full[0] - w0[0]).norm(), (half[0] - w0[0]).norm()
    assert abs(float(d_half / d_full) - 0.5) < 0.02 and torch.equal(full[2], half[2])
    # wd_norm: zero gradients, so only the decay acts - norm weights shrink, and only with the switch
    zero = lambda p: torch.zeros_like(p)
    still = run(base, names, steps=3, grad_fn=zero)
    decayed = run(dataclasses.replace(base, wd_norm=0.5), names, steps=3, grad_fn=zero)
    assert torch.equal(still[1], w0[1]) and float(decayed[1].mean()) < 1.5 and float(decayed[2].mean()) < 1.5
    assert torch.equal(still[0], decayed[0])
    # norm_anchor: the light block's norm weight is pulled from 1.5 towards 1, the final norm (no light_* prefix) is not
    anchored = run(dataclasses.replace(base, norm_anchor=True), names, steps=3, grad_fn=zero)
    assert 1.0 < float(anchored[1].mean()) < 1.5 and torch.equal(anchored[2], w0[2])


def test_trainer_with_the_experience_card_optimizer_learns():
    """Stage AX with `OptConfig(kind="experience")`: the host-synchronous card optimizer behind the trainer; a repeated
    batch is learned and the batch's situation picked a card."""
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.optim.experience import ExperienceOpt
    from memarch_b200.train import Trainer
    torch.manual_seed(0)
    m = build("tiny", 256, env={"NO_MEM": "1", "MOE_ACT": "relu2"})
    tr = Trainer(m, TrainConfig(name="tiny", stage="AX", steps=50, batch=4, micro=4, seq=32, lr=3e-3, warmup=2),
                 OptConfig(kind="experience", lr=3e-3, norm="row"), stage="AX")
    assert isinstance(tr.opt, ExperienceOpt)
    xy = batches(1)[0]
    losses = [float(tr.step(xy, s)) for s in range(8)]
    assert losses[-1] < losses[0] - 0.2, losses
    assert any(tr.opt.used) and tr.opt.last["card"] == 0


def _needle_model(**env):
    from memarch_b200 import build
    torch.manual_seed(0)
    e = {"NO_MEM": "1", "MOE_ACT": "relu2", "REMIND_W": "1.0", "REMIND_N": "4", "REMIND_TOK0": "1000"}
    e.update(env)
    return build("tiny", 2048, env=e).train()


def _needle_batch(blank=False, strict=False, B=6, T=64, n=4):
    from memarch_b200.data.reminders import Reminders
    r = Reminders(1.0, T=T, n=n, dist=8, seed=1, V=2048, tok0=1000, synth=10 ** 6, blank=blank,
                  pack=dict(strict=strict, round_to=T))
    xy, ex = r(np.zeros((B, T + 1), np.int32), n=0)
    return torch.from_numpy(xy).long(), {k: torch.from_numpy(v) for k, v in ex.items()}


def test_answer_loss_of_recall_needles():
    xy, ex = _needle_batch()
    x, y = xy[:, :-1], xy[:, 1:]
    rem = ex["rem"] > 0
    m = _needle_model()
    out, _ = m(x)
    plain = m.train_loss(out, y, True)
    with_term = m.train_loss(out, y, True, extra=ex)
    lo = m._logits(out[0]).float()
    nll = F.cross_entropy(lo.reshape(-1, lo.shape[-1]), y.reshape(-1), reduction="none").view_as(y)
    want = (nll * rem).sum() / (len(y) * 4)                                # sum over answers / (B * questions per row)
    assert abs(float(with_term - plain) - float(want)) < 1e-4
    assert abs(float(m.stats["remind_nll"]) - float(want)) < 1e-4 and abs(float(m.stats["remind_n"]) - 1.0) < 1e-6
    hits = ((nll < math.log(2.0)) & rem).sum() / (len(y) * 4)
    assert abs(float(m.stats["remind_hit"]) - float(hits)) < 1e-6
    # mean over the answers instead, the answers only (auxiliary terms stay), a softmax over the values only
    mean = _needle_model(REMIND_MEAN="1")
    mean.load_state_dict(m.state_dict())
    out2, _ = mean(x)
    d = mean.train_loss(out2, y, True, extra=ex) - mean.train_loss(out2, y, True)
    assert abs(float(d) - float((nll * rem).sum() / rem.sum())) < 1e-4 and "remind_hit_q2" in mean.stats
    only = _needle_model(REMIND_ONLY="1")
    only.load_state_dict(m.state_dict())
    out3, _ = only(x)
    main = float(nll.mean())
    assert abs(float(only.train_loss(out3, y, True, extra=ex)) - (float(with_term) - main)) < 1e-4
    cand = _needle_model(REMIND_CAND="1")
    cand.load_state_dict(m.state_dict())
    out4, _ = cand(x)
    d = cand.train_loss(out4, y, True, extra=ex) - cand.train_loss(out4, y, True)
    lv = lo[..., 1512:1576].log_softmax(-1).gather(-1, (y - 1512).clamp(0, 63)[..., None])[..., 0]
    assert abs(float(d) - float((-lv * rem).sum() / (len(y) * 4))) < 1e-4
    loss = cand.train_loss(out4, y, True, extra=ex)
    loss.backward()
    g = cand.head.weight.grad
    assert g is not None and torch.isfinite(g).all()
    # needle tokens do not teach the main loss
    mm = _needle_model(REMIND_MASK_MAIN="1", REMIND_W="0.0")
    mm.load_state_dict(m.state_dict())
    out5, _ = mm(x)
    keep = ~((y >= 1000) & (y <= 1576))
    base = _needle_model(REMIND_W="0.0")
    base.load_state_dict(m.state_dict())
    aux = float(base.train_loss(base(x)[0], y, True)) - main
    assert abs(float(mm.train_loss(out5, y, True, extra=ex)) - aux - float((nll * keep).sum() / y.numel())) < 1e-4
    assert 0 < float(mm.stats["remind_main_masked"]) < 1


def test_hidden_answers_and_the_strict_test():
    xy, ex = _needle_batch(blank=True, strict=True)
    x, y = xy[:, :-1], xy[:, 1:]
    rem = ex["rem"] > 0
    assert (y[rem] == 1000 + 576).all()                                    # the text shows the marker
    m = _needle_model(REMIND_STRICT="1", REMIND_STRICT_W="0.5")
    out, _ = m(x)
    total = m.train_loss(out, y, True, extra=ex)
    base = m.train_loss(out, torch.where(rem, ex["rem_y"].long(), y), True)  # main and auxiliaries on the true targets
    lo = m._logits(out[0]).float()
    lsm = lo.log_softmax(-1)
    yt = torch.where(rem, ex["rem_y"].long(), y)
    nll = -lsm.gather(-1, yt[..., None])[..., 0]
    hit = nll < math.log(2.0)
    term, pen, n_ans = 0.0, 0.0, 0
    for b in range(len(y)):
        ok = True
        vals = ex["rem_vals"][b]
        vals = vals[vals >= 0].long()
        for t in torch.nonzero(rem[b])[:, 0]:
            if ok:
                term += float(nll[b, t])
            ok = ok and bool(hit[b, t])
            others = vals[vals != yt[b, t]]
            pen += -math.log(max(1.0 - float(lsm[b, t, others].exp().sum()), 1e-6))
            n_ans += 1
    want = term / (len(y) * 4) + 0.5 * pen / n_ans
    assert abs(float(total - base) - want) < 1e-3
    assert 0 < float(m.stats["remind_strict_keep"]) <= 1 and float(m.stats["remind_strict_pother"]) > 0
    total.backward()
    assert torch.isfinite(m.head.weight.grad).all()


def test_episode_stage_trains_through_the_loop(tmp_path, monkeypatch):
    from memarch_b200.train.loop import train
    monkeypatch.chdir(tmp_path)
    w = make_corpus(str(tmp_path / "corpus"), docs=60)
    env = {"VOCAB": "2048", "NO_MEM": "1", "WATCHDOG": "0", "CORPUS": json.dumps(w), "CORPUS_ROOT": str(tmp_path / "corpus"),
           "REMIND_P": "1.0", "REMIND_N": "4", "REMIND_DIST": "4", "REMIND_TOK0": "1000", "REMIND_SYNTH": "4",
           "REMIND_PACK": "1", "REMIND_PACK_ROUND": "16", "REMIND_BLANK": "1", "REMIND_WIN": "4", "REMIND_THR": "0.0",
           "REMIND_LAG": "1", "REMIND_W": "1.0", "REMIND_MEAN": "1", "REMIND_ONLY": "1", "INDUCT": "lock",
           "OPT_KW": json.dumps({"norm": "hs", "scale": 0.12})}
    a = Args(seq=64, batch=4, micro=4, steps=6, eval_every=1)
    buf = io.StringIO()
    log = train(a, "cpu", env=env, out=buf)["tiny"]
    text = buf.getvalue()
    assert "episodes: step 0 -> 1" in text and "remind_hit" in text         # short rows, then text rows, one run
    assert all(math.isfinite(e["val"]) for e in log) and "needles" in log[-1]["sets"]
    # the curriculum may start further up its table, and the step on text batches ramps up after the stage
    import memarch_b200.train.loop as loop_mod
    seen = []
    real = loop_mod.Trainer.step

    def spy(self, xy, step, preps=None, lr_mul=1.0):
        seen.append((tuple(xy.shape), lr_mul))
        return real(self, xy, step, preps, lr_mul)
    monkeypatch.setattr(loop_mod.Trainer, "step", spy)
    train(Args(seq=64, batch=4, micro=4, steps=5, eval_every=5), "cpu",
          env=dict(env, REMIND_SYNTH="2", REMIND_PACK_LEVEL="3", REMIND_THR="2.0", TEXT_LR_RAMP="3"), out=io.StringIO())
    assert seen[0][0][1] == 49                                             # step 3 of the table: 4 pairs, fill 32 -> rows of 48 + 1
    assert [m for _, m in seen] == [1.0, 1.0, 1 / 3, 2 / 3, 1.0]


def test_instinct_blames_by_own_history_and_cards_by_kind():
    from memarch_b200 import OptConfig
    from memarch_b200.optim import Instinct
    torch.manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(8, 8)) for _ in range(10)]
    cfg = OptConfig(lr=1e-2, norm="hs", scale=0.12, rel_every=2, culprit="ema", top=0.2, g_max=1.5, card_by_kind=True,
                    cards=4, bad=0.5)
    opt = Instinct(ps, cfg)
    sit = torch.randn(16)
    opt.prepare(torch.tensor(1.0), sit, card=2)
    assert int(opt.k) == 2 and bool(opt.used[2]) and not bool(opt.used[0])
    opt.prepare(torch.tensor(1.0), sit, card=9)
    assert int(opt.k) == 3                                                  # clipped to the last card
    opt.prepare(torch.tensor(1.0), -sit)                                    # no number: by similarity (a new card)
    assert int(opt.k) == 0
    # blame: tensor 7 is far above its own mean although tensors 0, 1 are the largest in absolute terms
    opt.rel_avg.copy_(torch.tensor([5.0, 4.0] + [1.0] * 8))
    opt.rel.copy_(torch.tensor([5.0, 4.0, 1, 1, 1, 1, 1, 3.0, 1.2, 1]))
    opt.s = torch.tensor(-0.2)
    opt.g = torch.ones(10)
    opt.oh = F.one_hot(torch.tensor(1), 4).float()
    opt.n_step = 4
    opt.finish()
    row = opt.gain[1]
    assert row.argmax() == 7 and row[8] > row[0] and abs(float(row[0]) - float(row[1])) < 1e-6
    assert torch.allclose(opt.rel_avg[7], torch.tensor(0.9 * 1.0 + 0.1 * 3.0)) and opt.n_step == 5
    before = opt.rel_avg.clone()
    opt.finish()                                                            # step 5: |g|/|w| not measured, mean stays
    assert torch.equal(opt.rel_avg, before)
    opt.g = torch.full((10,), 1.4)
    opt.s = torch.tensor(-1.0)
    opt.finish()
    assert float((opt.gain[1] * 0 + 1).sum()) == 10 and "rel_avg" in opt.state_dict()
    plain = Instinct(ps, OptConfig(lr=1e-2, norm="hs", scale=0.12, top=0.2))
    plain.rel.copy_(opt.rel)
    plain.s, plain.g, plain.oh = torch.tensor(-0.2), torch.ones(10), opt.oh
    plain.finish()
    assert plain.gain[1].argmax() in (0, 1) and not hasattr(plain, "rel_avg")
    with pytest.raises(ValueError):
        Instinct(ps, OptConfig(culprit="mean"))


def test_idle_units_of_a_layer_pool_do_not_move():
    from memarch_b200 import OptConfig
    from memarch_b200.models.fishki import FishPool
    from memarch_b200.optim import Instinct
    torch.manual_seed(0)
    pool = FishPool(16, n=6, hf=32, kinds=3, pool=3)
    ps = [pool.up, pool.down, pool.norm]
    opt = Instinct(ps, OptConfig(lr=1e-2, norm="hs", scale=0.12, weight_decay=0.1, rel_every=1), names=["up", "down", "norm"])
    used = pool.sets[1]
    idle = [i for i in range(6) if i not in used]
    for step in range(3):
        before = [p.detach().clone() for p in ps]
        m_before = [m.clone() for m in opt.m]
        h = torch.randn(2, 5, 16)
        pool(h, used).square().sum().backward()
        opt.prepare(torch.tensor(1.0), torch.randn(8))
        for p in ps:
            opt.update(p)
            p.grad = None
        opt.finish()
        for p, b, m, mb in zip(ps, before, opt.m, m_before):
            assert torch.equal(p[idle], b[idle]) and torch.equal(m[idle], mb[idle])      # neither decay nor momentum
            assert not torch.equal(p[used], b[used])
    # without the mark the idle units would have decayed
    pool.up._idle_rows = False
    before = pool.up.detach().clone()
    pool(torch.randn(2, 5, 16), used).square().sum().backward()
    opt.prepare(torch.tensor(1.0), torch.randn(8))
    opt.update(pool.up)
    assert not torch.equal(pool.up[idle], before[idle])


def test_rules_on_the_common_vector_of_the_stream():
    from memarch_b200 import OptConfig
    from memarch_b200.optim import Instinct
    torch.manual_seed(0)
    d = 16
    names = ["light_b.0.o.weight", "light_b.0.down.weight", "light_b.0.qkv.weight", "light_b.0.up.weight", "heavy.0.o.weight"]
    shapes = [(d, d), (d, 4 * d), (3 * d, d), (8 * d, d), (d, d)]
    mk = lambda: [torch.nn.Parameter(torch.randn(*s) * 0.1) for s in shapes]
    ps = mk()
    opt = Instinct(ps, OptConfig(lr=1e-2, norm="hs", scale=0.12, stream_proj=True), names=names)
    # the port's "first axis of size d" in (in, out) layout: o and qkv along their inputs, down along its outputs
    assert opt._stream_ax == [1, 0, 1, None, None]
    sm = torch.randn(d)
    opt.observe_stream(sm)
    U = F.normalize(sm, dim=0)
    assert torch.allclose(opt.U, U, atol=1e-6)
    opt.observe_stream(-sm)                                                # a running mean, renormalised
    assert torch.allclose(opt.U, F.normalize(0.9 * U + 0.1 * (-U), dim=0), atol=1e-6)
    U = opt.U.clone()
    opt.prepare(torch.tensor(1.0), torch.randn(8))
    before = [p.detach().clone() for p in ps]
    for p in ps:
        p.grad = torch.randn_like(p)
        opt.update(p)
    along = lambda t, ax: (t.movedim(ax, -1) @ U).abs().max()
    assert along(opt.m[0], 1) < 1e-6 and along(opt.m[1], 0) < 1e-6 and along(opt.m[2], 1) < 1e-6   # nothing along U
    assert along(opt.m[3], 1) > 1e-3 and along(opt.m[4], 1) > 1e-3                                  # others untouched
    assert all(not torch.equal(p, b) for p, b in zip(ps, before))

    # rate limit: in the warm-up the weights are exactly those of the plain optimizer; afterwards a surge along U is cut
    # to kappa x the usual speed, the rest waits in the bank and comes out later
    torch.manual_seed(1)
    pa, pb = mk(), None
    torch.manual_seed(1)
    pb = mk()
    a = Instinct(pa, OptConfig(lr=1e-2, norm="hs", scale=0.12, m_rate=True, m_rate_warm=4, m_rate_kappa=1.5), names=names)
    b = Instinct(pb, OptConfig(lr=1e-2, norm="hs", scale=0.12), names=names)
    a.observe_stream(sm)
    g = torch.Generator().manual_seed(5)
    for step in range(4):
        for o_, ps_ in ((a, pa), (b, pb)):
            o_.prepare(torch.tensor(1.0), torch.ones(8))
        gs = [torch.randn(*s, generator=g) for s in shapes]
        for o_, ps_ in ((a, pa), (b, pb)):
            for p, gr in zip(ps_, gs):
                o_.update(p, gr.clone())
            o_.finish()
    assert all(torch.allclose(x, y, atol=1e-7) for x, y in zip(pa, pb)) and a.mrl_n == 4 and float(a.mrl_cut) == 0
    assert float(a.mrl_base[0]) > 0 and a.mrl_bank[3] is None
    u = a.U
    for step in range(3):                                                  # every weight is pushed along U, hard
        for o_ in (a, b):
            o_.prepare(torch.tensor(1.0), torch.ones(8))
        for o_, ps_ in ((a, pa), (b, pb)):
            w0 = ps_[1].detach().clone()
            o_.update(ps_[1], (torch.ones(4 * d)[None, :] * u[:, None]) * 50)
            o_.finish()
            if o_ is a:
                ca = (ps_[1] - w0).T @ u
            else:
                cb = (ps_[1] - w0).T @ u
    assert float(a.mrl_cut) > 0 and ca.norm() < cb.norm() and a.mrl_bank[1].norm() > 0
    moved_total = a.mrl_bank[1].norm()
    a.m[1].zero_()
    w0 = pa[1].detach().clone()
    for step in range(200):                                                # no more pressure along U: the bank drains
        a.prepare(torch.tensor(1.0), torch.ones(8))
        gr = torch.randn(d, 4 * d, generator=g)
        a.update(pa[1], gr - u[:, None] * (u @ gr)[None, :])
        a.finish()
    assert a.mrl_bank[1].norm() < 0.5 * moved_total
    released = (pa[1].detach() - w0).T @ u                                 # ... into the weights: nothing is thrown away
    assert released.norm() > 0.4 * moved_total
    sd = a.state_dict()
    assert "U" in sd and "mrl_bank" in sd and "mrl_base" in sd and sd["mrl_n"] == a.mrl_n


def test_trainer_feeds_the_stream_mean_to_the_optimizer():
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.train import Trainer
    torch.manual_seed(0)
    m = build("tiny", 256, env={"NO_MEM": "1", "MOE_ACT": "relu2"})
    tr = Trainer(m, TrainConfig(name="tiny", stage="ABX", steps=50, batch=4, micro=4, seq=32, lr=1e-2, warmup=2),
                 OptConfig(lr=1e-2, norm="hs", scale=0.12, rel_every=2, stream_proj=True, m_rate=True, m_rate_warm=2),
                 stage="ABX")
    assert m.want_stream_mean and any(ax is not None for ax in tr.opt._stream_ax)
    losses = [float(tr.step(xy, s)) for s, xy in enumerate(batches(6))]
    assert tr.opt.U is not None and abs(float(tr.opt.U.norm()) - 1) < 1e-5 and tr.opt.mrl_n == 6
    assert all(math.isfinite(v) for v in losses) and losses[-1] < losses[0] + 0.5


def test_safe_step_never_goes_against_the_fresh_gradient():
    from memarch_b200 import OptConfig
    from memarch_b200.optim import Instinct
    torch.manual_seed(0)
    names = ["light_a.0.up.weight", "norm.weight", "heavy.0.up.weight"]
    def mk():
        g = torch.Generator().manual_seed(3)
        return [torch.nn.Parameter(torch.randn(12, 8, generator=g) * 0.1),
                torch.nn.Parameter(torch.cat([torch.ones(7), torch.tensor([0.004])])),
                torch.nn.Parameter(torch.randn(12, 8, generator=g) * 0.1)]
    ps = mk()
    opt = Instinct(ps, OptConfig(lr=1e-2, norm="hs", scale=0.12, safe16=True, weight_decay=0.0), names=names)
    plain = Instinct(mk(), OptConfig(lr=1e-2, norm="hs", scale=0.12, weight_decay=0.0), names=names)
    assert opt._safe == [True, True, False]
    g0 = [torch.randn_like(p) for p in ps]
    for o_ in (opt, plain):
        o_.prepare(torch.tensor(1.0), torch.ones(8))
        for p, g in zip(o_.plist, g0):
            o_.update(p, g.clone())
        o_.finish()
    # first step: momentum and gradient agree everywhere, both optimizers take the same step on the matrix
    assert torch.allclose(opt.plist[0], plain.plist[0], atol=1e-7)
    # the sink channel (|w| = 0.004) of the norm weight moves in proportion to its size, not by a full step
    w_before = mk()[1]
    assert abs(float(opt.plist[1][7] - w_before[7])) < 0.05 * abs(float(plain.plist[1][7] - w_before[7]))
    # second step with a gradient that turned round: the plain step still coasts along the old momentum (up the
    # fresh gradient), the safe one moves up it nowhere
    g1 = -0.5 * g0[0]
    for o_ in (opt, plain):
        o_.prepare(torch.tensor(1.0), torch.ones(8))
        before = o_.plist[0].detach().clone()
        o_.update(o_.plist[0], g1.clone())
        o_.finish()
        step = o_.plist[0].detach() - before
        assert bool(((step * g1) > 1e-12).any()) == (o_ is plain)
    assert torch.allclose(opt.m[0], plain.m[0], atol=1e-7)                    # the stored momentum is the plain EMA
    assert torch.allclose(opt.plist[2], plain.plist[2])                       # other tensors: untouched by the rule


def test_raw_gradient_blame_and_brake_scopes():
    from memarch_b200 import OptConfig
    from memarch_b200.optim import Instinct
    torch.manual_seed(0)
    names = ["light_a.0.up.weight", "fish.up", "heavy.0.up.weight"]
    ps = [torch.nn.Parameter(torch.randn(8, 8)) for _ in names]
    a = Instinct(ps, OptConfig(lr=1e-2, norm="hs", scale=0.12, gnorm=True, gnorm_rawrel=True, rel_every=1, snr=True,
                               snr_skip=("fish.",)), names=names)
    assert a._snr_on == [True, False, True]
    b = Instinct(ps, OptConfig(lr=1e-2, norm="hs", scale=0.12, snr=True, snr_only=("light_a.",)), names=names)
    assert b._snr_on == [True, False, False]
    a.prepare(torch.tensor(1.0), torch.ones(4))
    gs = [torch.randn(8, 8) * s for s in (1.0, 10.0, 100.0)]
    w = [p.detach().clone() for p in ps]
    for p, g in zip(ps, gs):
        a.update(p, g.clone())
    want = torch.stack([g.norm() / (x.norm() + 1e-8) for g, x in zip(gs, w)])
    assert torch.allclose(a.rel, want, rtol=2e-2) and a.rel[2] > 50 * a.rel[0]    # not the constant of a unit gradient


def test_layer_pool_training_by_kind_through_the_loop(tmp_path, monkeypatch):
    from memarch_b200.train.loop import make_data, train
    monkeypatch.chdir(tmp_path)
    w = make_corpus(str(tmp_path / "corpus"), docs=60)
    env = {"VOCAB": "2048", "NO_MEM": "1", "WATCHDOG": "0", "CORPUS": json.dumps(w), "CORPUS_ROOT": str(tmp_path / "corpus"),
           "KINDS": json.dumps({"prose": {"web": 2.0}, "formal": {"code": 1.0}}), "FISH_N": "6", "FISH_HF": "64",
           "FISH_KINDS": "2", "FISH_POOL": "4", "FISH_C": "2",
           "OPT_KW": json.dumps({"norm": "hs", "scale": 0.12, "card_by_kind": True, "cards": 3})}
    a = Args(seq=48, batch=4, micro=4, steps=6, eval_every=3)
    data = make_data(a, "cpu", env)
    kinds = []
    for _ in range(6):
        data.batch(4, 48)
        ex = data.extra
        assert ex["kind"].shape == (4, 1) and ex["fish"].shape == (4, 2)
        kinds.append(int(ex["kind"][0, 0]))
    assert kinds.count(0) == 4 and kinds.count(1) == 2                     # 2:1 by the weights of the kinds
    data.loader.close()
    buf = io.StringIO()
    env2 = dict(env, EVAL_NOFISH="1", CKPT_DIR=str(tmp_path / "ck"), CKPT_EVERY="3")
    log = train(a, "cpu", env=env2, out=buf)["tiny"]
    assert all(math.isfinite(e["val"]) for e in log) and "fish_router_acc" in buf.getvalue()
    assert "val_nofish" in log[-1]["sets"] and log[-1]["sets"]["val_nofish"] != log[-1]["val"]
    buf = io.StringIO()
    a2 = Args(seq=48, batch=4, micro=4, steps=8, eval_every=8)
    train(a2, "cpu", env=dict(env2, FISH_RESET="1", FISH_FULL_FROM="8"), out=buf)
    assert "resuming at step 7" in buf.getvalue() and "layer pool reset to its initial weights" in buf.getvalue()


def test_total_diagnostics_of_a_run(tmp_path, monkeypatch):
    from memarch_b200.train.diag import Diag
    from memarch_b200.train.loop import train
    monkeypatch.chdir(tmp_path)
    quiet = io.StringIO()
    d = Diag({}, quiet)
    d.phase("x"), d.step(50), d.close()
    assert quiet.getvalue() == ""                                          # off: nothing at all
    buf = io.StringIO()
    env = {"VOCAB": "512", "NO_MEM": "1", "WATCHDOG": "0", "DIAG": "1", "DIAG_EVERY": "2", "DIAG_PROF": "2",
           "DIAG_DIR": str(tmp_path / "tr"), "OPT_KW": json.dumps({"norm": "hs", "scale": 0.12})}
    train(Args(seq=32, batch=2, micro=2, steps=6, eval_every=6), "cpu", env=env, out=buf)
    text = buf.getvalue()
    for want in ("[diag] phase 'start'", "phase 'data ready'", "phase 'model tiny and optimizer built'",
                 "phase 'first step enqueued'", "[diag] step 2:", "[diag] step 4:", "host RSS", "trace: started at step 2"):
        assert want in text, want
    trace = tmp_path / "tr" / "trace_step2.json"
    assert trace.exists() and trace.stat().st_size > 1000 and "trace: written" in text


def test_rollback_guard_by_kind_and_steps_of_another_shape():
    from memarch_b200.train.guards import RollbackGuard
    xs = batches(8)
    tr = tiny_trainer()
    rb = RollbackGuard(tr, ratio=1.5, warm=2, lr_mul=0.5, kinds=3)
    real = tr.step
    scale = {"v": 1.0}

    def scaled(xy, step, **kw):
        return real(xy, step, **kw) * scale["v"]
    tr.step = scaled
    for s in range(3):
        rb.step(xs[s], s, kind=0)
    scale["v"] = 3.0                                         # kind 1 lives at three times the loss: its own running mean
    rb.step(xs[3], 3, kind=1)
    assert int(rb.n_hit) == 0 and float(rb.lema[1]) > 2 * float(rb.lema[0]) and float(rb.lema[2]) == 0
    rb.step(xs[4], 4, kind=1)
    assert int(rb.n_hit) == 0                                # judged against kind 1's mean: no spike
    rb.step(xs[5], 5, kind=0)                                # the same loss under kind 0 IS a spike
    assert int(rb.n_hit) == 1 and bool(rb.cool[0]) and not bool(rb.cool[1]) and bool(rb.rep)
    scale["v"] = 1.0
    rb.step(xs[6], 6, kind=0)                                # the replay; the kind's flag stays until its own next step
    assert bool(rb.cool[0]) and not bool(rb.rep)
    scale["v"] = 3.0
    rb.step(xs[7], 7, kind=0)                                # just rejected: this time the kind learns
    assert int(rb.n_hit) == 1 and not bool(rb.cool[0])
    # a batch of another shape (short synthetic rows) is stepped, not judged, and becomes undoable
    scale["v"] = 1.0
    before = [p.detach().clone() for p in tr.params]
    short = torch.randint(0, 256, (8, 17))
    n0 = rb.n
    rb.step(short, 8, kind=2)
    assert rb.n == n0 + 1 and float(rb.lema[2]) == 0 and rb.prev_xy.shape == xs[0].shape
    assert all(torch.equal(a, b) for a, b in zip(rb.snap_p, before))
    scale["v"] = 100.0
    rb.step(xs[0], 9, kind=1)                                # a spike right after it: the synthetic step is undone too
    assert int(rb.n_hit) == 2
    assert all(torch.equal(p.data, b) for p, b in zip(tr.params, before))


def test_token_preparation_on_the_loader_thread(tmp_path, monkeypatch):
    from memarch_b200 import build
    from memarch_b200.train.loop import train
    import memarch_b200.train.loop as loop_mod
    monkeypatch.chdir(tmp_path)
    torch.manual_seed(0)
    m = build("tiny", 2048, env={"NO_MEM": "1", "INDUCT": "lock", "INDUCT_MIX": "1"})
    hp = m.host_prep()
    x = torch.randint(0, 50, (3, 40))
    want, got = m.prep(x), hp(x)
    assert set(want) == set(got) and all(torch.equal(want[k], got[k]) for k in want)
    w = make_corpus(str(tmp_path / "corpus"), docs=60)
    env = {"VOCAB": "2048", "NO_MEM": "1", "WATCHDOG": "0", "CORPUS": json.dumps(w), "CORPUS_ROOT": str(tmp_path / "corpus"),
           "INDUCT": "lock", "INDUCT_MIX": "1", "OPT_KW": json.dumps({"norm": "hs", "scale": 0.12})}
    a = Args(seq=48, batch=4, micro=2, steps=4, eval_every=4)
    seen = []
    real = loop_mod.Trainer.step

    def spy(self, xy, step, preps=None, lr_mul=1.0):
        seen.append(preps)
        return real(self, xy, step, preps, lr_mul)
    monkeypatch.setattr(loop_mod.Trainer, "step", spy)
    plain = train(a, "cpu", env=env, out=io.StringIO())["tiny"]
    assert all(p is None for p in seen)
    seen.clear()
    fed = train(a, "cpu", env=dict(env, CPU_PREP="1"), out=io.StringIO())["tiny"]
    assert len(seen) == 4 and all(len(p) == 2 and {"ind_cand", "ind_on", "ind_bk", "ind_src"} <= set(p[0]) for p in seen)
    assert seen[0][0]["ind_cand"].shape[0] == 2                            # one dict per micro-batch
    assert abs(plain[-1]["val"] - fed[-1]["val"]) < 1e-5                   # the same run, prepared elsewhere


def test_experiment_switches_combined_train_together():
    """Everything at once, as a long run would have it: tethered light blocks, hoop, word-level rules, needle terms,
    rotating full heavy layer, trunk guard, dump-proof final norm, and the optimizer's late rules."""
    from memarch_b200 import OptConfig, TrainConfig, build
    from memarch_b200.data.reminders import Reminders
    from memarch_b200.train import Trainer
    from memarch_b200.train.loop import needle_preps
    torch.manual_seed(0)
    env = {"NO_MEM": "1", "MOE_ACT": "relu2", "ROPE_MEM": "1", "ROPE_WIN": "8", "ROPE_SPAN_CAP": "12", "ROPE_K": "2",
           "ROPE_LINKS": "3", "ROPE_HIER_G": "4", "ROPE_HIER_BM": "16", "ROPE_CHUNK": "32", "ROPE_QFRAC": "0.8",
           "UROBOROS": "1", "INST_WORD": "1", "IW_REWRITE": "1", "REMIND_W": "1.0", "REMIND_N": "4", "REMIND_USE_W": "0.2",
           "REMIND_MASK_MAIN": "1", "HEAVY_ROTATE": "1", "LAYER_STATS": "1", "HN_GUARD_W": "0.5", "HN_GUARD_MEAN": "0.5",
           "NORM_DUMP_PROJ": "1", "ATTN_GAIN": "1.1", "PREV_IN": "1"}
    m = build("tiny", 2048, env=env)
    tr = Trainer(m, TrainConfig(name="tiny", stage="ABX", steps=20, batch=4, micro=2, seq=64, lr=3e-3, warmup=2),
                 OptConfig(lr=3e-3, norm="hs", scale=0.12, rel_every=2, stream_proj=True, m_rate=True, m_rate_warm=2, safe16=True,
                           culprit="ema", gnorm=True, gnorm_rawrel=True, wd_norm=0.01, norm_anchor=True), stage="ABX")
    rem = Reminders(1.0, T=64, n=4, dist=8, seed=0, V=2048, tok0=1000, same_fmt=True, blank=True)
    g = np.random.default_rng(0)
    losses = []
    for step in range(5):
        xy, extra = rem(g.integers(0, 900, (4, 65)).astype(np.int32), n=step)
        xy_t = torch.from_numpy(xy).long()
        losses.append(float(tr.step(xy_t, step, needle_preps(m, xy_t, extra, 2))))
    assert all(math.isfinite(v) for v in losses), losses
    assert tr.opt.U is not None and m.stream_u is tr.opt.U and tr.opt.mrl_n == 5
    for k in ("rope_share", "uroboros_corr", "iw", "remind_hit", "remind_rope_share", "remind_main_masked", "moe_fill", "hn_mean"):
        assert k in m.stats, k
    assert all(torch.isfinite(p).all() for p in m.parameters())


def test_hoop_budget_steps_down_in_the_loop(tmp_path, monkeypatch):
    from memarch_b200.models.fishki import Uroboros
    from memarch_b200.train.loop import train
    monkeypatch.chdir(tmp_path)
    # the head "knows its errors" and most words count as eaten: the budget goes down one level per evaluation
    monkeypatch.setattr(Uroboros, "stats", staticmethod(lambda pred, nll, idx, eat: {
        "uroboros_eaten": torch.tensor(0.97), "uroboros_corr": torch.tensor(0.9),
        "uroboros_nll_sel": nll.mean().detach(), "uroboros_nll_skip": nll.mean().detach()}))
    env = {"VOCAB": "512", "NO_MEM": "1", "WATCHDOG": "0", "UROBOROS": "1", "UROBOROS_LEVELS": "0.25,0.125,0.0625",
           "OPT_KW": json.dumps({"norm": "hs", "scale": 0.12})}
    buf = io.StringIO()
    log = train(Args(seq=64, batch=2, micro=2, steps=3, eval_every=1), "cpu", env=env, out=buf)["tiny"]
    text = buf.getvalue()
    assert "hoop: budget 0.25 -> 0.125" in text and "hoop: budget 0.125 -> 0.0625" in text
    assert all(math.isfinite(e["val"]) for e in log)
