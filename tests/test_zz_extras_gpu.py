"""The PyTorch-level components (rope memory, fishki pools, uroboros head, int8 numerics, legacy model families) on a
B200: the device result must agree with the same module evaluated on the CPU in fp32."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda", 0)


def test_rope_memory_device_matches_cpu():
    from memarch_b200.models import rope_memory as rm
    dev = _dev()
    torch.manual_seed(0)
    B, H, T, hd = 2, 2, 256, 32
    cfg = rm.RopeCfg(K=2, links=3, win=16, span_cap=24, chunk=64)
    q, k, v = (torch.randn(B, H, T, hd) for _ in range(3))
    s = torch.rand(B, T) * 2
    own, apos, avalid = rm.anchors_from_surprise(s.clone(), 1.4, 32)
    qc = q.clone().requires_grad_(True)
    out_c, share_c, _ = rm.rope_attention(qc, k, v, own, apos, avalid, cfg)
    out_c.square().sum().backward()
    own_g, apos_g, avalid_g = rm.anchors_from_surprise(s.to(dev), 1.4, 32)
    assert torch.equal(apos_g.cpu(), apos) and torch.equal(avalid_g.cpu(), avalid)
    qg = q.to(dev).requires_grad_(True)
    out_g, share_g, _ = rm.rope_attention(qg, k.to(dev), v.to(dev), own_g, apos_g, avalid_g, cfg)
    out_g.square().sum().backward()
    # fp32 on both sides: only the summation order differs.  A near-tie between two anchors' scores may still route a
    # query differently on the two devices, so the comparison allows a handful of rows to disagree.
    bad = ((out_g.cpu() - out_c).abs() > 2e-3).float().mean().item()
    assert bad < 0.01, bad
    assert abs(float(share_g) - float(share_c)) < 1e-2
    gbad = ((qg.grad.cpu() - qc.grad).abs() > 5e-3 * qc.grad.abs().max().clamp(min=1.0)).float().mean().item()
    assert gbad < 0.01, gbad


def test_fishki_and_uroboros_device_match_cpu():
    from memarch_b200.models import fishki
    dev = _dev()
    torch.manual_seed(0)
    p = fishki.FishPool(64, n=8, hf=128, kinds=4, pool=3, center=True)
    h = torch.randn(2, 40, 64)
    y_c = p(h, p.sets[2])
    pg = copy.deepcopy(p).to(dev)
    y_g = pg(h.to(dev), pg.sets[2])
    assert (y_g.cpu() - y_c).abs().max() < 2e-3 * y_c.abs().max().clamp(min=1.0)
    ce_c, _, lg_c = p.router_loss(h, torch.tensor([1, 3]))
    ce_g, _, lg_g = pg.router_loss(h.to(dev), torch.tensor([1, 3], device=dev))
    assert (lg_g.cpu() - lg_c).abs().max() < 2e-3 and abs(ce_g.item() - ce_c.item()) < 2e-3
    u = fishki.Uroboros(32)
    lh, s = torch.randn(2, 64, 32), torch.rand(2, 64) * 5
    pred_c = u.predict(lh, s)
    ug = copy.deepcopy(u).to(dev)
    pred_g = ug.predict(lh.to(dev), s.to(dev))
    assert (pred_g.cpu() - pred_c).abs().max() < 2e-3
    idx_c, _ = u.select(pred_c, 0.25)
    idx_g, _ = ug.select(pred_c.to(dev), 0.25)                 # same scores: the selection itself must agree exactly
    assert torch.equal(idx_g.cpu(), idx_c)


def test_int8_numerics_device_match_cpu():
    from memarch_b200.ops import int8
    dev = _dev()
    torch.manual_seed(0)
    x, w = torch.randn(64, 128), torch.randn(96, 128) * 0.1
    (qg, sg), (qc, sc) = int8.fq(x.to(dev), 1), int8.fq(x, 1)
    assert torch.equal(qg.cpu(), qc) and torch.allclose(sg.cpu(), sc)
    xc, wc = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    yc = int8._I8Linear.apply(xc, wc)
    yc.sum().backward()
    xg, wg = x.to(dev).requires_grad_(True), w.to(dev).requires_grad_(True)
    yg = int8._I8Linear.apply(xg, wg)
    yg.sum().backward()
    assert (yg.cpu() - yc).abs().max() < 2e-3 * yc.abs().max()
    assert (wg.grad.cpu() - wc.grad).abs().max() < 1e-2 * wc.grad.abs().max()          # bf16 products: one ulp apart at most


@pytest.mark.parametrize("name", ["cards", "plan8", "planwc8", "sketch8", "surpc20", "surpq20", "Fsmall"])
def test_legacy_families_run_on_device(name):
    """One forward + backward of an earlier model generation on the GPU: loss and cost agree with the CPU fp32 run of
    the same weights, gradients reach the parameters."""
    from memarch_b200.build import build
    dev = _dev()
    torch.manual_seed(0)
    m = build(name, 512)
    m.train()
    T = 128 if name == "surpq20" else 64
    xy = torch.randint(0, 512, (2, T + 1))
    mg = copy.deepcopy(m).to(dev)
    torch.manual_seed(1)
    out_c, cost_c = m(xy[:, :-1])
    loss_c = m.train_loss(out_c, xy[:, 1:], True)
    torch.manual_seed(1)
    xg = xy.to(dev)
    out_g, cost_g = mg(xg[:, :-1])
    loss_g = mg.train_loss(out_g, xg[:, 1:], True)
    (loss_g + 0.01 * cost_g.float()).backward()
    assert torch.isfinite(loss_g).item()
    assert abs(loss_g.item() - loss_c.item()) < 2e-2 * max(1.0, abs(loss_c.item()))
    assert abs(float(cost_g.detach()) - float(cost_c.detach())) < 2e-2 * max(1.0, abs(float(cost_c.detach())))
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in mg.parameters())


@pytest.mark.parametrize("name,env", [
    ("tether", {"ROPE_MEM": "1", "ROPE_WIN": "16", "ROPE_SPAN_CAP": "24", "ROPE_LINKS": "3", "ROPE_K": "2", "ROPE_HIER_G": "4",
                "ROPE_HIER_BM": "32", "ROPE_CHUNK": "64", "ROPE_QFRAC": "0.7", "REMIND_USE_W": "0.5"}),
    ("hoop", {"UROBOROS": "1", "UROBOROS_BUDGET": "0.25"}),
    ("pool", {"FISH_N": "6", "FISH_HF": "128", "FISH_KINDS": "2", "FISH_POOL": "4"}),
    ("all_words", {"HEAVY_ALL": "1"}),
    ("words", {"INST_WORD": "1", "IW_OK": "0.05", "IW_REWRITE": "1", "NORM_DUMP_PROJ": "1", "HN_GUARD_W": "1.0",
               "HN_GUARD_MEAN": "0.1"}),
    ("needles", {"REMIND_CAND": "1", "REMIND_MASK_MAIN": "1", "REMIND_STRICT": "1"}),
])
def test_main_model_switches_device_matches_cpu(name, env):
    """The experiment switches of the main model (anchor-routed read, hoop, layer pool, heavy layers on all words,
    word-level rules, needle terms): loss on the device against the same weights on the CPU, and a finite backward."""
    from memarch_b200 import build
    dev = _dev()
    torch.manual_seed(0)
    e = {"NO_MEM": "1", "MOE_ACT": "relu2", "REMIND_W": "1.0", "REMIND_N": "4", "REMIND_TOK0": "100"}
    e.update(env)
    mc = build("tiny", 1024, env=e).train()
    mg = copy.deepcopy(mc).to(dev)
    xy = torch.randint(0, 1024, (2, 129))
    rem = torch.zeros(2, 128, dtype=torch.int8)
    rem[:, 90:98:2] = 1
    xy[:, 91:99:2] = torch.randint(612, 676, (2, 4))                       # targets of the answers: value tokens (< vocabulary)
    extra = {"rem": rem, "rem_vals": xy[:, 91:99:2].int()}
    prep = {"kind": torch.ones(2, 1, dtype=torch.long), "fish": torch.tensor([mc.fish.sets[1][:2]] * 2)} if name == "pool" else None
    on = lambda t, d: {k: v.to(d) for k, v in t.items()} if t is not None else None
    losses = []
    for m, d in ((mc, torch.device("cpu")), (mg, dev)):
        out, cost = m(xy[:, :-1].to(d), on(prep, d))
        loss = m.train_loss(out, xy[:, 1:].to(d), True, extra=on(extra, d))
        loss.backward()
        losses.append(float(loss))
        assert all(torch.isfinite(p.grad).all() for p in m.parameters() if p.grad is not None)
    assert abs(losses[0] - losses[1]) < 3e-2 * max(1.0, abs(losses[0])), (name, losses)
