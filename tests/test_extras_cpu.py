"""Secondary model features on CPU: routed long-range attention against a per-query brute force, fishki pools,
uroboros selection, int8 numerics, recall toy task."""
import math

import numpy as np
import pytest
import torch

from memarch_b200.models import fishki
from memarch_b200.models import rope_memory as rm
from memarch_b200.ops import int8


def brute_rope(q, k, v, s, tau, A, cfg):
    """Per-query Python loop straight from the definition."""
    B, H, T, hd = q.shape
    out = torch.zeros_like(q)
    sc = 1 / math.sqrt(hd)
    for b in range(B):
        anchor = (s[b] > tau).clone()
        anchor[0] = True
        pos = [t for t in range(T) if anchor[t]][:A]
        nxt = pos[1:] + [T]
        for h in range(H):
            for i in range(T):
                cand = []
                for a, (p0, p1) in enumerate(zip(pos, nxt)):
                    if max(p1, p0 + cfg.win) > i:
                        continue
                    links = [p0 + l for l in range(min(cfg.links, cfg.span_cap)) if p0 + l < p1 and p0 + l < T]
                    sco = [(float(q[b, h, i] @ k[b, h, j]) * sc, j) for j in links]
                    best = max(sco)
                    cand.append((best[0], -a, a, best[1]))
                cand.sort(reverse=True)
                keys, bias = [], []
                for sc_a, _, a, tp in cand[:cfg.K]:
                    en = min(nxt[a], pos[a] + cfg.span_cap, i - cfg.win + 1)
                    for t in range(pos[a], en):
                        keys.append(t)
                        bias.append(sc_a * cfg.rgrad_scale if cfg.rgrad else 0.0)
                for t in range(max(0, i - cfg.win + 1), i + 1):
                    keys.append(t)
                    bias.append(0.0)
                kk = torch.tensor(keys)
                logit = (k[b, h, kk] @ q[b, h, i]) * sc + torch.tensor(bias)
                out[b, h, i] = logit.softmax(0) @ v[b, h, kk]
    return out


def test_rope_memory_matches_brute_force_and_has_gradients():
    torch.manual_seed(0)
    B, H, T, hd = 2, 2, 96, 16
    cfg = rm.RopeCfg(K=2, links=3, win=8, span_cap=12, chunk=32)
    q, k, v = (torch.randn(B, H, T, hd) for _ in range(3))
    s = torch.rand(B, T) * 2
    own, apos, avalid = rm.anchors_from_surprise(s.clone(), 1.4, 24)
    qq = q.clone().requires_grad_(True)
    out, share, (tidx, tval, tpos) = rm.rope_attention(qq, k, v, own, apos, avalid, cfg)
    want = brute_rope(q, k, v, s, 1.4, 24, cfg)
    assert (out - want).abs().max() < 1e-4
    assert 0 < float(share) < 1 and bool(tval.any())
    out.square().sum().backward()
    assert qq.grad.abs().sum() > 0
    layer = rm.RopeMemoryAttention(32, 2, cfg)
    y, _ = layer(torch.randn(2, 96, 32), s, 1.4)
    assert y.shape == (2, 96, 32)


def _rope_case(T=200, A=60, seed=0):
    torch.manual_seed(seed)
    B, H, hd = 2, 2, 16
    q, k = torch.randn(B, H, T, hd), torch.randn(B, H, T, hd)
    s = torch.rand(B, T) * 2
    return q, k, s, rm.anchors_from_surprise(s.clone(), 1.3, A)


def test_rope_two_level_search():
    q, k, s, (own, apos, avalid) = _rope_case()
    base = dict(K=3, links=3, win=8, span_cap=12, chunk=64, G=4, BM=16)
    exact = rm.route_exact(q, k, own, apos, avalid, rm.RopeCfg(route="exact", **base))
    # every complete group kept: the exact search (T not a multiple of BM, A not a multiple of G)
    full = rm.route_hier(q, k, own, apos, avalid, rm.RopeCfg(NB=64, **base))
    for a, b in zip(exact, full):
        assert torch.equal(a, b)
    # few groups kept: a subset of what may open, recent anchors (the tail) always reachable
    cfg = rm.RopeCfg(NB=2, **base)
    tidx, tval, tpos = rm.route_hier(q, k, own, apos, avalid, cfg)
    assert bool(tval.any()) and not all(torch.equal(a, b) for a, b in zip(exact, (tidx, tval, tpos)))
    nx = rm._open_from(apos, avalid, q.shape[2], cfg)
    qi = torch.arange(q.shape[2])[None, None, :, None]
    opened_at = nx.gather(1, tidx.reshape(2, -1)).view_as(tidx)
    assert bool(((opened_at <= qi) | ~tval).all())
    assert bool((own.gather(1, tpos.reshape(2, -1)).view_as(tidx) == tidx)[tval].all())
    # nothing flows backwards in time: what lies after position t does not change the choice up to t
    t = 117
    q2, k2 = q.clone(), k.clone()
    q2[:, :, t + 1:], k2[:, :, t + 1:] = torch.randn_like(q2[:, :, t + 1:]), torch.randn_like(k2[:, :, t + 1:])
    again = rm.route_hier(q2, k2, own, apos, avalid, cfg)
    for a, b in zip((tidx, tval, tpos), again):
        assert torch.equal(a[:, :, :t + 1], b[:, :, :t + 1])
    with pytest.raises(ValueError):
        rm.route(q, k, own, apos, avalid, rm.RopeCfg(route="flat"))
    # bf16 operands (the device path's arithmetic): the exact search on the rounded queries and keys
    rounded = rm.route_exact(q.bfloat16().float(), k.bfloat16().float(), own, apos, avalid, rm.RopeCfg(route="exact", **base))
    low = rm.route_exact(q, k, own, apos, avalid, rm.RopeCfg(route="exact", route_bf16=True, **base))
    assert all(torch.equal(a, b) for a, b in zip(rounded, low))


def test_rope_query_and_document_masks():
    q, k, s, (own, apos, avalid) = _rope_case(T=96, A=30, seed=1)
    v = torch.randn_like(q)
    cfg = rm.RopeCfg(K=2, links=3, win=8, span_cap=12, chunk=32, G=4, BM=16)
    out, share, (tidx, tval, _) = rm.rope_attention(q, k, v, own, apos, avalid, cfg)
    qmask = torch.rand(2, 96) < 0.5
    out_m, share_m, _ = rm.rope_attention(q, k, v, own, apos, avalid, cfg, qmask=qmask)
    only_win, _, _ = rm.rope_attention(q, k, v, own, apos, avalid, cfg, qmask=torch.zeros(2, 96, dtype=torch.bool))
    sel = qmask[:, None, :, None].expand_as(out)
    assert torch.allclose(out_m[sel], out[sel]) and torch.allclose(out_m[~sel], only_win[~sel])
    assert float(share_m) < float(share)
    docs = (torch.arange(96)[None] >= torch.tensor([[40], [70]])).long()
    tv = rm.mask_route(tidx, tval, apos, docs=docs)
    a_doc = docs.gather(1, apos).gather(1, tidx.reshape(2, -1)).view_as(tidx)
    assert bool((a_doc == docs[:, None, :, None])[tv].all()) and int(tv.sum()) < int(tval.sum())
    out_d, _, _ = rm.rope_attention(q, k, v, own, apos, avalid, cfg, docs=docs)
    assert torch.allclose(out_d[0, :, :40], out[0, :, :40]) and not torch.allclose(out_d, out)


def test_fishki_pool_and_router():
    torch.manual_seed(0)
    assert fishki.pools(4, 16, 6) == [[0, 1, 2, 3, 4, 5], [4, 5, 6, 7, 8, 9], [8, 9, 10, 11, 12, 13], [12, 13, 14, 15, 0, 1]]
    p = fishki.FishPool(32, n=8, hf=64, kinds=4, pool=3, center=True)
    h = torch.randn(2, 10, 32, requires_grad=True)
    y = p(h, p.sets[1])
    y.sum().backward()
    used = {i for i in range(8) if p.up.grad[i].abs().sum() > 0}
    assert used == set(p.sets[1])
    ce, acc, logits = p.router_loss(h, torch.tensor([1, 3]))
    assert logits.shape == (2, 4) and ce.item() > 0


def test_uroboros_select_loss_budget():
    torch.manual_seed(0)
    u = fishki.Uroboros(16)
    lh, s = torch.randn(2, 20, 16), torch.rand(2, 20) * 5
    pred = u.predict(lh, s)
    assert pred.shape == (2, 20) and bool((pred >= 0).all())
    idx, valid = u.select(pred, 0.25)
    assert idx.shape == (2, 5) and bool((idx[:, 0] == 0).all()) and bool((idx[:, 1:] > idx[:, :-1]).all())
    nll = torch.rand(2, 20) * 6
    u.loss(pred, nll).backward()
    assert u.l1.weight.grad.abs().sum() > 0
    st = u.stats(pred, nll, idx, eat=1.0)
    assert set(st) == {"uroboros_eaten", "uroboros_corr", "uroboros_nll_sel", "uroboros_nll_skip"}
    lv = (0.25, 0.2, 0.15, 0.1)
    assert u.next_budget(0.25, 0.9, lv) == 0.2             # one level at a time
    assert u.next_budget(0.25, 0.5, lv) == 0.25            # need 0.625: stays
    assert u.next_budget(0.2, 0.95, lv, corr=0.1) == 0.2   # head does not know its errors yet


def test_int8_linear_and_bmm_close_to_fp32():
    torch.manual_seed(0)
    x, w = torch.randn(64, 256, requires_grad=True), torch.randn(320, 256, requires_grad=True)
    y = int8.linear_i8(x, w)
    ref = x @ w.t()
    assert (y - ref).norm() / ref.norm() < 0.02
    g = torch.randn_like(y)
    y.backward(g)
    assert (x.grad - g @ w).norm() / (g @ w).norm() < 0.03
    assert (w.grad - g.t() @ x).norm() / (g.t() @ x).norm() < 0.02      # weight gradient is bf16, not int8
    xe, we = torch.randn(2, 16, 256, requires_grad=True), torch.randn(2, 256, 300, requires_grad=True)
    ye = int8.bmm_i8(xe, we)
    assert (ye - torch.bmm(xe, we)).norm() / torch.bmm(xe, we).norm() < 0.02
    ye.sum().backward()
    assert xe.grad is not None and we.grad is not None
    q, s = int8.fq(torch.tensor([[0.5, -1.0, 0.25]]), 1)
    assert q.tolist() == [[64.0, -127.0, 32.0]] and abs(float(s) - 1 / 127) < 1e-9


def test_recall_toy_task():
    from memarch_b200.data.synth import recall_batch
    x, y, mask = recall_batch(8, n_pairs=4, n_keys=16, n_vals=16, seed=0)
    assert x.shape == (8, 10) and mask.sum() == 8
    for b in range(8):
        key = int(x[b, -1])
        pairs = x[b, :8].view(4, 2)
        val = int(pairs[pairs[:, 0] == key][0, 1])
        assert int(y[b, -1]) == val


def test_long_context_generators_and_runs():
    import numpy as np
    from memarch_b200.experiments import long_context as lc
    g = torch.Generator().manual_seed(0)
    x, y, ans = lc.recall_task(4, pairs=3, filler=20, queries=2, g=g)
    assert x.shape == (4, 2 * 3 + 20 + 2 * 2 - 1) and (y != -100).sum() == 8
    for b in range(4):
        kv = x[b, :6].view(3, 2)
        for a in ans:
            key = int(x[b, a])
            assert int(y[b, a]) == int(kv[kv[:, 0] == key][0, 1])
    toks = np.random.default_rng(0).integers(100, 1000, size=5000)
    xb, tgt, depth = lc.needle_batch(toks, 3, 256, (3000, 3001), g)
    for b in range(3):
        d = depth[b]
        assert xb[b, d:d + 3].tolist() == [11, 12, 13] and int(xb[b, d + 4]) == int(tgt[b])
        assert xb[b, -4:-1].tolist() == [11, 12, 13] and int(xb[b, -1]) == int(xb[b, d + 3])
    s = torch.rand(6, 256) * 3
    r = lc.anchor_chunks(s, 1.5, 0.25, chunks=(64, 128))
    assert 0 < r["per_text"] < 1 and r["per_chunk_64"] >= r["per_text"] - 1e-6
    acc, m = lc.recall_run("Fv2s", steps=3, B=2, pairs=2, fillers=(8,), device="cpu", vocab=32768, eval_B=2, out=lambda *a: None)
    assert set(acc) == {8}
    d = lc.recall_diagnose(m, pairs=2, filler=64, B=2)
    assert 0 <= d["stored"] <= 1 and d["cards"] > 0
    rows = lc.long_speed(models=("tiny",), lens=(64,), warmup=1, n=1, device="cpu", vocab=512, out=lambda *a: None)
    assert rows[0]["ms"] > 0


def test_instinct_gradient_surge_damping_and_surprise_brake():
    from memarch_b200.config import OptConfig
    from memarch_b200.optim.instinct import Instinct

    def run(damp, surge, spike):
        torch.manual_seed(0)
        p = torch.nn.Parameter(torch.randn(16, 8))
        w0 = p.detach().clone()
        opt = Instinct([p], OptConfig(lr=1e-2, norm="tensor", scale=1.0, damp=damp, surge_thr=surge))
        steps = []
        for s in range(6):
            g = torch.randn(16, 8) * (0.01 * (50.0 if (spike and s == 5) else 1.0))
            loss = torch.tensor(3.0 if not (surge and s == 5) else 9.0)
            before = p.detach().clone()
            opt.prepare(loss, torch.ones(4))
            opt.update(p, g)
            opt.finish()
            steps.append((p.detach() - before).norm().item())
        return steps, opt
    plain, _ = run(0.0, 0.0, True)
    damped, opt = run(3.0, 0.0, True)
    assert abs(plain[4] - damped[4]) < 1e-9                       # calm steps are bit-identical in size
    assert damped[5] < 0.2 * plain[5] and float(opt.df[0]) < 0.2   # the 50x surge is braked
    calm, _ = run(0.0, 0.3, False)
    assert calm[5] < 0.3 * calm[4]                                 # loss 3x the expectation: -s = 2 > 0.3


def test_layer_diag_times_heavy_layers():
    from memarch_b200 import build
    from memarch_b200.utils.profile import LayerDiag, bucket_of
    torch.manual_seed(0)
    m = build("tiny", 256, env={"NO_MEM": "1"})
    d = LayerDiag(m)
    x = torch.randint(0, 256, (2, 33))
    out, cost = m(x[:, :-1])
    m.train_loss(out, x[:, 1:], True).backward()
    rows = d.report()
    d.close()
    assert len(rows) == len(m.heavy) and all(r["fwd_ms"] > 0 and r["bwd_ms"] > 0 for r in rows)
    assert bucket_of("void mb::gemm_tc2_kernel<false, true>") == "own tcgen05 gemm"
    assert bucket_of("nvjet_tst_256x256_64x4_2x1_2cta_v_bz_TNT") == "library gemm"
    assert bucket_of("mb::instinct_apply<4>") == "optimizer"


def test_ce_exact_under_a_common_logit_offset():
    """Adding a huge constant to every logit of a row must not change the loss or the gradient, and every gradient
    row sums to zero (the softmax null space): the forward LSE and the backward probabilities use one rounding."""
    from memarch_b200.ops import ref
    torch.manual_seed(0)
    N, d, V = 64, 32, 500
    h = torch.randn(N, d)
    w = torch.randn(V, d) * 0.2
    y = torch.randint(0, V, (N,))
    hb = torch.cat([h, torch.ones(N, 1)], 1)                  # a bias column carries the offset
    for off in (0.0, 3000.0):
        wb = torch.cat([w, torch.full((V, 1), off)], 1)
        total, gh, gw, *_ = ref.linear_ce(hb, wb, y, None, None, None, None, None, 16, None)
        if off == 0.0:
            base, gh0 = total, gh
        else:
            assert abs(float(total) - float(base)) < 2e-3 * abs(float(base))
            cos = torch.nn.functional.cosine_similarity(gh[:, :d].flatten(), gh0[:, :d].flatten(), dim=0)
            assert cos > 0.995
    lo = hb @ wb.t()
    G = torch.softmax(lo - lo.max(-1, keepdim=True).values, -1)
    G[torch.arange(N), y] -= 1
    assert G.sum(-1).abs().max() < 1e-5


def test_slot_table_and_flat_index_are_mutual_inverses():
    from memarch_b200.ops import ref
    torch.manual_seed(0)
    N, k, E, C = 200, 2, 8, 40
    e_flat = torch.randint(0, E + 1, (N, k))                 # E = nowhere
    w = torch.rand(N, k)
    table, wtab, flat_idx, dropped = ref.moe_slots(e_flat, w, E, C)
    ok = flat_idx < E * C
    tok = torch.arange(N)[:, None].expand(-1, k)
    assert torch.equal(table[flat_idx[ok]], tok[ok])          # a placed choice finds its own token in its slot
    used = table < N
    assert int(used.sum()) == int(ok.sum())
    assert torch.allclose(wtab[flat_idx[ok]], w[ok])
    per = torch.bincount(e_flat[e_flat < E], minlength=E)
    assert abs(float(dropped) - float(1 - ok.sum() / (e_flat < E).sum())) < 1e-6
    assert all(int(used.view(E, C)[e].sum()) == min(int(per[e]), C) for e in range(E))


def test_nomem_model_ignores_its_memory():
    """Honest-task control: with `use_memory=False` the memory and re-reading contribute nothing."""
    from memarch_b200 import build
    torch.manual_seed(0)
    m = build("Fv2s_nomem", 256, env={})
    x = torch.randint(0, 256, (2, 97))
    out, cost = m(x[:, :-1])
    loss = m.train_loss(out, x[:, 1:], True)
    loss.backward()
    assert float(cost) == 0.0
    g = [p.grad for n, p in m.named_parameters() if n.startswith(("memory.", "reread.")) and p.grad is not None]
    assert all(float(t.abs().max()) == 0.0 for t in g)


def test_momentum_host_offload_is_bit_identical_and_checkpoints():
    """The momentum rests in host memory and visits the device of its weight only for the update: same weights as the
    resident optimizer after every step, state survives a checkpoint blob, bank swaps keep the offload."""
    from memarch_b200.config import OptConfig
    from memarch_b200.optim.instinct import Instinct
    torch.manual_seed(0)
    shapes = [(64, 32), (4, 32, 48), (100, 16), (16,)]
    w0 = [torch.randn(s) for s in shapes]

    def run(offload, steps, opt=None, ps=None):
        if opt is None:
            ps = [torch.nn.Parameter(w.clone()) for w in w0]
            opt = Instinct(ps, OptConfig(lr=1e-2, norm="hs", scale=0.12, offload_m=offload))
        g = torch.Generator().manual_seed(5 + opt.n_step)
        for _ in range(steps):
            for p in ps:
                opt.update(p, torch.randn(p.shape, generator=g))
        return opt, ps
    a, pa = run(False, 4)
    b, pb = run(True, 4)
    assert b.offload and all(t.device.type == "cpu" for t in b.m)
    assert all(torch.equal(x, y) for x, y in zip(pa, pb)) and all(torch.equal(x, y) for x, y in zip(a.m, b.m))
    sd = b.state_dict()
    assert "offload" not in sd and all(s_.data_ptr() != t.data_ptr() for s_, t in zip(sd["m"], b.m))
    ps2 = [torch.nn.Parameter(p.detach().clone()) for p in pb]
    c = Instinct(ps2, OptConfig(lr=1e-2, norm="hs", scale=0.12, offload_m=True))
    c.load_state_dict(sd)
    assert all(torch.equal(x, y) for x, y in zip(c.m, b.m)) and all(t.device.type == "cpu" for t in c.m)
    new = torch.nn.Parameter(torch.randn(6, 32, 48))
    old_m = b.m[1].clone()
    b.swap(pb[1], new, [0, None, 3, None, 1, None])
    assert b.m[1].shape == (6, 32, 48) and torch.equal(b.m[1][2], old_m[3]) and float(b.m[1][1].abs().sum()) == 0
    b.update(new, torch.randn(6, 32, 48))
    assert float(b.m[1][1].abs().sum()) > 0
    from memarch_b200.config import opt_from_env
    assert opt_from_env(OptConfig(), {"OPT_OFFLOAD": "1"}).offload_m


def test_dump_proof_norm_removes_the_common_direction():
    from memarch_b200.ops.extras import dump_proof_norm
    torch.manual_seed(0)
    x = (torch.randn(2, 40, 32) + 3.0 * torch.randn(32)).requires_grad_(True)    # a strong common vector
    w = torch.ones(32)
    u = torch.randn(32, requires_grad=True)
    y = dump_proof_norm(x, w, u)
    uh = (u / u.norm()).detach()
    assert (y @ uh).abs().max() < 1e-5
    plain = x.detach() * torch.rsqrt(x.detach().pow(2).mean(-1, keepdim=True) + 1e-6)
    assert torch.allclose(y.detach(), plain - (plain @ uh)[..., None] * uh, atol=1e-6)
    y.square().sum().backward()
    assert x.grad.abs().sum() > 0 and u.grad is None                             # the direction carries no gradient
    mean = x.detach().reshape(-1, 32).mean(0)
    a, b, c = dump_proof_norm(x, w, None), dump_proof_norm(x, w, torch.zeros(32)), dump_proof_norm(x, w, mean)
    assert torch.equal(a, b) and torch.allclose(a, c, atol=1e-6)
    assert dump_proof_norm(x.bfloat16(), w.bfloat16(), u).dtype == torch.bfloat16


def test_cap_shared_is_causal_and_leaves_small_common_vectors_alone():
    from memarch_b200.ops.extras import cap_shared
    torch.manual_seed(0)
    free = torch.randn(2, 96, 24)                                # zero-mean rows: nothing to cap
    assert torch.equal(cap_shared(free, 0.5, t0=8), free)
    off = free + 4.0 * torch.randn(24)
    out = cap_shared(off, 0.5, t0=16)
    assert torch.equal(out[:, :16], off[:, :16]) and not torch.equal(out[:, 16:], off[:, 16:])
    # a capped position is the input minus a multiple of its running mean
    n = torch.arange(1, 97.0)[:, None]
    m = off.cumsum(1) / n
    t = 50
    diff, mt = off[:, t] - out[:, t], m[:, t]
    k = (diff * mt).sum(-1) / (mt * mt).sum(-1)
    assert torch.allclose(diff, k[:, None] * mt, atol=1e-5) and bool(((k > 0) & (k < 1)).all())
    # causal: the future does not change the past
    other = off.clone()
    other[:, 60:] = torch.randn(2, 36, 24)
    assert torch.equal(cap_shared(other, 0.5, t0=16)[:, :60], out[:, :60])
    x = off.clone().requires_grad_(True)
    cap_shared(x, 0.5, t0=16).square().sum().backward()
    assert torch.isfinite(x.grad).all()


def test_short_top_names_the_leading_short_vocabulary_word(tmp_path):
    from memarch_b200.build import build
    cnt = np.zeros(512, np.int64)
    cnt[:100] = np.arange(100, 0, -1) * 50
    cnt[100:511] = 1
    np.save(tmp_path / "cnt.npy", cnt)
    torch.manual_seed(0)
    m = build("tiny", 512, env={"SHORT_V": "64", "TOKEN_COUNTS": str(tmp_path / "cnt.npy"), "NO_MEM": "1"})
    assert m.short_v == 64
    h = torch.randn(10, m.head.weight.shape[1])
    p, tok = m.short_top(h)
    lo = h @ m.head.weight[m.sv_ids].t()
    full = torch.cat([lo, (h @ m.head.weight[m.sv_bucket]).unsqueeze(1) + m.sv_prior0], 1)
    assert torch.equal(tok, m.sv_ids[lo.argmax(-1)])
    assert torch.allclose(p, full.softmax(-1)[:, :64].max(-1).values, atol=1e-5)
    assert bool((tok < 64).all()) and bool((p > 0).all()) and bool((p < 1).all())


def test_confidence_brake_slows_noise_and_spares_a_steady_direction():
    from memarch_b200.config import OptConfig
    from memarch_b200.optim.instinct import Instinct
    torch.manual_seed(0)

    def run(kind, **kw):
        p = torch.nn.Parameter(torch.randn(32, 16))
        q = torch.nn.Parameter(torch.randn(32, 16))
        opt = Instinct([p, q], OptConfig(lr=1e-2, norm="hs", scale=0.12, snr=True, **kw))
        steady = torch.randn(32, 16)
        g = torch.Generator().manual_seed(1)
        fs = []
        for _ in range(60):
            opt.update(p, steady + 0.05 * torch.randn(32, 16, generator=g))        # the same direction every step
            opt.update(q, torch.randn(32, 16, generator=g))                        # pure noise
            fs.append(opt.snr_f.clone())
        return opt, torch.stack(fs)
    opt, f = run("plain")
    assert f[-10:, 0].min() > 0.9 and f[-10:, 1].max() < 0.4
    b = opt.beta
    assert abs(float(f[-20:, 1].mean()) - ((1 - b) / (1 + b)) ** 0.5) < 0.1           # noise level of the ratio
    opt.update(opt.plist[0], torch.zeros(32, 16))                                     # idle tensor: state untouched
    assert float(opt.snr_f[0]) == 1.0
    _, f = run("dz", snr_dz=True, snr_horizon=50.0)
    assert f[-10:, 0].min() == 1.0 and f[-10:, 1].max() < 0.9
    # the brake scales the step, not its direction
    torch.manual_seed(0)
    w0, g0 = torch.randn(8, 8), torch.randn(8, 8)
    outs = []
    for snr in (False, True):
        p = torch.nn.Parameter(w0.clone())
        o = Instinct([p], OptConfig(lr=1e-2, norm="hs", scale=0.12, snr=snr, snr_ref=4.0))
        o.update(p, g0.clone())
        outs.append(p.detach() - w0)
    cos = torch.nn.functional.cosine_similarity(outs[0].flatten(), outs[1].flatten(), dim=0)
    assert cos > 0.9999 and outs[1].norm() < 0.5 * outs[0].norm()
    sd = o.state_dict()
    assert "snr_v" in sd and "snr_f" in sd


def test_weight_tree_round_trip_through_npz(tmp_path):
    from memarch_b200.build import build
    from memarch_b200.train import convert
    torch.manual_seed(0)
    m = build("tiny", 512)
    sd = m.state_dict()
    tree, beside = convert.to_tree(sd)
    L = len([k for k in sd if k.startswith("heavy.") and k.endswith(".up")])
    assert tree["heavy"]["up"].shape == (L,) + tuple(sd["heavy.0.up"].shape) and set(tree["heavy"]) == set(convert.HEAVY)
    assert len(tree["light_a"]) >= 1 and set(tree["light_a"][0]) == set(convert.BLOCK_KEYS) and "tau" in beside
    flat = convert.from_tree(tree, beside)
    assert all(np.array_equal(v, sd[k].float().numpy()) for k, v in flat.items())
    params = {k for k, _ in m.named_parameters()}
    assert params <= set(flat), sorted(params - set(flat))                  # every trained weight is in the tree
    convert.save_npz(str(tmp_path / "w.npz"), tree, beside, step=7)
    tree2, beside2, step = convert.load_npz(str(tmp_path / "w.npz"))
    assert step == 7
    flat2 = convert.from_tree(tree2, beside2)
    assert set(flat2) == set(flat) and all(np.array_equal(flat2[k], flat[k]) for k in flat)
    torch.manual_seed(1)
    m2 = build("tiny", 512)
    left = convert.load_into(m2, tree2, beside2)
    assert all(torch.equal(m2.state_dict()[k], sd[k]) for k in flat) and not (set(left) & params)
    x = torch.randint(0, 512, (2, 64))
    m.eval(); m2.eval()
    with torch.no_grad():
        a, b = m(x)[0], m2(x)[0]
    a, b = (a[0] if isinstance(a, (tuple, list)) else a), (b[0] if isinstance(b, (tuple, list)) else b)
    assert torch.equal(a, b)
    grads = {"emb.weight": torch.ones(512, 4), "heavy.0.up": torch.zeros(2, 3, 4), "heavy.1.up": torch.ones(2, 3, 4)}
    gt, _ = convert.to_tree(grads)                                           # partial dicts convert too
    assert gt["heavy"]["up"].shape == (2, 2, 3, 4) and set(gt["heavy"]) == {"up"}


def test_three_word_table_skip_tables_and_phrase_units(tmp_path):
    """The remaining phrase builders: three-word context table and draft-ahead tables load into the model and feed its
    input; the phrase vocabulary rewrites a corpus reversibly; the slice report accounts for the whole gap."""
    import numpy as np
    from memarch_b200.build import build
    from memarch_b200.data import phrasebook
    from memarch_b200.data.synth import MarkovCorpus
    vocab, phr_v, d = 512, 500, 256
    toks = MarkovCorpus(vocab=phr_v, n_succ=8, seed=0).stream(40_000, text_len=256, seed=1)
    paths = phrasebook.build_all(toks, d, str(tmp_path), vocab=phr_v, phrase_k=1024, quad_k=512, skip=True)
    quad, skip = torch.load(paths["quad"]), torch.load(paths["skip"])
    assert quad["keys"].shape == (512,) and quad["vec"].shape == (512, d)
    assert bool((quad["keys"][1:] > quad["keys"][:-1]).all())
    # a stored key is the three words as base-V digits, and that triple occurs in the corpus
    k0 = int(quad["keys"][100])
    w = [k0 // phr_v ** 2, (k0 // phr_v) % phr_v, k0 % phr_v]
    a = np.asarray(toks, dtype=np.int64)
    assert ((a[:-2] == w[0]) & (a[1:-1] == w[1]) & (a[2:] == w[2])).any()
    assert sorted(skip) == [2, 3, 4] and all(skip[o].shape == (phr_v, d) for o in skip)
    np.save(tmp_path / "token_counts.npy", phrasebook.token_counts(toks, vocab))
    env = {"PHRASE_INIT": paths["bigram"], "PHRASE3": paths["trigram"], "PHRASE4": paths["quad"], "SKIP": paths["skip"],
           "PHR_V": str(phr_v), "VOCAB": str(vocab), "NO_MEM": "1"}
    m = build("Fv2s", vocab, env=env)
    assert hasattr(m, "phr4") and hasattr(m, "skip")
    x = torch.tensor(a[:2 * 65].reshape(2, 65))
    out, cost = m(x[:, :-1])
    loss = m.train_loss(out, x[:, 1:], True)
    loss.backward()
    assert torch.isfinite(loss) and m.phr4.weight.grad is not None

    # phrase vocabulary: every unit expands back to the original words
    eot = phr_v - 1
    new, units = phrasebook.phrase_units(a[:20_000], 200, vocab=phr_v, eot=eot)
    assert units.shape == (200, 4) and len(new) < 20_000
    back = []
    for t in new.astype(np.int64):
        back += [int(t)] if t < phr_v else [int(u) for u in units[t - phr_v] if u >= 0]
    assert back == a[:20_000].tolist()
    assert not (units == eot).any()                                  # no unit crosses a document end

    # slice report: the shares of the gap sum to one inside every slice group
    g = np.random.default_rng(0)
    x1, y1 = a[:4096], a[1:4097]
    ours, theirs = g.random(4096) + 3.0, g.random(4096) + 2.8
    rep = phrasebook.slice_report(ours, theirs, x1, y1, phrasebook.token_counts(toks, vocab), torch.load(paths["bigram"]), T=1024)
    assert len(rep) == 4
    for rows in rep.values():
        assert abs(sum(r[5] for r in rows) - 1.0) < 1e-9 and abs(sum(r[1] for r in rows) - 1.0) < 1e-9


def test_dropless_moe_keeps_every_token():
    """MOE_GMM: with a place for every anchor in every expert nothing is dropped and the layer equals the capacity
    form at a capacity large enough to hold everything; the default capacity does drop on a skewed router."""
    from memarch_b200.models.moe import AnchorMoE
    torch.manual_seed(0)
    kw = dict(E=4, k_avg=2, k_max=4, budget=False, act="relu2")
    a, b = AnchorMoE(32, dropless=True, **kw), AnchorMoE(32, **kw)
    b.load_state_dict(a.state_dict())
    with torch.no_grad():                                     # a skewed router: most tokens want expert 0
        a.router.weight[0] += 2.0
        b.router.weight[0] += 2.0
    a.train(); b.train()
    x = torch.randn(2, 40, 32) + 0.5                           # positive mean: the raised router row wins almost everywhere
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya = a(xa)
    assert a.capacity(80) == 80 and float(a.dropped) == 0.0
    yb = b(xb)
    assert float(b.dropped) > 0                                # the capacity form loses tokens here
    b.fill = 10.0                                              # room for everything
    yb = b(xb)
    assert float(b.dropped) == 0.0
    assert torch.allclose(ya, yb, atol=1e-5)
    go = torch.randn_like(ya)
    ya.backward(go); yb.backward(go)
    assert torch.allclose(xa.grad, xb.grad, atol=1e-5) and torch.allclose(a.up.grad, b.up.grad, atol=1e-5)
    from memarch_b200.config import model_from_env, ModelConfig
    assert model_from_env(ModelConfig(vocab=64), {"MOE_GMM": "1"}).moe_dropless


def test_tether_inside_the_main_model():
    from memarch_b200 import build
    torch.manual_seed(0)
    env = {"NO_MEM": "1", "MOE_ACT": "relu2", "ROPE_MEM": "1", "ROPE_WIN": "8", "ROPE_SPAN_CAP": "12", "ROPE_LINKS": "3",
           "ROPE_K": "2", "ROPE_HIER_G": "4", "ROPE_HIER_BM": "16", "ROPE_CHUNK": "32", "ROPE_TAU0": "5.5",
           "ROPE_DOC_EOS": "7", "ROPE_QFRAC": "0.6", "ROPE_KEY_DIAG": "1", "REMIND_USE_W": "0.5", "REMIND_W": "1.0",
           "REMIND_N": "4", "REMIND_TOK0": "100"}
    m = build("tiny", 256, env=env).train()
    assert m.cfg.rope_mem and m.cfg.no_mem and "rope_tau" in m.state_dict() and "rope_qtau" in m.state_dict()
    xy = torch.randint(0, 256, (2, 97))
    x, y = xy[:, :-1], xy[:, 1:]
    tau0 = float(m.rope_tau)
    out, cost = m(x)
    assert float(m.rope_tau) != tau0                                       # the threshold follows the surprise
    for k in ("rope_anchors", "rope_share", "rope_qfrac_real", "rope_key_link"):
        assert k in m.stats and math.isfinite(float(m.stats[k])), k
    assert 0 < float(m.stats["rope_anchors"]) <= m.cfg.cap + 1e-6 and 0 < float(m.stats["rope_qfrac_real"]) < 1
    rem = torch.zeros(2, 96, dtype=torch.int8)
    rem[:, 60:68:2] = 1
    loss = m.train_loss(out, y, True, extra={"rem": rem})
    plain = m.train_loss(out, y, True)
    use = float(m.stats["remind_rope_share"])
    assert 0 <= use <= 1
    loss.backward()
    g = m.light_b[0].qkv.weight.grad
    assert g is not None and torch.isfinite(g).all() and g.abs().sum() > 0
    # the local window alone (tether closed for every word) differs from the tethered read
    m.eval()
    with torch.no_grad():
        a, _ = m(x)
        frozen = float(m.rope_tau)
        m.rope_qtau.fill_(1e9)
        b, _ = m(x)
    assert float(m.rope_tau) == frozen and not torch.allclose(a[0], b[0])
    # only the first layers tethered, the choice of anchors shared
    m2 = build("tiny", 256, env=dict(env, ROPE_LAYERS="1", ROPE_SHARE_ROUTE="1", ROPE_QFRAC="1.0")).train()
    o2, _ = m2(x)
    assert hasattr(m2.light_b[0], "tether_out") and torch.isfinite(o2[0]).all()
    if len(m2.light_b) > 1:
        assert not hasattr(m2.light_b[1], "tether_out")


def test_hoop_inside_the_main_model():
    from memarch_b200 import build
    from memarch_b200.models.fishki import Uroboros
    torch.manual_seed(0)
    env = {"NO_MEM": "1", "MOE_ACT": "relu2", "UROBOROS": "1", "UROBOROS_BUDGET": "0.25", "UROBOROS_W": "0.2"}
    m = build("tiny", 256, env=env).train()
    assert isinstance(m.hoop, Uroboros) and m.hoop_budget == 0.25
    xy = torch.randint(0, 256, (2, 65))
    x, y = xy[:, :-1], xy[:, 1:]
    tau0 = float(m.tau)
    out, _ = m(x)
    pred, idx = m._hoop
    assert idx.shape == (2, 16) and bool((idx[:, 0] == 0).all()) and float(m.tau) == tau0     # a budget, no threshold
    assert abs(float(m.stats["anchors"]) - 0.25) < 1e-6
    top = pred.detach().clone()
    top[:, 0] = 1e9
    assert torch.equal(idx, top.topk(16, -1).indices.sort(-1).values)                         # the words it fears most
    loss = m.train_loss(out, y, True)
    lo = m._logits(out[0]).float()
    nll = torch.nn.functional.cross_entropy(lo.reshape(-1, 256), y.reshape(-1), reduction="none").view_as(y)
    for k in ("uroboros_eaten", "uroboros_corr", "uroboros_nll_sel", "uroboros_nll_skip"):
        assert k in m.stats
    m._hoop = None
    base = m.train_loss(out, y, True)                                                         # same terms without the head's
    want = 0.2 * (pred.clamp(0, 20) - nll.clamp(0, 20)).pow(2).mean()
    assert abs(float(loss - base) - float(want)) < 1e-4
    m._hoop = (pred, idx)
    m.train_loss(out, y, True).backward()
    assert m.hoop.l1.weight.grad.abs().sum() > 0 and m.head.weight.grad.abs().sum() > 0
    # causal choice by a threshold (evaluation), and the head before the memory point
    m2 = build("tiny", 256, env=dict(env, UROBOROS_THR="2.5", UROBOROS_AT="light_a")).eval()
    with torch.no_grad():
        o2, _ = m2(x)
    p2, i2 = m2._hoop
    assert i2.shape == (2, 64) and torch.isfinite(o2[0]).all()
    assert abs(float(m2.stats["anchors"]) - float(((p2 > 2.5) | (torch.arange(64) == 0)).float().mean())) < 1e-6


def test_layer_pool_inside_the_main_model():
    from memarch_b200 import build
    torch.manual_seed(0)
    env = {"NO_MEM": "1", "FISH_N": "8", "FISH_HF": "64", "FISH_KINDS": "3", "FISH_POOL": "4", "FISH_C": "2"}
    m = build("tiny", 256, env=env).train()
    assert len(m.heavy) == 0 and not m.moe and m.fish.up.shape[0] == 8 and len(m.fish.sets) == 3
    xy = torch.randint(0, 256, (3, 49))
    x, y = xy[:, :-1], xy[:, 1:]
    order = m.fish.sets[1][:2]
    prep = {"kind": torch.full((3, 1), 1), "fish": torch.tensor([order] * 3)}
    out, _ = m(x, prep)
    loss = m.train_loss(out, y, True)
    assert "fish_router_acc" in m.stats and m._fish_aux is not None
    loss.backward()
    used = {i for i in range(8) if m.fish.up.grad[i].abs().sum() > 0}
    assert used == set(order) and m.fish.router.weight.grad.abs().sum() > 0                  # only the step's layers work
    base = float(loss) - 0.1 * float(m._fish_aux)
    m._fish_aux = None
    assert abs(float(m.train_loss(out, y, True)) - base) < 1e-5
    # finished model: the router sends each row through the whole set of its kind
    m.eval()
    with torch.no_grad():
        a, _ = m(x)
    assert torch.isfinite(a[0]).all()
    m2 = build("tiny", 256, env=dict(env, FISH_EVAL="1", FISH_EVAL_C="2")).eval()
    m2.load_state_dict(m.state_dict())
    with torch.no_grad():
        b, _ = m2(x, prep)
    assert torch.isfinite(b[0]).all() and not torch.allclose(a[0], b[0])                     # a subset of the set


def test_heavy_layers_on_all_words():
    from memarch_b200 import build
    torch.manual_seed(0)
    env = {"NO_MEM": "1", "MOE_ACT": "relu2"}
    base = build("tiny", 256, env=env).train()
    rot = build("tiny", 256, env=dict(env, HEAVY_ROTATE="1", HEAVY_FULL_EVERY="2")).train()
    full = build("tiny", 256, env=dict(env, HEAVY_ALL="1")).train()
    rot.load_state_dict(base.state_dict())
    full.load_state_dict(base.state_dict())
    L = len(base.heavy)
    x = torch.randint(0, 256, (2, 64))
    # the rotation: every second step one layer, in turn
    seen = []
    for step in range(2 * L + 2):
        rot.before_step(step)
        seen.append(rot._hfull)
    assert seen[:4] == [0, -1, 1 % L, -1] and seen[2 * L] == 0
    for m in (base, rot, full):
        m.tau.fill_(5.0)
    rot.before_step(1)                                                     # no full layer in this step: the plain model
    a, _ = base(x)
    b, _ = rot(x)
    assert torch.allclose(a[0], b[0], atol=1e-5)
    rot.tau.fill_(5.0)
    rot.before_step(0)                                                     # layer 0 on all words
    c, _ = rot(x)
    assert not torch.allclose(a[0], c[0], atol=1e-4)
    rot.tau.fill_(5.0)
    d, _ = rot(x, {"hfull": torch.full((2, 1), L - 1)})                    # the step's data may name the layer
    assert not torch.allclose(c[0], d[0], atol=1e-4) or L == 1
    e, _ = full(x)
    assert torch.isfinite(e[0]).all() and not torch.allclose(a[0], e[0], atol=1e-4)
    # words that are no anchors change only through a full layer
    e[0].square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in full.heavy[0].parameters() if p.requires_grad)
    rot.eval()
    with torch.no_grad():
        base.eval()
        f, _ = rot(x)
        g, _ = base(x)
    assert torch.allclose(f[0], g[0], atol=1e-5)                           # evaluation: anchors only
    # the pass itself against a hand-made one: anchors in, layer k over all words with every place real, anchors out
    torch.manual_seed(3)
    base.train()
    B, T, d = 2, 64, base.cfg.d
    h = torch.randn(B, T, d)
    s_ = torch.rand(B, T) * 6
    idx = torch.stack([torch.randperm(T)[:16].sort().values for _ in range(B)])
    valid = torch.rand(B, 16) < 0.8
    is_anchor = torch.zeros(B, T, dtype=torch.bool).scatter(1, idx, valid)
    with torch.no_grad():
        plain, _ = base.heavy_pass(h, idx, valid, s_)
        assert torch.equal(plain[~is_anchor], h[~is_anchor])               # without a full layer only anchors change
        k = L - 1
        got, a_got = base.heavy_pass(h, idx, valid, s_, full=k)
        assert not torch.equal(got[~is_anchor], h[~is_anchor])             # a full layer changes the other words too
        gi = idx[..., None].expand(-1, -1, d)
        sa = torch.where(valid, s_.gather(1, idx).clamp(0, 50), torch.full_like(s_[:, :16], -1.0))
        a = h.gather(1, gi)
        hh = h
        for li, blk in enumerate(base.heavy):
            if li == k:
                hh = hh.scatter(1, gi, torch.where(valid[..., None], a, hh.gather(1, gi)))
                keep, blk.fill = blk.fill, 1.0
                hh = blk(hh, s_.clamp(0, 50))
                blk.fill = keep
                a = hh.gather(1, gi)
            else:
                a = blk(a, sa)
        want = hh.scatter(1, gi, torch.where(valid[..., None], a, hh.gather(1, gi)))
        assert torch.allclose(got, want, atol=1e-5)
        every, _ = base.heavy_pass(h, idx, valid, s_, full=-1)            # all layers full = the layers in turn on all words
        hh = h
        for blk in base.heavy:
            keep, blk.fill = blk.fill, 1.0
            hh = blk(hh, s_.clamp(0, 50))
            blk.fill = keep
        assert torch.allclose(every, hh, atol=1e-5)


def test_final_norm_variants_and_trunk_guard_in_the_model():
    from memarch_b200 import build
    torch.manual_seed(0)
    env = {"NO_MEM": "1", "MOE_ACT": "relu2"}
    base = build("tiny", 256, env=env).train()
    x = torch.randint(0, 256, (2, 64))
    y = torch.randint(0, 256, (2, 64))
    a, _ = base(x)
    dp = build("tiny", 256, env=dict(env, NORM_DUMP_PROJ="1")).train()
    dp.load_state_dict(base.state_dict())
    dp.tau.fill_(float(5.0)); base.tau.fill_(5.0)
    u = torch.randn(dp.cfg.d)
    dp.stream_u = u
    b, _ = dp(x)
    uh = u / u.norm()
    w = dp.norm.weight.detach().float()
    assert ((b[0].float() / w) @ uh).abs().max() < 1e-4                    # nothing along the common direction
    cap = build("tiny", 256, env=dict(env, SAFE_NORM_RATIO="0.05", SAFE_NORM_T0="8")).train()
    cap.load_state_dict(base.state_dict())
    c_, _ = cap(x)
    a2, _ = base(x)
    assert torch.equal(c_[0][:, :8], a2[0][:, :8]) and not torch.equal(c_[0][:, 8:], a2[0][:, 8:])
    g = build("tiny", 256, env=dict(env, HN_GUARD_W="2.0", HN_GUARD_MEAN="0.01", HN_GUARD_LEN="1000")).train()
    g.load_state_dict(base.state_dict())
    o, _ = g(x)
    with_guard = g.train_loss(o, y, True)
    o2, _ = base(x)
    plain = base.train_loss(o2, y, True)
    assert float(with_guard) > float(plain) and float(g.stats["hn_mean"]) > 0.01 and "hn_len" in g.stats
    quiet = build("tiny", 256, env=dict(env, HN_GUARD_W="2.0", HN_GUARD_MEAN="1e6", HN_GUARD_LEN="1e6")).train()
    quiet.load_state_dict(base.state_dict())
    o3, _ = quiet(x)
    assert abs(float(quiet.train_loss(o3, y, True)) - float(base.train_loss(base(x)[0], y, True))) < 1e-3


def test_instinct_on_words_terms():
    from memarch_b200 import build
    torch.manual_seed(0)
    env = {"NO_MEM": "1", "MOE_ACT": "relu2"}
    base = build("tiny", 256, env=env).train()
    x, y = torch.randint(0, 256, (2, 48)), torch.randint(0, 256, (2, 48))
    o, _ = base(x)
    plain = float(base.train_loss(o, y, True))
    lsm = base._logits(o[0]).float().log_softmax(-1).detach()
    lp = lsm.gather(-1, y[..., None])[..., 0]
    ok = lp.exp() >= 0.02
    lpt, top = lsm.max(-1)

    def model(**kw):
        m = build("tiny", 256, env=dict(env, INST_WORD="1", IW_OK="0.02", **kw)).train()
        m.load_state_dict(base.state_dict())
        m.tau.fill_(float(5.0))
        return m
    base.tau.fill_(5.0)
    # base form: smeared distributions are pushed up to the target, a confident wrong leader is pressed down
    m = model(IW_SPREAD="0.5", IW_TARGET="0.3", IW_CW="0.01", IW_SPREAD_W="0.2", IW_CW_W="0.1")
    o1, _ = m(x)
    total = m.train_loss(o1, y, True)
    spread = ~ok & (lpt.exp() < 0.5)
    cw = ~ok & (lpt.exp() > 0.01) & (top != y)
    l_sp = ((math.log(0.3) - lp).clamp(min=0) * spread).sum()
    l_cw = ((-torch.log1p(-lpt.exp().clamp(max=1 - 1e-6)) + math.log1p(-0.01)).clamp(min=0) * cw).sum()
    want = (0.2 * l_sp + 0.1 * l_cw) / y.numel()
    assert abs(float(total) - plain - float(want)) < 1e-4 and float(want) > 0
    assert abs(float(m.stats["iw_ok_frac"]) - float(ok.float().mean())) < 1e-6
    assert abs(float(m.stats["iw_spread_frac"]) - float(spread.float().mean())) < 1e-6
    total.backward()
    assert torch.isfinite(m.head.weight.grad).all()
    # rewritten answer: the gradient on the logits touches the right word and its k competitors only, and sums to zero
    for kw in (dict(IW_REWRITE="1", IW_K="3", IW_DELTA="0.05"), dict(IW_RANDOM="1", IW_DELTA="0.05")):
        m = model(**kw)
        hn = o[0].detach().clone().requires_grad_(True)
        lo_holder = {}
        real = m._logits

        def spy(h_):
            lo_holder["lo"] = real(h_)
            lo_holder["lo"].retain_grad()
            return lo_holder["lo"]
        m._logits = spy
        part = m._iw_part(hn, y, 1.0, 0)
        part[0].backward()
        g = lo_holder["lo"].grad
        assert g.sum(-1).abs().max() < 1e-6
        n_touched = (g.abs() > 1e-7).sum(-1)
        assert int(n_touched.max()) <= (4 if "IW_REWRITE" in kw else 2)
        acted = n_touched > 0
        assert bool((g.gather(-1, y[..., None])[..., 0][acted] < 0).all())      # the right word goes up
        assert abs(float(part[4]) - float(acted.sum())) < 1e-6 and float(part[0]) != 0


def test_small_switches_of_the_light_blocks_and_inputs():
    from memarch_b200 import build
    from memarch_b200.ops import ref
    cos, sin = ref.rope_angles(16, 32, "cpu", pcut=40.0)
    cos0, _ = ref.rope_angles(16, 32, "cpu")
    inv = 1.0 / 10000.0 ** (torch.arange(0, 32, 2).float() / 32)
    rot = 2 * math.pi / inv <= 40.0
    assert 0 < int(rot.sum()) < 16 and torch.equal(cos[:, rot], cos0[:, rot])
    assert bool((cos[:, ~rot] == 1).all()) and bool((sin[:, ~rot] == 0).all())
    torch.manual_seed(0)
    env = {"NO_MEM": "1", "MOE_ACT": "relu2"}
    base = build("tiny", 256, env=env).eval()
    x = torch.randint(0, 256, (2, 48))
    with torch.no_grad():
        a, _ = base(x)
        for kw in ({"ATTN_GAIN": "1.5"}, {"PREV_IN": "1"},
                   {"ROPE_MEM": "1", "ROPE_WIN": "8", "ROPE_SPAN_CAP": "12", "ROPE_K": "2", "ROPE_PCUT": "16"}):
            m = build("tiny", 256, env=dict(env, **kw)).eval()
            missing = m.load_state_dict(base.state_dict(), strict=False)
            assert set(missing.missing_keys) <= {"prev_g", "rope_tau"} and not missing.unexpected_keys
            b, _ = m(x)
            assert torch.isfinite(b[0]).all() and not torch.allclose(a[0], b[0], atol=1e-4), kw
        assert m.light_b[0].tether_pcut == 16.0 and m.light_a[0].tether_pcut == 0.0
    g = build("tiny", 256, env=dict(env, REMIND_W="1.0", REMIND_W_SYNTH="3.0", REMIND_N="4")).train()
    o, _ = g(x)
    y = torch.randint(0, 256, (2, 48))
    rem = torch.zeros(2, 48, dtype=torch.int8)
    rem[:, 30:38:2] = 1
    plain = float(g.train_loss(o, y, True))
    text = float(g.train_loss(o, y, True, extra={"rem": rem, "synth": False})) - plain
    synth = float(g.train_loss(o, y, True, extra={"rem": rem, "synth": True})) - plain
    assert abs(synth - 3.0 * text) < 1e-4 and text > 0


def test_one_probe_bucket_table_for_phrase_keys():
    import numpy as np
    from memarch_b200.models.memarch import _BUCKET_MUL, bucket_table
    rng = np.random.default_rng(0)
    V = 50304
    for K in (0, 1, 700, 40000):
        keys = np.unique(rng.integers(0, V * V, K).astype(np.int64))
        rows, numbers, mask = bucket_table(keys)
        assert rows.shape == numbers.shape and rows.shape[1] == 8 and rows.shape[0] == mask + 1
        assert int((rows >= 0).sum()) == len(keys)                            # every key sits in exactly one place
        probe = torch.from_numpy(np.concatenate([keys[:3000], rng.integers(-V, V * V, 3000)])).long()
        row = ((probe * _BUCKET_MUL) >> 40) & mask
        same = torch.from_numpy(rows)[row] == probe[..., None]
        got = torch.where(same.any(-1), (torch.from_numpy(numbers)[row] * same).sum(-1), torch.full_like(probe, len(keys)))
        kt = torch.from_numpy(keys)
        if len(keys):
            pos = torch.searchsorted(kt, probe).clamp(max=len(keys) - 1)
            want = torch.where(kt[pos] == probe, pos, torch.full_like(pos, len(keys)))
        else:
            want = torch.zeros_like(probe)
        assert torch.equal(got, want)
    rows, _, mask = bucket_table((np.arange(4000, dtype=np.int64) * 7919) ** 2, width=2)
    assert int((rows >= 0).sum()) == 4000 and mask + 1 > 4096


def test_moe_layer_statistics():
    from memarch_b200 import build
    torch.manual_seed(0)
    m = build("tiny", 256, env={"NO_MEM": "1", "MOE_ACT": "relu2", "LAYER_STATS": "1"}).train()
    quiet = build("tiny", 256, env={"NO_MEM": "1", "MOE_ACT": "relu2"}).train()
    x = torch.randint(0, 256, (2, 64))
    m(x), quiet(x)
    L = len(m.heavy)
    assert m.stats["moe_drop_l"].shape == (L,) and m.stats["moe_active_l"].shape == (L,)
    assert abs(float(m.stats["moe_drop_l"].mean()) - float(m.stats["moe_drop"])) < 1e-6
    assert 0 < float(m.stats["moe_fill"]) <= 1 and bool((m.stats["moe_active_l"] <= m.heavy[0].E).all())
    b = m.heavy[0]
    # filled share = kept (token, choice) pairs over the capacity
    assert "moe_fill" not in quiet.stats and "moe_drop_l" not in quiet.stats


def test_light_moe_dispatch_serves_first_askers_when_over_capacity():
    """FineMoE against a plain statement of the same layer: stable sort of the (token, choice) pairs by expert, the
    first `cap` of every expert served, the rest dropped."""
    import torch.nn.functional as F
    from memarch_b200.models.blocks import FineMoE
    torch.manual_seed(0)
    d, E, k = 32, 4, 2
    moe = FineMoE(d, E=E, k=k)
    with torch.no_grad():
        moe.router.weight[0] += 2.0 * torch.ones(d) / d ** 0.5            # expert 0 is everybody's favourite: it overflows
    x = torch.randn(2, 40, d) + 0.5
    y = moe(x)
    xf = x.reshape(-1, d)
    N = xf.shape[0]
    logits = xf @ moe.router.weight.T
    gate, ex = logits.topk(k, -1)
    gate = gate.softmax(-1)
    cap = int(1.25 * N * k / E) + 1
    e_flat = ex.reshape(-1)
    order = e_flat.argsort(stable=True)
    es = e_flat[order]
    start = torch.searchsorted(es, torch.arange(E))
    slot = torch.arange(N * k) - start[es]
    keep = slot < cap
    assert int((~keep).sum()) > 0                                          # the case really drops something
    tok = order // k
    want = torch.zeros(N, d)
    for j in range(N * k):
        if keep[j]:
            e, t = int(es[j]), int(tok[j])
            a = xf[t] @ moe.up[e]
            g_, u_ = a.chunk(2, -1)
            want[t] += gate.reshape(-1)[order][j] * ((F.silu(g_) * u_) @ moe.down[e])
    assert torch.allclose(y.reshape(N, d), want, atol=1e-4), float((y.reshape(N, d) - want).abs().max())
    y.sum().backward()
    assert moe.up.grad.abs().sum() > 0 and moe.router.weight.grad is not None
