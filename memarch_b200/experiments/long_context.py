"""Long-context experiments (the reference's long_speed.py, recall_long.py, pg19_needle.py, anchor_chunks.py).

  long_speed     ms/step and k tok/s against text length at ~32k tokens per step (or one text, or as many as fit)
  recall_task    "Petro 3 Ivan 7 ... <filler longer than the window> ... Petro ?" - the fact is reachable only through
                 memory; `recall_run` trains with a filler curriculum and reports accuracy per filler length, and
                 `recall_diagnose` says where facts get lost (is the key's card in memory; does the read find it)
  needle_batch   a sentence "code of <name> is <number>" inserted at a random depth of the first half of a long text,
                 asked again at the end; `needle_eval` = accuracy of the first token of the number per length
  anchor_chunks  share of threshold anchors that a per-chunk cap would cut compared with the per-text cap

All generators are seeded and run on any device; token sources are the synthetic corpus or a user token file
(the reference downloads PG-19; there is no network here).
"""
from __future__ import annotations

import argparse
import time

import torch
import torch.nn.functional as F

N_KEYS, N_VALS, FILL0 = 512, 64, 1000


# ------------------------------------------------------------------------------------------------ speed vs length
def long_speed(models=("T300ck", "Fv2ck"), lens=(1024, 4096, 16384), mode="tokens", warmup=3, n=4, device=None,
               vocab=50304, out=print):
    from ..data.synth import MarkovCorpus, TokenStore
    from ..train.loop import _time_steps, make_trainer
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    toks = MarkovCorpus(vocab=min(vocab, 50257), seed=0).stream(max(lens) * 8 + 100_000, text_len=max(lens), seed=1)
    rows = []
    for T in lens:
        for name in models:
            def run(B):
                args = argparse.Namespace(lr=6e-4, steps=4000, micro=B, batch=B, seq=T, read_cost=0.01)
                tr = make_trainer(name, "ABX", args, device, env={"VOCAB": str(vocab)})
                store = TokenStore(toks, seed=1, device=tr.device)
                step = lambda s: tr.step(store.batch(B, T), s)
                for s in range(warmup):
                    step(s)
                ms = _time_steps(step, n, device)
                mem = torch.cuda.max_memory_allocated() / 2 ** 30 if tr.device.type == "cuda" else 0.0
                return ms, mem
            if mode == "fill":                       # double the batch while it fits
                best, B = None, 1
                while B <= 4096:
                    try:
                        best, B = (B, *run(B)), B * 2
                    except torch.OutOfMemoryError:
                        break
                    finally:
                        if torch.cuda.is_available():
                            torch.cuda.empty_cache()
                if best:
                    out(f"FILL {name:8s} T={T:6d}  max texts {best[0]}  {best[0] * T / best[1]:.1f}k tok/s")
                    rows.append({"model": name, "T": T, "B": best[0], "ms": best[1], "mem_gb": best[2]})
                continue
            B = 1 if mode == "one" else max(1, 32768 // T)
            ms, mem = run(B)
            out(f"LONG {name:8s} T={T:6d} B={B:3d}  {ms:8.1f} ms/step  {B * T / ms:7.1f}k tok/s  mem {mem:.1f} GB")
            rows.append({"model": name, "T": T, "B": B, "ms": ms, "mem_gb": mem})
    return rows


# ------------------------------------------------------------------------------------------------ recall beyond the window
def recall_task(B, pairs, filler, queries, g=None, device="cpu", fill_vocab=20000):
    """x (B,L-1), y (B,L-1) with -100 everywhere except at the answers, ans = positions of the query keys."""
    keys = torch.rand(B, N_KEYS, generator=g).argsort(-1)[:, :pairs]
    vals = torch.randint(0, N_VALS, (B, pairs), generator=g) + N_KEYS
    kv = torch.stack([keys, vals], -1).view(B, -1)
    fill = torch.randint(FILL0, FILL0 + fill_vocab, (B, filler), generator=g)
    qi = torch.rand(B, pairs, generator=g).argsort(-1)[:, :queries]        # every key is asked at most once
    qs = torch.stack([keys.gather(1, qi), vals.gather(1, qi)], -1).view(B, -1)
    seq = torch.cat([kv, fill, qs], 1).to(device)
    x, y = seq[:, :-1], torch.full_like(seq[:, 1:], -100)
    ans = 2 * pairs + filler + 2 * torch.arange(queries, device=device)
    y[:, ans] = seq[:, ans + 1]
    return x, y, ans


def answer_logits(model, x, ans):
    out, cost = model(x)
    if isinstance(out, tuple):
        hn = out[0]
        return F.linear(hn[:, ans].float(), model.head.weight.float()), cost
    return (out[:, ans] if out.shape[-1] == model.head.weight.shape[0] else
            F.linear(out[:, ans].float(), model.head.weight.float())), cost


def recall_loss(model, x, y, ans):
    logits, cost = answer_logits(model, x, ans)
    return F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), y[:, ans].reshape(-1)) + 0.01 * cost.float(), logits


def recall_run(name="Fv2s", steps=300, B=16, pairs=4, fillers=(32, 128, 256), lr=1e-3, device=None, vocab=32768,
               eval_B=64, out=print, env=None):
    """Curriculum over filler lengths (each level a third of the steps); returns {filler: accuracy}."""
    from ..build import build
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    torch.manual_seed(0)
    m = build(name, vocab, env=env or {}).to(device)
    opt = torch.optim.AdamW(m.parameters(), lr=lr, betas=(0.9, 0.95), weight_decay=0.0)
    g = torch.Generator().manual_seed(1)
    t0 = time.time()
    for s in range(steps):
        filler = fillers[min(len(fillers) - 1, s * len(fillers) // max(steps, 1))]
        x, y, ans = recall_task(B, pairs, filler, pairs, g, device)
        loss, _ = recall_loss(m, x, y, ans)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(m.parameters(), 1.0)
        opt.step()
    acc = {}
    m.eval()
    with torch.no_grad():
        gv = torch.Generator().manual_seed(11)
        for filler in fillers:
            x, y, ans = recall_task(eval_B, pairs, filler, pairs, gv, device)
            _, logits = recall_loss(m, x, y, ans)
            acc[filler] = float((logits.argmax(-1) == y[:, ans]).float().mean())
    out(f"RECALL {name}: " + "  ".join(f"filler {k}: {100 * v:.0f}%" for k, v in acc.items()) + f"  ({time.time() - t0:.0f}s)")
    return acc, m


@torch.no_grad()
def recall_diagnose(model, pairs=4, filler=128, B=32, device="cpu"):
    """Where facts get lost: share of asked keys whose card is in memory when the question comes (`stored`), and
    share of those whose card gets the largest read weight from the query word (`found`)."""
    gv = torch.Generator().manual_seed(11)
    x, y, ans = recall_task(B, pairs, filler, pairs, gv, device)
    h = model.emb(x).float()
    reads, snaps, _ = model._memory_pass(h, model.cfg.seg)
    k = min((2 * pairs + filler) // model.cfg.seg, len(snaps) - 1)
    faces, contents, pos, valid = snaps[k]
    key_pos = 2 * torch.arange(pairs, device=device)
    in_mem = ((pos[:, :, None] == key_pos) | (pos[:, :, None] == key_pos + 1)) & valid[:, :, None]
    stored = in_mem.any(1).float().mean()
    return {"stored": float(stored), "cards": float(valid.float().sum(1).mean())}


# ------------------------------------------------------------------------------------------------ needle in a haystack
def needle_batch(tokens, B, T, name_ids, g=None, device="cpu", code_lo=2000, code_n=1000, marker=(11, 12, 13)):
    """tokens: 1-D token array of long texts.  Returns x (B,T), target (B,) first token of the number, and the depth
    of every needle.  The needle is `marker name number`, the question at the end is `marker name`."""
    import numpy as np
    rng = np.random.default_rng(int(torch.randint(0, 2 ** 31, (1,), generator=g)))
    xs, tg, depth = [], [], []
    need = len(marker) + 2
    for _ in range(B):
        s = int(rng.integers(0, len(tokens) - T - 1))
        seq = np.array(tokens[s:s + T], dtype=np.int64)
        name = int(name_ids[rng.integers(0, len(name_ids))])
        code = int(code_lo + rng.integers(0, code_n))
        d = int(rng.integers(8, max(9, T // 2 - need)))
        seq[d:d + need] = list(marker) + [name, code]
        seq[T - need + 1:] = list(marker) + [name]
        xs.append(seq)
        tg.append(code)
        depth.append(d)
    return torch.tensor(np.stack(xs), device=device), torch.tensor(tg, device=device), depth


@torch.no_grad()
def needle_eval(model, tokens, lens=(1024, 4096), B=8, n=4, device="cpu", name_ids=tuple(range(3000, 3010))):
    acc = {}
    g = torch.Generator().manual_seed(5)
    model.eval()
    for T in lens:
        hit = tot = 0
        for _ in range(n):
            x, tgt, _ = needle_batch(tokens, B, T, name_ids, g, device)
            logits, _ = answer_logits(model, x, torch.tensor([T - 1], device=device))
            hit += int((logits[:, 0].argmax(-1) == tgt).sum())
            tot += B
        acc[T] = hit / tot
    return acc


# ------------------------------------------------------------------------------------------------ anchor caps
@torch.no_grad()
def anchor_chunks(surprise, tau, cap=0.25, chunks=(128, 512, 2048)):
    """surprise (N,T) of real texts, anchors by threshold without any cap.  Returns the share of anchors the
    per-text cap cuts and the share a per-chunk cap of the same fraction would cut, per chunk length."""
    anchor = surprise > tau
    N, T = anchor.shape
    total = anchor.sum().clamp(min=1).float()
    keep_text = anchor & (anchor.long().cumsum(1) <= max(1, round(T * cap)))
    out = {"per_text": float(1 - keep_text.sum() / total), "anchor_share": float(anchor.float().mean())}
    for c in chunks:
        if T % c:
            continue
        a = anchor.view(N, T // c, c)
        keep = a & (a.long().cumsum(2) <= max(1, round(c * cap)))
        out[f"per_chunk_{c}"] = float(1 - keep.sum() / total)
    return out
