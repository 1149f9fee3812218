"""Phrasebook artefacts built from a token corpus, in the file formats the reference's model loads.

  * `bigram_init`  - "born with ready phrases": PPMI of (word -> next word) pairs, rank-d SVD -> input table E,
                     output table H, log-frequency bias `logp_next`, and per-previous-word `lse` of the pair
                     forecast used for phrase surprise (tools/phr/bigram_init.py:10-24, lse.py:4-9).
  * `phrase_table` - top-K (previous, current) contexts -> ridge projection of their PPMI with the next word onto
                     H, a vector to add to the input (tools/phr/trigram_init.py:9-28).
  * `lock_trust`   - hit-rate of the 1/2/3-word locks by rarity bucket of the current word -> initial trust
                     (tools/phr/lock_trust.py:15-31).
  * `token_counts` - unigram counts.
  * `prior_top`    - top-32 continuations per word (tools/phr/prior_top.py), `entropy` per word (ent.py).
`build_all(tokens, d, out_dir)` writes bigram.pt, trigram.pt, lock_trust.pt, token_counts.npy.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from ..ops import ref


def token_counts(a, vocab):
    return np.bincount(np.asarray(a, dtype=np.int64), minlength=vocab)[:vocab]


def bigram_init(a, d, vocab=50257, phrase_c=0.05, niter=4, seed=0, with_ent=False, device="cpu"):
    a = np.asarray(a, dtype=np.int64)
    V = vocab
    pair = a[:-1] * V + a[1:]
    u, c = np.unique(pair, return_counts=True)
    prev, nxt = u // V, u % V
    cp = np.bincount(a[:-1], minlength=V).astype(np.float64)
    cn = np.bincount(a[1:], minlength=V).astype(np.float64)
    pmi = np.log(c * len(pair) / (cp[prev] * cn[nxt]))
    keep = (pmi > 0) & (c >= 2)
    idx = torch.tensor(np.stack([prev[keep], nxt[keep]]))
    M = torch.sparse_coo_tensor(idx, torch.tensor(pmi[keep], dtype=torch.float32), (V, V)).coalesce().to(device)
    torch.manual_seed(seed)
    U, S, Vt = torch.svd_lowrank(M, q=d, niter=niter)
    E, H = U * S.sqrt(), Vt * S.sqrt()
    logp = torch.tensor(np.log((cn + 1) / cn.sum()), dtype=torch.float32, device=device)
    En = E / E.pow(2).mean(1, keepdim=True).sqrt().clamp(min=1e-6)
    lse = torch.cat([torch.logsumexp(phrase_c * En[i:i + 2048] @ H.T + logp, -1) for i in range(0, V, 2048)])
    out = {"emb": E, "head": H, "S": S, "logp_next": logp, "lse": lse}
    if with_ent:
        ent = []
        for i in range(0, V, 2048):
            lp = torch.log_softmax(phrase_c * En[i:i + 2048] @ H.T + logp, -1)
            ent.append(-(lp.exp() * lp).sum(-1))
        out["ent"] = torch.cat(ent)
    return out


def phrase_table(a, H, K, vocab=50257, device="cpu"):
    a = np.asarray(a, dtype=np.int64)
    V = vocab
    ctx = a[:-2] * V + a[1:-1]
    uc, cc = np.unique(ctx, return_counts=True)
    K = min(K, len(uc))
    top = uc[np.argsort(-cc, kind="stable")[:K]]
    keys = np.sort(top)
    pos = np.searchsorted(keys, ctx)
    hit = (pos < K) & (keys[np.minimum(pos, K - 1)] == ctx)
    row, nxt = pos[hit], a[2:][hit]
    trip = row * V + nxt
    ut, ct = np.unique(trip, return_counts=True)
    r, n = ut // V, ut % V
    crow = np.bincount(row, minlength=K).astype(np.float64)
    cn = np.bincount(a[2:], minlength=V).astype(np.float64)
    pmi = np.log(ct * len(a) / (crow[r] * cn[n]))
    keep = (pmi > 0) & (ct >= 2)
    Hd = H.to(device).double()
    M = torch.sparse_coo_tensor(torch.tensor(np.stack([r[keep], n[keep]])), torch.tensor(pmi[keep]), (K, V)).coalesce().to(device)
    P = torch.linalg.solve(Hd.T @ Hd + 1e-3 * torch.eye(Hd.shape[1], dtype=Hd.dtype, device=device), (M @ Hd).T).T
    return {"keys": torch.tensor(keys), "vec": P.float()}


def lock_trust(a, vocab, counts, T=1024, max_tokens=4_000_000, device="cpu"):
    a = np.asarray(a[:max_tokens], dtype=np.int64)
    bucket = torch.tensor(np.clip(np.floor(np.log10(np.asarray(counts) + 1)), 0, 6).astype(np.int64), device=device)
    n = len(a) // (T + 1) * (T + 1)
    x = torch.tensor(a[:n], device=device).view(-1, T + 1)
    inp, tgt = x[:, :-1], x[:, 1:]
    cand, on, bk, _ = ref.find_locks(inp, vocab, 3, None)
    bk = bucket[inp.clamp(max=bucket.numel() - 1)]
    W = np.zeros((3, 7), dtype=np.float32)
    for k in range(3):
        ok = on[..., k]
        hit = (cand[..., k] == tgt) & ok
        for b in range(7):
            m = ok & (bk == b)
            cnt = int(m.sum())
            p = float(hit[m].sum()) / max(cnt, 1)
            W[k, b] = max(0.0, np.log(max(p, 1e-4) / np.exp(-4.5))) if cnt > 50 else 1.0
    return torch.tensor(W)


def prior_top(ph, k=32, phrase_c=0.05):
    E, H, lp = ph["emb"], ph["head"], ph["logp_next"]
    En = E / E.pow(2).mean(1, keepdim=True).sqrt().clamp(min=1e-6)
    idx, val = [], []
    for i in range(0, E.shape[0], 2048):
        lo = torch.log_softmax(phrase_c * En[i:i + 2048] @ H.T + lp, -1)
        v, j = lo.topk(k, -1)
        idx.append(j)
        val.append(v)
    return torch.cat(idx), torch.cat(val)


def build_all(tokens, d, out_dir, vocab=50257, phrase_k=262144, seed=0):
    """Write every artefact of the published recipe under `out_dir`; returns the paths."""
    os.makedirs(out_dir, exist_ok=True)
    paths = {k: os.path.join(out_dir, v) for k, v in
             dict(bigram="bigram.pt", trigram="trigram.pt", lock="lock_trust.pt", counts="token_counts.npy").items()}
    cnt = token_counts(tokens, vocab)
    np.save(paths["counts"], cnt)
    ph = bigram_init(tokens, d, vocab, seed=seed)
    torch.save(ph, paths["bigram"])
    torch.save(phrase_table(tokens, ph["head"], phrase_k, vocab), paths["trigram"])
    torch.save(lock_trust(tokens, vocab, cnt), paths["lock"])
    return paths


def write_corpus(out_dir, tokens=8_000_000, d=256, vocab=50304, phr_v=None, phrase_k=262144, shards=4, seed=0):
    """Seeded synthetic corpus as `tokens.npy` + shards `synthetic/shard_<i>.u32.npy` (loader layout) + every
    phrasebook artefact, and `env.json` with the environment switches that point the model at them."""
    import json
    from .loader import write_shard
    from .synth import MarkovCorpus
    phr_v = phr_v or min(vocab - 1, 50257)                 # the document separator is one id above: it must fit too
    os.makedirs(out_dir, exist_ok=True)
    mc = MarkovCorpus(vocab=phr_v, seed=seed)
    toks = mc.stream(tokens, text_len=2048, seed=seed + 1)
    np.save(os.path.join(out_dir, "tokens.npy"), toks.astype(np.int32))
    eos = phr_v                                            # one id above the corpus vocabulary ends a document
    docs = [toks[i:i + 2048] for i in range(0, len(toks) - 2047, 2048)]
    per = max(1, len(docs) // shards)
    for s in range(shards):
        write_shard(out_dir, "synthetic", f"shard_{s:03d}", docs[s * per:(s + 1) * per], eos)
    paths = build_all(toks, d, out_dir, vocab=phr_v, phrase_k=phrase_k, seed=seed)
    cnt = token_counts(toks, vocab)
    np.save(paths["counts"], cnt)
    env = {"PHRASE_INIT": paths["bigram"], "PHRASE3": paths["trigram"], "SURP_PHRASE": "1", "INDUCT": "lock",
           "LOCK_TRUST": paths["lock"], "INDUCT_IN": "1", "INDUCT_MIX": "1", "TOKEN_COUNTS": paths["counts"],
           "VOCAB": str(vocab), "PHR_V": str(phr_v), "DATA": os.path.join(out_dir, "tokens.npy"),
           "CORPUS": json.dumps({"synthetic": 1.0}), "CORPUS_ROOT": out_dir}
    json.dump(env, open(os.path.join(out_dir, "env.json"), "w"), indent=1)
    print(f"wrote {len(toks):,} tokens, {shards} shards and phrasebook artefacts to {out_dir}")
    return env
