"""Phrasebook artefacts built from a token corpus, in the file formats the reference's model loads.

  * `bigram_init`  - "born with ready phrases": PPMI of (word -> next word) pairs, rank-d SVD -> input table E,
                     output table H, log-frequency bias `logp_next`, and per-previous-word `lse` of the pair
                     forecast used for phrase surprise (tools/phr/bigram_init.py:10-24, lse.py:4-9).
  * `phrase_table` - top-K (previous, current) contexts -> ridge projection of their PPMI with the next word onto
                     H, a vector to add to the input (tools/phr/trigram_init.py:9-28).
  * `lock_trust`   - hit-rate of the 1/2/3-word locks by rarity bucket of the current word -> initial trust
                     (tools/phr/lock_trust.py:15-31).
  * `context_table` order 3 - the three-word table (`PHRASE4`, tools/phr/quad_init.py); `skip_table` - "draft ahead"
                     vectors for offsets 2..4 (`SKIP`, tools/phr/skip_init.py); `phrase_units` - phrase vocabulary and
                     the rewritten corpus (tools/phr/phrase_tok.py); `slice_report` - per-slice loss gap against a
                     rival model (tools/phr/diag_analyze.py).
  * `token_counts` - unigram counts.
  * `prior_top`    - top-32 continuations per word from the pair forecaster; `tongue_tables` - the counted top
                     continuations of words and pair contexts the model loads as `TONGUE` (tools/phr/prior_top.py);
                     `entropy` per word (ent.py).
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


def _project_onto_head(H, rows, cols, vals, n_rows, device="cpu"):
    """Rows of a sparse (n_rows, V) PPMI matrix M expressed in the basis of the output table H (V, d): the ridge
    solution P of P · Hᵀ ≈ M, so that a row of P can be added to the model's input like a word vector."""
    Hd = H.to(device).double()
    M = torch.sparse_coo_tensor(torch.tensor(np.stack([rows, cols])), torch.tensor(vals), (n_rows, Hd.shape[0])).coalesce().to(device)
    gram = Hd.T @ Hd + 1e-3 * torch.eye(Hd.shape[1], dtype=Hd.dtype, device=device)
    return torch.linalg.solve(gram, (M @ Hd).T).T.float()


def context_table(a, H, K, order=2, vocab=50257, device="cpu"):
    """The K most frequent contexts of `order` consecutive words -> a vector forecasting the word after them.
    order 2 is the phrase table (tools/phr/trigram_init.py:9-28), order 3 the three-word table the model loads as
    `PHRASE4` (tools/phr/quad_init.py:9-27).  Key of a context: its words as digits of a base-`vocab` number, first
    word most significant; returns {"keys": sorted int64 (K,), "vec": (K, d)}."""
    a = np.asarray(a, dtype=np.int64)
    V, n = vocab, order
    span = len(a) - n                                    # contexts that have a next word
    ctx = np.zeros(span, dtype=np.int64)
    for j in range(n):
        ctx = ctx * V + a[j:j + span]
    nxt_all = a[n:]
    uc, cc = np.unique(ctx, return_counts=True)
    K = min(K, len(uc))
    keys = np.sort(uc[np.argsort(-cc, kind="stable")[:K]])
    pos = np.searchsorted(keys, ctx)
    hit = (pos < K) & (keys[np.minimum(pos, K - 1)] == ctx)
    row, nxt = pos[hit], nxt_all[hit]
    ut, ct = np.unique(row * V + nxt, return_counts=True)
    r, w = ut // V, ut % V
    per_row = np.bincount(row, minlength=K).astype(np.float64)
    per_word = np.bincount(nxt_all, minlength=V).astype(np.float64)
    pmi = np.log(ct * len(a) / (per_row[r] * per_word[w]))
    keep = (pmi > 0) & (ct >= 2)
    return {"keys": torch.tensor(keys), "vec": _project_onto_head(H, r[keep], w[keep], pmi[keep], K, device)}


def phrase_table(a, H, K, vocab=50257, device="cpu"):
    return context_table(a, H, K, 2, vocab, device)


def skip_table(a, H, offsets=(2, 3, 4), vocab=50257, min_count=3, device="cpu"):
    """"Draft ahead": what usually stands o words after this word, for each o in `offsets` - PPMI(word_t, word_t+o)
    in the basis of H; the file the model loads as `SKIP` is {o: (V, d)} (tools/phr/skip_init.py:9-21)."""
    a = np.asarray(a, dtype=np.int64)
    V = vocab
    freq = np.bincount(a, minlength=V).astype(np.float64)
    out = {}
    for o in offsets:
        u, c = np.unique(a[:-o] * V + a[o:], return_counts=True)
        first, later = u // V, u % V
        pmi = np.log(c * (len(a) - o) / (freq[first] * freq[later]))
        keep = (pmi > 0) & (c >= min_count)
        out[int(o)] = _project_onto_head(H, first[keep], later[keep], pmi[keep], V, device)
    return out


def phrase_units(a, n_units, vocab=50257, eot=50256, count_from=None):
    """Phrase vocabulary: the `n_units` n-grams (n = 2..4, not crossing a document end) whose merging saves the most
    steps (count x (n-1)) become units with ids vocab, vocab+1, ...; the text is rewritten greedily, longest units
    first, left to right within a length (tools/phr/phrase_tok.py:6-61).  Returns (rewritten tokens uint32, units as
    an (n_units, 4) int64 array padded with -1).  `count_from`: slice of `a` the frequencies are taken from."""
    a = np.asarray(a, dtype=np.int64)
    V = vocab
    src = a[count_from] if count_from is not None else a

    def keys_of(t, n):
        k = np.zeros(len(t) - n + 1, dtype=np.int64)
        for j in range(n):
            k = k * V + t[j:len(t) - n + 1 + j]
        return k

    scored = []
    for n in (2, 3, 4):
        if len(src) < n:
            continue
        k = keys_of(src, n)
        inside = np.ones(len(k), dtype=bool)
        for j in range(n):
            inside &= src[j:len(src) - n + 1 + j] != eot
        u, c = np.unique(k[inside], return_counts=True)
        best = np.argsort(-c, kind="stable")[:n_units]
        scored += [(int(c[i]) * (n - 1), n, int(u[i])) for i in best]
    scored.sort(reverse=True)
    by_len = {}
    for _, n, key in scored[:n_units]:
        by_len.setdefault(n, []).append(key)
    units, unit_id = [], {}
    for n in (4, 3, 2):
        for key in by_len.get(n, []):
            unit_id[(n, key)] = V + len(units)
            digits = [(key // V ** (n - 1 - j)) % V for j in range(n)]
            units.append(digits + [-1] * (4 - n))
    covered = np.zeros(len(a), dtype=bool)
    starts = np.full(len(a), -1, dtype=np.int64)
    for n in (4, 3, 2):
        if n not in by_len or len(a) < n:
            continue
        k = keys_of(a, n)
        table = np.sort(np.asarray(by_len[n], dtype=np.int64))
        at = np.searchsorted(table, k).clip(max=len(table) - 1)
        free_from = 0                                       # first position not inside a unit of this length
        for i in np.nonzero(table[at] == k)[0]:
            if i >= free_from and not covered[i:i + n].any():
                covered[i:i + n] = True
                starts[i] = unit_id[(n, int(k[i]))]
                free_from = i + n
    keep = ~covered | (starts >= 0)
    return np.where(starts >= 0, starts, a)[keep].astype(np.uint32), np.asarray(units, dtype=np.int64).reshape(-1, 4)


def slice_report(ours, theirs, x, y, counts, ph=None, T=1024, phrase_c=0.05):
    """Where a rival model is better: mean per-word loss of both and the share of the total gap, by slices of the
    target word's frequency, the position in the window, the pair forecaster's surprise (with `ph`, the bigram
    artefact) and whether the target already occurred in the window (tools/phr/diag_analyze.py:3-41).
    ours / theirs: per-word losses; x / y: inputs and targets (flat, windows of T).  Returns {slice group: rows}
    with rows (label, share of words, ours, theirs, gap, share of the gap)."""
    ours, theirs = np.asarray(ours, dtype=np.float64), np.asarray(theirs, dtype=np.float64)
    x, y = np.asarray(x, dtype=np.int64), np.asarray(y, dtype=np.int64)
    gap = ours - theirs
    total = gap.sum()

    def rows(masks, labels):
        out = []
        for m, l in zip(masks, labels):
            if m.any():
                out.append((l, float(m.mean()), float(ours[m].mean()), float(theirs[m].mean()), float(gap[m].mean()),
                            float(gap[m].sum() / total) if total else 0.0))
            else:
                out.append((l, 0.0, float("nan"), float("nan"), float("nan"), 0.0))
        return out

    fq = np.asarray(counts)[np.minimum(y, len(counts) - 1)]
    pos = np.tile(np.arange(T), len(x) // T + 1)[:len(x)]
    rep = np.zeros(len(x), dtype=bool)
    for w0 in range(0, len(x), T):
        seen = set()
        for i in range(w0, min(w0 + T, len(x))):
            rep[i] = y[i] in seen
            seen.add(x[i])
    report = {
        "frequency of the target": rows([fq >= 1e5, (fq >= 1e4) & (fq < 1e5), (fq >= 1e3) & (fq < 1e4), (fq >= 100) & (fq < 1e3),
                                         fq < 100], [">=100k", "10k-100k", "1k-10k", "100-1k", "<100"]),
        "position in the window": rows([pos < 16, (pos >= 16) & (pos < 128), (pos >= 128) & (pos < 512), pos >= 512],
                                       ["0-15", "16-127", "128-511", "512+"]),
        "target seen in the window": rows([rep, ~rep], ["seen", "new"]),
    }
    if ph is not None:
        E, H, lp = ph["emb"], ph["head"], ph["logp_next"]
        En = E / E.pow(2).mean(1, keepdim=True).sqrt().clamp(min=1e-6)
        top = E.shape[0] - 1
        xx, yy = torch.tensor(np.minimum(x, top)), torch.tensor(np.minimum(y, top))
        sp = (ph["lse"][xx] - (phrase_c * (En[xx] * H[yy]).sum(-1) + lp[yy])).numpy()
        report["surprise of the pair forecaster"] = rows([sp < 2, (sp >= 2) & (sp < 5), (sp >= 5) & (sp < 8), sp >= 8],
                                                         ["<2", "2-5", "5-8", ">=8 (anchors)"])
    return report


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


def _top_continuations(ctx, nxt, n_ctx, log_unigram, vocab, k_top):
    """For every context row the `k_top` next words with the highest PMI (log of the conditional frequency minus the
    log unigram probability), among (context, next) pairs seen at least twice; PMI below zero is stored as zero.
    Returns (idx (n_ctx, k_top) int32, val (n_ctx, k_top) float16), empty places zero."""
    pair, cnt = np.unique(ctx * vocab + nxt, return_counts=True)
    row, word = pair // vocab, pair % vocab
    per_row = np.bincount(row, weights=cnt, minlength=n_ctx)
    pmi = np.where(cnt >= 2, np.log(cnt / per_row[row]) - log_unigram[word], -1e9)
    by_score = np.argsort(-pmi, kind="stable")
    order = by_score[np.argsort(row[by_score], kind="stable")]          # rows ascending, best PMI first inside a row
    row, word, pmi = row[order], word[order], pmi[order]
    place = np.arange(len(row)) - np.searchsorted(row, np.arange(n_ctx))[row]
    keep = place < k_top
    idx = np.zeros((n_ctx, k_top), dtype=np.int64)
    val = np.zeros((n_ctx, k_top), dtype=np.float32)
    idx[row[keep], place[keep]] = word[keep]
    val[row[keep], place[keep]] = np.maximum(pmi[keep], 0)
    return torch.tensor(idx, dtype=torch.int32), torch.tensor(val, dtype=torch.float16)


def tongue_tables(a, keys, vocab=50257, k_top=32):
    """"Words on the tip of the tongue": counted top continuations of every word and of every pair context of the
    phrase table `keys`, with their PMI - the file the model loads as `TONGUE` and adds to its output logits
    ({bi_idx, bi_val, tri_idx, tri_val, keys}; tools/phr/prior_top.py:3-32)."""
    a = np.asarray(a, dtype=np.int64)
    freq = np.bincount(a, minlength=vocab).astype(np.float64)
    log_unigram = np.log((freq + 1) / freq.sum())
    bi_idx, bi_val = _top_continuations(a[:-1], a[1:], vocab, log_unigram, vocab, k_top)
    kk = np.asarray(keys, dtype=np.int64)
    pair = a[:-2] * vocab + a[1:-1]
    at = np.searchsorted(kk, pair).clip(max=len(kk) - 1)
    known = kk[at] == pair
    tri_idx, tri_val = _top_continuations(at[known], a[2:][known], len(kk), log_unigram, vocab, k_top)
    return {"bi_idx": bi_idx, "bi_val": bi_val, "tri_idx": tri_idx, "tri_val": tri_val, "keys": torch.as_tensor(kk)}


def build_all(tokens, d, out_dir, vocab=50257, phrase_k=262144, seed=0, quad_k=0, skip=False):
    """Write every artefact of the published recipe under `out_dir` (plus the three-word table with `quad_k` and the
    draft-ahead tables with `skip`); returns the paths."""
    os.makedirs(out_dir, exist_ok=True)
    paths = {k: os.path.join(out_dir, v) for k, v in
             dict(bigram="bigram.pt", trigram="trigram.pt", lock="lock_trust.pt", counts="token_counts.npy").items()}
    cnt = token_counts(tokens, vocab)
    np.save(paths["counts"], cnt)
    ph = bigram_init(tokens, d, vocab, seed=seed)
    torch.save(ph, paths["bigram"])
    torch.save(phrase_table(tokens, ph["head"], phrase_k, vocab), paths["trigram"])
    torch.save(lock_trust(tokens, vocab, cnt), paths["lock"])
    if quad_k:
        paths["quad"] = os.path.join(out_dir, "quad.pt")
        torch.save(context_table(tokens, ph["head"], quad_k, 3, vocab), paths["quad"])
    if skip:
        paths["skip"] = os.path.join(out_dir, "skip.pt")
        torch.save(skip_table(tokens, ph["head"], vocab=vocab), paths["skip"])
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
