"""Prune a byte-level BPE tokenizer to a token budget without breaking it (the reference's tok/build_pruned.py,
check_pruned.py, sample_counts.py), as pure functions on the `tokenizer.json` dictionary so that they run offline.

Rules that keep the pruned tokenizer sound:
  * all 256 byte tokens stay (any text still encodes) and all special tokens stay;
  * tokens are taken by descending weighted frequency; with a token come all its *ancestors* in the merge table,
    otherwise BPE could never produce it;
  * a merge (a, b) stays only if a, b and a+b all stayed, so the tokenizer emits only kept tokens;
  * new ids are consecutive in the old order, special tokens follow; `old2new` maps ids (for distillation).
"""
from __future__ import annotations

import copy
import json

import numpy as np


def byte_tokens():
    """The 256 symbols byte-level BPE uses for raw bytes (GPT-2 convention)."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs, n = bs[:], 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {chr(c) for c in cs}


def weighted_scores(counts_by_source, weights, V):
    """Sum over sources of weight x (token share within the source): a large source does not drown a small one."""
    score = np.zeros(V)
    for name, w in weights.items():
        c = np.asarray(counts_by_source[name], dtype=np.float64)[:V]
        score[:len(c)] += w * c / max(c.sum(), 1)
    return score


def prune(tok, score, budget):
    """tok: parsed tokenizer.json (dict); score: per old id; budget: ordinary tokens to keep.
    Returns (new tokenizer dict, old2new dict)."""
    t = copy.deepcopy(tok)
    vocab = t["model"]["vocab"]
    merges = [m.split(" ", 1) if isinstance(m, str) else list(m) for m in t["model"]["merges"]]
    inv = {i: s for s, i in vocab.items()}
    parents = {}
    for a, b in merges:
        parents.setdefault(a + b, (a, b))
    keep = set(byte_tokens()) & set(vocab)

    def add(token):
        stack = [token]
        while stack:
            x = stack.pop()
            if x in keep:
                continue
            keep.add(x)
            if x in parents:
                stack.extend(parents[x])

    for i in np.argsort(-np.asarray(score), kind="stable"):
        if len(keep) >= budget or score[i] <= 0:
            break
        if int(i) in inv:
            add(inv[int(i)])
    for a, b in merges:                                   # frequencies ran out: earliest merges are the most general
        if len(keep) >= budget:
            break
        add(a + b)
    order = sorted(keep, key=lambda s: vocab[s])
    new_vocab = {s: j for j, s in enumerate(order)}
    ks = set(order)
    t["model"]["vocab"] = new_vocab
    t["model"]["merges"] = [f"{a} {b}" for a, b in merges if a in ks and b in ks and (a + b) in ks]
    old2new = {vocab[s]: new_vocab[s] for s in order}
    nid = len(new_vocab)
    for at in t.get("added_tokens", []):
        old2new[at["id"]] = nid
        at["id"] = nid
        nid += 1
    if t.get("post_processor"):
        s = json.dumps(t["post_processor"])
        for old, new in old2new.items():
            s = s.replace(f'"id": {old}', f'"id": {new}')
        t["post_processor"] = json.loads(s)
    return t, old2new


def bpe_encode(text_symbols, tok):
    """Reference BPE over a list of byte symbols with the tokenizer's merge ranks (for the round-trip check; the
    production encoder is the `tokenizers` library when it is installed)."""
    ranks = {tuple(m.split(" ", 1)) if isinstance(m, str) else tuple(m): r for r, m in enumerate(tok["model"]["merges"])}
    parts = list(text_symbols)
    while len(parts) > 1:
        best, at = None, -1
        for i in range(len(parts) - 1):
            r = ranks.get((parts[i], parts[i + 1]))
            if r is not None and (best is None or r < best):
                best, at = r, i
        if best is None:
            break
        parts[at:at + 2] = [parts[at] + parts[at + 1]]
    v = tok["model"]["vocab"]
    return [v[p] for p in parts]


def check(pruned, texts_as_symbols):
    """Every text must encode to kept tokens only and decode back to itself; returns (bad, tokens)."""
    inv = {i: s for s, i in pruned["model"]["vocab"].items()}
    bad = n = 0
    for sym in texts_as_symbols:
        try:
            ids = bpe_encode(sym, pruned)
        except KeyError:
            bad += 1
            continue
        n += len(ids)
        bad += "".join(inv[i] for i in ids) != "".join(sym)
    return bad, n


def sample_counts(token_id_streams, V):
    """Token frequencies per source from iterables of id arrays: {source: counts (V,)}."""
    out = {}
    for name, stream in token_id_streams.items():
        c = np.zeros(V, dtype=np.int64)
        for ids in stream:
            c += np.bincount(np.asarray(ids, dtype=np.int64), minlength=V)[:V]
        out[name] = c
    return out
