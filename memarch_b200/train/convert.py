"""Weights as a nested tree with the heavy layers stacked along a layer axis, and that tree as one `.npz` file.

The reference's second code base keeps its parameters in this form and exchanges them with the PyTorch `state_dict`
through a one-to-one name map (memarch_jax/memarch_jax/convert.py:1-71, ckpt.py); a checkpoint written by either side
can therefore be read here:

    emb.weight -> emb, head.weight -> head, norm.weight -> norm, l_norm.weight -> l_norm,
    l_head.0/1.weight -> l_head0/1, book.weight -> book, mix_w, ind_in_g,
    light_a.i.K.weight -> light_a[i][K]   (K in n1, qkv, o, n2, up, down; the same for light_b and final),
    heavy.i.{norm.weight, router.weight, up, down} -> heavy[*] stacked over i,
    memory.X -> memory[X], reread.X -> reread[X];  lock_w, ind_a (frozen) and tau travel beside the tree.

Bookkeeping buffers of the layers (error probes, bank indices, snapshots) are not part of the tree; loading a tree
into a model leaves them at their initial values (`strict=False`).
"""
from __future__ import annotations

import numpy as np
import torch

BLOCK_KEYS = ("n1", "qkv", "o", "n2", "up", "down")
TOP = {"emb": "emb.weight", "book": "book.weight", "head": "head.weight", "norm": "norm.weight",
       "l_norm": "l_norm.weight", "l_head0": "l_head.0.weight", "l_head1": "l_head.1.weight",
       "mix_w": "mix_w", "ind_in_g": "ind_in_g"}
HEAVY = {"norm": "norm.weight", "router": "router.weight", "up": "up", "down": "down"}
GROUPS = ("light_a", "light_b", "final")
BESIDE = ("lock_w", "ind_a", "tau")


def _arr(t):
    if torch.is_tensor(t):
        t = t.detach()
        return (t.float() if t.is_floating_point() else t).cpu().numpy()
    return np.asarray(t)


def _layers(sd, prefix):
    ids = {int(k[len(prefix):].split(".")[0]) for k in sd if k.startswith(prefix)}
    return max(ids) + 1 if ids else 0


def to_tree(sd):
    """state_dict (or any dict with the same names, e.g. gradients) -> (tree, beside); names missing from `sd` are
    skipped, so a dict of gradients with holes converts too."""
    tree = {k: _arr(sd[n]) for k, n in TOP.items() if n in sd}
    for grp in GROUPS:
        tree[grp] = [{k: _arr(sd[f"{grp}.{i}.{k}.weight"]) for k in BLOCK_KEYS if f"{grp}.{i}.{k}.weight" in sd}
                     for i in range(_layers(sd, grp + "."))]
    L = _layers(sd, "heavy.")
    tree["heavy"] = {k: np.stack([_arr(sd[f"heavy.{i}.{n}"]) for i in range(L)])
                     for k, n in HEAVY.items() if L and f"heavy.0.{n}" in sd}
    for grp in ("memory", "reread"):
        tree[grp] = {k[len(grp) + 1:]: _arr(v) for k, v in sd.items() if k.startswith(grp + ".")}
    beside = {k: _arr(sd[k]) for k in BESIDE if k in sd}
    return tree, beside


def from_tree(tree, beside=None):
    """The inverse map -> {state_dict name: numpy array}."""
    out = {n: np.asarray(tree[k]) for k, n in TOP.items() if k in tree}
    for grp in GROUPS:
        for i, blk in enumerate(tree.get(grp, [])):
            for k, v in blk.items():
                out[f"{grp}.{i}.{k}.weight"] = np.asarray(v)
    for k, n in HEAVY.items():
        if k in tree.get("heavy", {}):
            for i, v in enumerate(tree["heavy"][k]):
                out[f"heavy.{i}.{n}"] = np.asarray(v)
    for grp in ("memory", "reread"):
        for k, v in tree.get(grp, {}).items():
            out[f"{grp}.{k}"] = np.asarray(v)
    for k, v in (beside or {}).items():
        out[k] = np.asarray(v)
    return out


def _flatten(node, prefix, out):
    if isinstance(node, dict):
        for k, v in node.items():
            _flatten(v, f"{prefix}/{k}" if prefix else str(k), out)
    elif isinstance(node, (list, tuple)):
        for i, v in enumerate(node):
            _flatten(v, f"{prefix}/{i}", out)
    else:
        out[prefix] = np.asarray(node)


def save_npz(path, tree, beside=None, step=0):
    """One compressed-free `.npz` with path-like keys (`heavy/up`, `light_a/0/qkv`, `beside/tau`), written as a
    temporary file and renamed."""
    import os
    flat = {}
    _flatten(tree, "", flat)
    _flatten(beside or {}, "beside", flat)
    flat["step"] = np.asarray(int(step))
    tmp = path + ".tmp.npz"
    np.savez(tmp, **flat)
    os.replace(tmp, path)


def load_npz(path):
    """-> (tree, beside, step) as written by `save_npz`."""
    z = np.load(path)
    tree, beside = {g: [] for g in GROUPS}, {}
    for key in z.files:
        if key == "step":
            continue
        parts = key.split("/")
        if parts[0] == "beside":
            beside[parts[1]] = z[key]
        elif parts[0] in GROUPS:
            i = int(parts[1])
            while len(tree[parts[0]]) <= i:
                tree[parts[0]].append({})
            tree[parts[0]][i][parts[2]] = z[key]
        elif len(parts) == 2:
            tree.setdefault(parts[0], {})[parts[1]] = z[key]
        else:
            tree[key] = z[key]
    for grp in ("heavy", "memory", "reread"):
        tree.setdefault(grp, {})
    return tree, beside, int(z["step"]) if "step" in z.files else 0


def load_into(model, tree, beside=None):
    """Copy a tree into a model (dtype and device of the model's tensors are kept); returns the names not covered."""
    flat = from_tree(tree, beside)
    sd = model.state_dict()
    with torch.no_grad():
        for k, v in flat.items():
            if k in sd:
                sd[k].copy_(torch.as_tensor(np.array(v)).to(sd[k].dtype).reshape(sd[k].shape))
    return sorted(set(sd) - set(flat))
