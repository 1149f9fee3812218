"""Loader of the in-tree sm_100a extension (`memarch_b200/_C*.so`, built by `__graft_entry__.build()`).

Every op in this package has two bodies: the hand-written CUDA kernel (used whenever the tensors live on a GPU)
and a plain PyTorch statement of the same maths (used on CPU, and as the numerics oracle in the tests).  On a
machine with a GPU a missing extension is an error, never a silent fallback.
"""
from __future__ import annotations

import glob
import importlib.util
import os
import threading

import torch

_lock = threading.Lock()
_mod = None
_err = None
launch_count = 0          # kernels of this package launched since process start (bench.py reports the delta)
gemm_flops = 0            # nominal 2·M·N·K of the tensor-core GEMMs issued through `ops.gemm` (padding places included)


def _pkg_dir():
    return os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def so_path():
    hits = sorted(glob.glob(os.path.join(_pkg_dir(), "_C*.so")))
    return hits[0] if hits else None


def load(required: bool = False):
    """Return the extension module or None.  `required=True` raises with the reason instead."""
    global _mod, _err
    if _mod is not None:
        return _mod
    with _lock:
        if _mod is None and _err is None:
            p = so_path()
            if p is None:
                _err = "memarch_b200/_C*.so not built (run `python -c 'import __graft_entry__ as g; g.build()'`)"
            else:
                try:
                    spec = importlib.util.spec_from_file_location("memarch_b200._C", p)
                    m = importlib.util.module_from_spec(spec)
                    spec.loader.exec_module(m)
                    _mod = m
                except Exception as e:   # noqa: BLE001 - reported verbatim to the caller
                    _err = f"{type(e).__name__}: {e}"
    if _mod is None and required:
        raise RuntimeError(f"memarch_b200 CUDA extension unavailable: {_err}")
    return _mod


def C():
    """The extension, required.  Ops call this on their CUDA path so a GPU box without the .so fails loudly."""
    return load(required=True)


def available() -> bool:
    return load() is not None


def use_cuda(*tensors) -> bool:
    """True when the op must take its CUDA-kernel body: a tensor argument lives on a GPU."""
    for t in tensors:
        if isinstance(t, torch.Tensor) and t.is_cuda:
            if os.environ.get("MEMARCH_FORCE_TORCH") == "1":      # oracle mode for A/B numerics checks on the GPU
                return False
            return True
    return False


def count(n: int = 1):
    global launch_count
    launch_count += n


def count_flops(n: int):
    global gemm_flops
    gemm_flops += n
