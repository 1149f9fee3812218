"""`build(name, vocab)`: the model registry (the reference's `lm.build`, lm.py:752-807).

FullLM2-family names (`Fv2*`, `Fv3*`, `Fn*`, `Fns*`) and the presets of this package build a `MemArchLM`;
`T300`, `Td<d>L<L>`, `transformer` build the plain transformer control.  The v0/v1 prototype names of the reference
(`surp*`, `plan*`, `sketch*`, `img_*`, `cards`, `tail`, `S300*`, `F300*`) are served by `memarch_b200.models.legacy`.
"""
from __future__ import annotations

from .config import ModelConfig, preset
from .models import MemArchLM, TransformerLM


def build(name: str, vocab: int = 50304, env=None, **overrides):
    if isinstance(name, ModelConfig):
        return MemArchLM(name)
    if name == "T300":
        return TransformerLM(vocab, d=1024, layers=16, heads=16)
    if name.startswith("Td") and "L" in name:
        d, L = name[2:].split("L")
        return TransformerLM(vocab, d=int(d), layers=int(L), heads=int(d) // 128)
    if name == "transformer":
        return TransformerLM(vocab)
    try:
        cfg = preset(name, vocab, env)
    except ValueError:
        from .models import legacy
        return legacy.build_legacy(name, vocab)
    if overrides:
        cfg = cfg.replace(**overrides)
    return MemArchLM(cfg)
