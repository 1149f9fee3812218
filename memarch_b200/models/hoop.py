"""Old name of the self-error predictor ("hoop"); kept as an alias of `models.fishki.Uroboros` for code that still
imports it under that name (memarch_jax/memarch_jax/hoop.py:1-3)."""
from .fishki import S_MAX, Uroboros  # noqa: F401

Hoop = Uroboros
