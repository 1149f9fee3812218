"""memarch_b200: a Blackwell-native (sm_100a) training framework for the memarch model family.

Light sliding-window layers on every token; heavy top-2 MoE layers only on causally selected surprise anchors;
phrasebook initialisation, phrase table and keys-and-locks pointer head; fresh/dim card memory with re-reading; the
Instinct one-momentum optimizer with homeostasis applied inside backward; wave training with a frozen expert bank.
"""
from .build import build                                   # noqa: F401
from .config import ModelConfig, OptConfig, ParallelConfig, TrainConfig, preset   # noqa: F401

__version__ = "0.1.0"
