"""Model families: MemArchLM (product), TransformerLM (control) and their building blocks."""
from .blocks import DenseFFN, FineMoE, LightBlock, TransformerLM   # noqa: F401
from .memarch import MemArchLM                                      # noqa: F401
from .memory import CardMemory, VolumeMemory                        # noqa: F401
from .moe import AnchorMoE                                          # noqa: F401
from .reread import Reread                                          # noqa: F401
