"""Ops of the memarch B200 framework: sm_100a CUDA kernels with PyTorch oracles (see `_ext`, `ref`)."""
from . import _ext, ref                                            # noqa: F401
from .basic import rmsnorm, relu2, swiglu, linear, linear_act, ffn, gemm, gemm_ok, resid_add, add_rmsnorm   # noqa: F401
from .attention import attention                                   # noqa: F401
from .ce import linear_ce, chunk_ce                                # noqa: F401
from .anchors import select_anchors, find_locks, gather_tokens, scatter_back   # noqa: F401
from .embed import embed_sum                                      # noqa: F401
from .moe import slot_gather, combine, expert_ffn, route_and_slot  # noqa: F401
