"""Multi-GPU engines: NCCL baseline and fused peer-memory kernels (one process per GPU)."""
from .engine import NcclExpertExchange, ParallelEngine, init_distributed   # noqa: F401
