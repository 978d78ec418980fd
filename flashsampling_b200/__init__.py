"""B200-native fused LM-head sampling (matmul + Gumbel-max in one pass over the weight)."""

from .core import (  # noqa: F401
    PROVIDERS,
    PreparedSampler,
    Sampler,
    SimpleSampler,
    check_status,
    fused_mm_sample,
    fused_mm_sample_triton,
    get_sampler,
    last_path,
)
from .tp_info import TP1, TPInfo, run_maybe_distributed  # noqa: F401

__version__ = "0.1.0"
