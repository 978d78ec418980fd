"""`fused_mm_sampling.core` names served by the B200 library."""
from flashsampling_b200.core import (  # noqa: F401
    Sampler,
    SimpleSampler,
    fused_mm_sample,
    fused_mm_sample_triton,
    get_sampler,
)
from flashsampling_b200.tp_info import TP1, TPInfo  # noqa: F401
