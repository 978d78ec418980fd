"""`fused_mm_sampling.tp_info` names served by the B200 library."""
from flashsampling_b200.tp_info import TP1, TPInfo, run_maybe_distributed  # noqa: F401
