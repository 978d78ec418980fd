"""`fused_mm_sampling.testing` names served by the B200 library."""
from flashsampling_b200.testing import (  # noqa: F401
    SyntheticInputs,
    assert_sampling_distribution,
    make_synthetic_inputs,
    shard_weights,
)
