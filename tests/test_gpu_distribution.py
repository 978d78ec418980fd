"""Statistical exactness on the GPU: histograms of sampled ids against softmax(logits / T)."""

import numpy as np
import pytest
import torch

from oracle import fmms_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fs():
    import flashsampling_b200 as fs
    from flashsampling_b200 import build

    build.build_library()
    return fs


@pytest.mark.parametrize("nh", [1, 2])
@pytest.mark.parametrize("V", [100, 256, 512])
@pytest.mark.parametrize("provider", ["fused-triton", "fused-b200"])
def test_sampling_distribution(fs, provider, V, nh):
    """The reference's load-bearing test (tests/test_core.py:58-75): 10 000 draws per row in one
    call, ramps of known logits shifted negative, chi-square p > 0.001."""
    from flashsampling_b200.testing import assert_sampling_distribution

    assert_sampling_distribution(provider, V, nh)
    fs.check_status()


@pytest.mark.parametrize("V", [100, 512])
def test_sampling_distribution_gemv_kernel(fs, V):
    """Same protocol through the weight-streaming kernel: 16 draws per call, 625 calls."""
    from flashsampling_b200.testing import assert_sampling_distribution

    assert_sampling_distribution("fused-b200", V, 2, num_samples=10_000, samples_per_call=16,
                                 sampler_kwargs={"kernel": "gemv"})
    assert fs.last_path() == "gemv"
    fs.check_status()


def _million_draws(fs, kernel, B, S, V=32768, D=64, T=1.0, draws=1_000_000):
    from flashsampling_b200.testing import gaussian_head

    dev = torch.device("cuda", 0)
    w, h1 = gaussian_head(V, D, 1, 1.0 / np.sqrt(D) * 1.5, seed=21)
    h = h1.expand(B, D).contiguous()  # one fixed row, replicated: rows draw independently
    wd, hd = w.to(dev), h.to(dev)
    t = torch.tensor(T, device=dev)
    counts = torch.zeros(V, dtype=torch.int64, device=dev)
    calls = -(-draws // (B * S))
    for c in range(calls):
        ids = fs.fused_mm_sample(wd, hd, S, t, seed=c * S, kernel=kernel)
        counts += torch.bincount(ids.flatten(), minlength=V)
    fs.check_status()
    n = calls * B * S
    probs = O.softmax_probs(O.logits_fp32(w, h1)[0], T)
    p, stat, dof, mass = O.chi_square_pvalue(counts.cpu().numpy(), probs, n)
    print(f"{kernel}: draws={n} dof={dof} mass={mass:.4f} reduced chi2={stat / dof:.5f} p={p:.4f}")
    return p, mass


def test_million_draws_tensor_core_kernel(fs):
    """10^6 draws of one fixed row (B=256 replicas x 4 draws x 977 calls), chi-square p > 0.01."""
    p, mass = _million_draws(fs, "mma", B=256, S=4)
    assert mass > 0.9 and p > 0.01


def test_million_draws_weight_streaming_kernel(fs):
    p, mass = _million_draws(fs, "gemv", B=8, S=4, draws=1_000_000)
    assert mass > 0.9 and p > 0.01
