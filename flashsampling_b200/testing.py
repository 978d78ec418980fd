"""Test inputs and statistical checks for the sampling path.

Restates the helpers of the reference's ``src/fused_mm_sampling/testing.py`` that
its own tests are built on, so that tests written against this package read like
the reference's: inputs with known logits (testing.py:29-74), vocabulary sharding
(:96-104) and the chi-square acceptance protocol (:107-206).  Everything here
runs on whatever device it is given; only ``assert_sampling_distribution`` needs
a GPU, because it calls the sampler.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from .tp_info import TP1, TPInfo


@dataclass
class SyntheticInputs:
    """With tensor parallelism ``weights`` is this rank's vocabulary block."""

    weights: torch.Tensor  # [V, D] bf16
    hidden_states: torch.Tensor  # [B, D] bf16
    logits: torch.Tensor  # [B, V] fp32: the intended logits (before the negative shift)
    vocab_size: int
    hidden_size: int


def shard_weights(weights: torch.Tensor, tp: TPInfo, keep_remainder: bool = False) -> torch.Tensor:
    """Contiguous vocabulary block of ``tp.rank`` (testing.py:96-104).

    Like the reference, ``V % size`` trailing rows are dropped; ``keep_remainder=True`` gives
    them to the last rank instead (``TPInfo.shard_rows``; the sampler then needs
    ``tp.vocab_size``)."""
    if tp.size == 1:
        return weights
    if keep_remainder:
        begin, end = tp.shard_rows(weights.shape[0])
        return weights.narrow(0, begin, end - begin)
    per = weights.shape[0] // tp.size
    return weights.narrow(0, tp.rank * per, per)


def make_synthetic_inputs(
    vocab_size: int = 256,
    hidden_size: int = 10,
    n_hidden_states: int = 2,
    device: torch.device | str = "cuda",
    tp: TPInfo = TP1,
) -> SyntheticInputs:
    """Weights and hidden states whose logits are known ramps (testing.py:29-74).

    Row 0 has logits ``arange(-V/2, V/2)`` and row 1 the reverse.  The hidden
    states are the left singular vectors of the logit matrix padded with
    uniform noise (seed 0), the weights the least-squares solution; both are
    rounded to bf16.  A bias column then shifts every logit by ``-V`` so that a
    zero-filled (instead of -inf-filled) out-of-range row of a ragged tile
    would win the argmax (testing.py:300-327), and D is zero-padded to a
    multiple of 8 for 16-byte row alignment (testing.py:77-93).
    """
    device = torch.device(device)
    half = vocab_size / 2
    ramps = [
        torch.arange(-half, half, dtype=torch.float32)[None, :],
        torch.arange(half, -half, step=-1, dtype=torch.float32)[None, :],
    ]
    logits = torch.cat(ramps[:n_hidden_states], dim=0).to(device)
    n = logits.shape[0]

    u, _, _ = torch.linalg.svd(logits, full_matrices=False)
    torch.manual_seed(0)
    filler = torch.rand((n, hidden_size - n), device=device)
    hidden = torch.cat([u, filler], dim=1).to(device)
    w_t = torch.linalg.pinv(hidden) @ logits  # [D, V]

    w = w_t.bfloat16().T.contiguous()
    h = hidden.bfloat16()
    # bias column: h_new @ w_new^T = h @ w^T - V
    w = torch.cat([w, torch.ones(vocab_size, 1, dtype=w.dtype, device=device)], dim=1)
    h = torch.cat([h, torch.full((n, 1), -float(vocab_size), dtype=h.dtype, device=device)], dim=1)
    # pad D to a multiple of 8 bf16 = 16 bytes
    pad = (-w.shape[1]) % 8
    if pad:
        w = torch.nn.functional.pad(w, (0, pad))
        h = torch.nn.functional.pad(h, (0, pad))
    w = shard_weights(w, tp)
    return SyntheticInputs(weights=w, hidden_states=h, logits=logits, vocab_size=vocab_size, hidden_size=w.shape[1])


def gaussian_head(
    vocab: int, hidden: int, batch: int, w_std: float, seed: int,
    hidden_dtype: torch.dtype = torch.bfloat16, device: torch.device | str = "cpu",
):
    """Seeded stand-in for an LM head: W ~ N(0, w_std^2) in bf16, H ~ N(0, 1).

    Generated on the CPU (so that the values do not depend on the GPU generator)
    and moved to ``device``.
    """
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(vocab, hidden, generator=g) * w_std).bfloat16()
    h = torch.randn(batch, hidden, generator=g).to(hidden_dtype)
    return w.to(device), h.to(device)


def chi_square_row(counts: np.ndarray, probs: np.ndarray, num_draws: int):
    """p-value of one row's histogram against ``probs`` (testing.py:178-206).

    Bins with expected count < 5 are dropped and the rest rescaled to the
    observed total.  Returns (p_value, statistic, dof, tested_mass).
    """
    from scipy.stats import chisquare

    expected = np.asarray(probs, dtype=np.float64) * num_draws
    keep = expected >= 5
    obs = np.asarray(counts, dtype=np.float64)[keep]
    exp = expected[keep]
    mass = float(exp.sum() / num_draws)
    exp = exp * (obs.sum() / exp.sum())
    stat, p = chisquare(obs, exp)
    return float(p), float(stat), int(keep.sum() - 1), mass


def assert_sampling_distribution(
    provider: str,
    vocab_size: int,
    n_hidden_states: int,
    num_samples: int = 10_000,
    tp: TPInfo = TP1,
    inputs: SyntheticInputs | None = None,
    temperature: torch.Tensor | None = None,
    print_result: bool = False,
    samples_per_call: int | None = None,
    p_threshold: float = 0.001,
    sampler_kwargs: dict | None = None,
) -> list[float]:
    """Draw ``num_samples`` per row and test the histogram (testing.py:107-206).

    Same protocol as the reference: temperature ``V / 20`` unless given, seeds
    advancing by ``samples_per_call`` per call, chi-square with the expected>=5
    mask, failure below ``p_threshold``.  Returns the per-row p-values.
    """
    from .core import get_sampler

    device = torch.device("cuda")
    if inputs is None:
        inputs = make_synthetic_inputs(vocab_size=vocab_size, n_hidden_states=n_hidden_states, device=device, tp=tp)
    if temperature is None:
        temperature = torch.tensor(vocab_size / 20.0, device=device)
    sampler = get_sampler(provider, weights=inputs.weights).prepare()
    samples_per_call = samples_per_call or num_samples
    if num_samples % samples_per_call:
        raise ValueError("num_samples must be divisible by samples_per_call")
    rows = inputs.logits.shape[0]
    counts = torch.zeros((rows, inputs.vocab_size), dtype=torch.int64, device=device)
    row_offset = torch.arange(rows, device=device, dtype=torch.int64)[:, None] * inputs.vocab_size
    for call in range(num_samples // samples_per_call):
        ids = sampler.sample(
            weights=inputs.weights,
            hidden_states=inputs.hidden_states,
            num_samples=samples_per_call,
            temperature=temperature,
            tp=tp,
            seed=tp.rank * num_samples + call * samples_per_call,
            **(sampler_kwargs or {}),
        )
        counts += torch.bincount((ids + row_offset).flatten(), minlength=rows * inputs.vocab_size).reshape_as(counts)

    pvals = []
    for r in range(rows):
        probs = (inputs.logits[r].double() / float(temperature)).softmax(dim=0).cpu().numpy()
        p, stat, dof, mass = chi_square_row(counts[r].cpu().numpy(), probs, num_samples)
        if print_result:
            print(
                f"chi-square: provider={provider} V={vocab_size} row={r} draws={num_samples} "
                f"dof={dof} mass={mass:.6f} stat={stat:.2f} reduced={stat / max(dof, 1):.5f} p={p:.5g}"
            )
        assert not math.isnan(p), f"row {r}: chi-square is NaN (all draws in one bin: masked-fill bug?)"
        assert p > p_threshold, f"row {r}: p={p:.3g} - draws do not follow softmax(logits / T)"
        pvals.append(p)
    return pvals
