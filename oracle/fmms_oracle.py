"""CPU oracle for the fused LM-head sampling path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module: it is the checker that the
tests, the smoke run and the CPU-baseline leg of the benchmark compare the CUDA
kernels against.  It restates, in plain torch/numpy on the CPU,

* the reference's torch sampling path ``sample()``
  (src/fused_mm_sampling/core.py:33-65: matmul -> fp32 / temperature ->
  softmax -> ``torch.multinomial(replacement=True)``),
* its greedy baseline (core.py:142-158),
* its cross-tile reduction ``_local_reduce`` (core.py:359-370),
* the Gumbel-max form of the same draw (core.py:199-201:
  ``-(-u.log()).log()`` noise, ``max(logits + noise)``) with externally
  supplied noise, which is what the CUDA kernels are compared with index by
  index,
* the chi-square goodness-of-fit protocol of
  src/fused_mm_sampling/testing.py:178-206,
* the second stage of its top-k/top-p path (tl_fused_mm_topk.py:76-107), ahead of
  a CUDA epilogue for it (no kernel uses it yet),

and, for seeded sampling, the counter-based noise stream of the CUDA kernels
themselves (Philox-4x32-10 keyed by global coordinates), so that a seeded GPU
draw can be replayed on the CPU.

Pinning: ``sample``, ``greedy`` and ``local_reduce`` are checked in
tests/test_oracle_golden.py against outputs of the reference's own functions,
produced by importing the reference on the CPU (tests/golden/make_golden.py).
The Philox block function is checked against the published Random123
known-answer vectors.  The reference's in-kernel random stream
(triton.language.random, triton 3.6.0, a third-party dependency) is not
reproduced: no reference test pins it, only distributions are pinned, so seeded
sampling is "parity unpinned" at the bit-stream level and is judged by the
chi-square protocol instead.
"""

from __future__ import annotations

import math

import numpy as np
import torch

# ---------------------------------------------------------------------------
# Reference torch path (core.py:33-65) and friends
# ---------------------------------------------------------------------------


def logits_fp32(weights: torch.Tensor, hidden_states: torch.Tensor) -> torch.Tensor:
    """Exact-input fp32 logits ``H.float() @ W.float().T`` -> [B, V].

    This is the comparison target of the reference's deterministic tests
    (tests/test_core.py:213, :233).  bf16 values upcast exactly to fp32.
    """
    return hidden_states.float() @ weights.float().T


def sample(
    weights: torch.Tensor,  # [V, D]
    hidden_states: torch.Tensor,  # [B, D]
    num_samples: int,
    temperature: torch.Tensor,  # 0-d
    seed: int | None = None,
    return_probs: bool = False,
):
    """The reference's baseline sampler, single rank, no top-k/top-p.

    Follows core.py:46-47 (seed), :51 (matmul in the input dtype), :57
    (upcast to fp32, then divide by the temperature), :95 (softmax) and :62
    (multinomial with replacement).
    """
    if seed is not None:
        torch.manual_seed(seed)
    logits = hidden_states @ weights.T
    logits = logits.float() / temperature
    probs = logits.softmax(dim=-1)
    samples = torch.multinomial(probs, num_samples, replacement=True)
    if return_probs:
        return samples, probs
    return samples


def greedy(weights: torch.Tensor, hidden_states: torch.Tensor) -> torch.Tensor:
    """core.py:142-158: matmul then argmax, returns [B, 1]."""
    logits = hidden_states @ weights.T
    return logits.argmax(dim=-1, keepdim=True)


def local_reduce(maxs: torch.Tensor, maxs_idx: torch.Tensor, vocab_start_index: int = 0):
    """core.py:359-370: argmax over the tile axis of [S, n_tiles, B] candidates.

    Returns (samples [B, S] int64, max_values [B, S] fp32).
    """
    idxs = maxs.max(dim=1).indices
    samples = maxs_idx.gather(1, idxs.unsqueeze(1)).squeeze(1)
    max_values = maxs.gather(1, idxs.unsqueeze(1)).squeeze(1)
    samples = samples + vocab_start_index
    return samples.T.contiguous(), max_values.T.contiguous()


def gumbel_from_uniform(u: torch.Tensor) -> torch.Tensor:
    """core.py:199-200 / :644: ``-log(-log(u))``."""
    return -(-u.log()).log()


def gumbel_argmax(
    logits: torch.Tensor,  # [B, V] fp32
    temperature,  # float, 0-d tensor or [B] tensor; None = greedy
    noise: torch.Tensor | None,  # [S, B, V] or [B, V] fp32; None = greedy
    rel_gap: float = 1e-3,
):
    """Gumbel-max draw with supplied noise: ``argmax(logits / T + noise)``.

    Returns ``(idx [B, S] int64, decisive [B, S] bool, y_max [B, S])``.
    ``decisive`` marks the draws whose two largest perturbed logits differ by
    more than ``rel_gap`` relative to the largest: only those are required to
    match a different-order fp32 accumulation index for index.
    Ties resolve to the lowest index (``torch.argmax`` on CPU).
    """
    logits = logits.float()
    B, V = logits.shape
    if temperature is None:
        y = logits[None]
    else:
        t = torch.as_tensor(temperature, dtype=torch.float32)
        t = t.reshape(-1, 1) if t.ndim > 0 and t.numel() > 1 else t.reshape(1, 1)
        y = (logits / t)[None]
    if noise is not None:
        n = noise.float()
        if n.ndim == 2:
            n = n[None]
        y = y + n
    top2 = y.topk(2, dim=-1).values if V >= 2 else torch.cat([y, y - 1e30], -1)
    idx = y.argmax(dim=-1)  # [S, B]
    gap = (top2[..., 0] - top2[..., 1]) / top2[..., 0].abs().clamp_min(1e-30)
    return idx.T.contiguous(), (gap > rel_gap).T.contiguous(), top2[..., 0].T.contiguous()


# ---------------------------------------------------------------------------
# Noise stream of the CUDA kernels: Philox-4x32-10 keyed by global coordinates
# ---------------------------------------------------------------------------

PHILOX_M0 = np.uint64(0xD2511F53)
PHILOX_M1 = np.uint64(0xCD9E8D57)
PHILOX_W0 = np.uint32(0x9E3779B9)
PHILOX_W1 = np.uint32(0xBB67AE85)
_MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(counter: np.ndarray, key: np.ndarray) -> np.ndarray:
    """Philox-4x32 with 10 rounds (Salmon et al., "Parallel random numbers: as
    easy as 1, 2, 3", SC'11).  ``counter`` [..., 4] and ``key`` [..., 2] uint32.
    """
    c = [counter[..., i].astype(np.uint64) for i in range(4)]
    k0 = np.asarray(key[..., 0], dtype=np.uint32).copy()
    k1 = np.asarray(key[..., 1], dtype=np.uint32).copy()
    with np.errstate(over="ignore"):
        for _ in range(10):
            p0 = PHILOX_M0 * c[0]
            p1 = PHILOX_M1 * c[2]
            hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK32
            hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK32
            c = [
                (hi1 ^ c[1] ^ k0.astype(np.uint64)) & _MASK32,
                lo1,
                (hi0 ^ c[3] ^ k1.astype(np.uint64)) & _MASK32,
                lo0,
            ]
            k0 = (k0 + PHILOX_W0).astype(np.uint32)
            k1 = (k1 + PHILOX_W1).astype(np.uint32)
    return np.stack([x.astype(np.uint32) for x in c], axis=-1)


def kernel_noise_bits(seed: int, sample: int, batch_rows: int, v_begin: int, v_end: int) -> np.ndarray:
    """The 32 random bits the kernels use for every (row b, global vocab id v).

    Key = the 64-bit sum ``seed + sample`` (low word, high word); counter =
    (v >> 2, b, v >> 34, 0); the element takes word ``v & 3`` of the block.
    Independent of tiling, CTA schedule, kernel choice and vocabulary sharding.
    Returns uint32 [batch_rows, v_end - v_begin].
    """
    stream = (int(seed) + int(sample)) & 0xFFFFFFFFFFFFFFFF
    v = np.arange(v_begin, v_end, dtype=np.uint64)
    b = np.arange(batch_rows, dtype=np.uint64)
    vv, bb = np.meshgrid(v, b)  # [B, n]
    ctr = np.stack(
        [
            (vv >> np.uint64(2)) & _MASK32,
            bb,
            (vv >> np.uint64(34)) & _MASK32,
            np.zeros_like(vv),
        ],
        axis=-1,
    ).astype(np.uint32)
    key = np.empty(vv.shape + (2,), dtype=np.uint32)
    key[..., 0] = stream & 0xFFFFFFFF
    key[..., 1] = stream >> 32
    blk = philox4x32_10(ctr, key)
    word = (vv & np.uint64(3)).astype(np.int64)
    return np.take_along_axis(blk, word[..., None], axis=-1)[..., 0]


def kernel_gumbel_from_bits(bits: np.ndarray) -> np.ndarray:
    """fp32 Gumbel variate the kernels derive from 32 random bits.

    w = (r + 0.5) * 2^-32 rounded to fp32; the unit-exponential variate is
    E = -log1p(-w), evaluated as the cubic w(1 + w/2 + w^2/3) below 2^-7 and
    as -ln(1 - w) above; G = -ln(E).  Small w is the upper Gumbel tail (the
    draws that win), and fp32 keeps 24 significant bits of w there.  The
    kernels use the hardware base-2 logarithm approximation, so this agrees
    with them to about 1e-5 absolute, not bit for bit.
    """
    r = bits.astype(np.uint32).astype(np.float32)  # round-to-nearest like cvt.rn.f32.u32
    w = (r * np.float32(2.0**-32) + np.float32(2.0**-33)).astype(np.float32)
    w64 = w.astype(np.float64)
    with np.errstate(divide="ignore"):
        e_small = w64 * (1.0 + w64 * (0.5 + w64 / 3.0))
        e_big = -np.log(np.maximum((np.float32(1.0) - w).astype(np.float32).astype(np.float64), 0.0))
        e = np.where(w < np.float32(2.0**-7), e_small, e_big)
        g = -np.log(e)
    return g.astype(np.float32)


def kernel_noise(seed: int, num_samples: int, batch_rows: int, v_begin: int, v_end: int) -> torch.Tensor:
    """[S, B, v_end - v_begin] fp32 Gumbel noise replaying the kernels' stream."""
    out = np.stack(
        [
            kernel_gumbel_from_bits(kernel_noise_bits(seed, s, batch_rows, v_begin, v_end))
            for s in range(num_samples)
        ]
    )
    return torch.from_numpy(out)


# ---------------------------------------------------------------------------
# Chi-square protocol (testing.py:178-206)
# ---------------------------------------------------------------------------


def chi_square_pvalue(counts: np.ndarray, expected_probs: np.ndarray, num_draws: int):
    """Goodness of fit of one row's histogram against ``expected_probs``.

    Bins with an expected count below 5 are dropped and the remaining expected
    counts rescaled to the observed total, as testing.py:183-188 does.
    Returns (p_value, statistic, dof, tested_probability_mass).
    """
    from scipy.stats import chisquare

    expected = np.asarray(expected_probs, dtype=np.float64) * num_draws
    obs_all = np.asarray(counts, dtype=np.float64)
    mask = expected >= 5
    obs, exp = obs_all[mask], expected[mask]
    mass = exp.sum() / num_draws
    exp = exp * (obs.sum() / exp.sum())
    stat, p = chisquare(obs, exp)
    return float(p), float(stat), int(mask.sum() - 1), float(mass)


def softmax_probs(logits_row: torch.Tensor, temperature: float) -> np.ndarray:
    """fp64 softmax(logits / T) of one row as numpy."""
    z = logits_row.double() / float(temperature)
    return torch.softmax(z, dim=0).numpy()


def log_probs(logits: torch.Tensor, temperature, ids: torch.Tensor):
    """ln softmax(logits / T)[ids] and the log-normaliser, in fp64.

    ``logits`` [B, V], ``temperature`` scalar or [B] (values <= 0 mean greedy
    rows, which use T = 1), ``ids`` [B, S].  The same quantities as
    core.py:57 + :95 of the reference (fp32 logits / T, softmax), taken in log
    space.  Returns (log-probabilities [B, S], log-normaliser [B]).
    """
    t = torch.as_tensor(temperature, dtype=torch.float64).reshape(-1)
    t = torch.where(t > 0, t, torch.ones_like(t))
    z = logits.double() / (t[:, None] if t.numel() > 1 else t)
    lse = torch.logsumexp(z, dim=-1)
    return z.gather(1, ids.long()) - lse[:, None], lse


def topk_topp_probs(logits: torch.Tensor, temperature: float, top_k: int, top_p: float | None = None):
    """Candidates and probabilities of the reference's top-k/top-p path.

    Follows src/fused_mm_sampling/tl_fused_mm_topk.py: logits / T in fp32 (:213),
    the k largest per row in descending order with their ids (:87-88, the merge of
    the per-tile lists is a global top-k), softmax over those k (:91), and for
    ``top_p`` the nucleus mask ``cumsum - p >= top_p`` that always keeps the most
    probable token, followed by renormalisation (:93-98).  Returns (ids [B, k],
    probabilities [B, k]).
    """
    z = logits.float() / temperature
    vals, ids = z.topk(top_k, dim=-1)
    probs = vals.softmax(dim=-1)
    if top_p is not None:
        cumsum = torch.cumsum(probs, dim=-1)
        mask = (cumsum - probs) >= top_p
        mask[:, 0] = False
        probs = probs.masked_fill(mask, 0.0)
        probs = probs / probs.sum(dim=-1, keepdim=True)
    return ids, probs


def topk_topp_sample(logits, temperature, top_k, top_p, num_samples: int, seed: int | None = None):
    """``torch.multinomial`` over ``topk_topp_probs`` (tl_fused_mm_topk.py:101-107)."""
    ids, probs = topk_topp_probs(logits, temperature, top_k, top_p)
    if seed is not None:
        torch.manual_seed(seed)
    picks = torch.multinomial(probs, num_samples=num_samples, replacement=True)
    return ids.gather(dim=-1, index=picks)


# ---------------------------------------------------------------------------
# e4m3 weights: what the fp8 kernels compute, restated (no reference counterpart:
# the reference leaves quantised LM heads to future work,
# findings/cutlass-fmms-kernel-plan.md:1076-1077)
# ---------------------------------------------------------------------------


def e4m3_round_nearest_even(y: torch.Tensor) -> torch.Tensor:
    """Nearest e4m3 value (1 sign, 4 exponent, 3 mantissa bits, bias 7, no infinities, largest finite value
    448), ties to the even mantissa, saturating: what the CUDA conversion does."""
    a = y.double().abs()
    e = torch.floor(torch.log2(a.clamp_min(2.0 ** -40))).clamp_min(-6.0)
    step = torch.pow(torch.tensor(2.0, dtype=torch.float64), e - 3.0)
    q = (torch.round(a / step) * step).clamp_max(448.0)
    return torch.copysign(q, y.double()).float()


def quantize_rows_e4m3(x: torch.Tensor):
    """Per-row e4m3 quantisation: ``q = e4m3(x * (448 / amax))`` (round to nearest even),
    ``scale = amax / 448``; returns ``(q float8_e4m3fn, scale fp32 [rows])``."""
    xf = x.float()
    amax = xf.abs().amax(dim=1).clamp_min(1e-12)
    inv = torch.full_like(amax, 448.0) / amax  # true division (`scalar / tensor` would be reciprocal * scalar)
    return e4m3_round_nearest_even(xf * inv[:, None]).to(torch.float8_e4m3fn), amax / torch.full_like(amax, 448.0)


def quantized_logits(w_q: torch.Tensor, w_scale: torch.Tensor, hidden_states: torch.Tensor) -> torch.Tensor:
    """fp32 logits of the e4m3 path: both operands dequantised (the products of two e4m3 values are exact
    in fp32), hidden states quantised per row exactly as the kernels do on the way in."""
    h_q, h_scale = quantize_rows_e4m3(hidden_states)
    acc = h_q.float() @ w_q.float().T
    return acc * (w_scale.float()[None, :] * h_scale[:, None])


def weight_read_time_us(vocab: int, hidden: int, tb_per_s: float = 8.0) -> float:
    """Pure weight-streaming time of a [vocab, hidden] bf16 matrix in microseconds."""
    return 2.0 * vocab * hidden / (tb_per_s * 1e12) * 1e6


def algorithmic_bytes(vocab: int, hidden: int, batch: int, num_samples: int = 1) -> int:
    """benchmarking/plot-triton-bench.py:236-248: W once + H + int64 ids."""
    return 2 * vocab * hidden + 2 * batch * hidden + 8 * batch * num_samples


def algorithmic_flops(vocab: int, hidden: int, batch: int) -> int:
    return 2 * vocab * hidden * batch


__all__ = [name for name in dir() if not name.startswith("_") and name not in ("math", "np", "torch", "annotations")]
