"""The oracle against outputs of the reference itself (tests/golden/reference_golden.npz,
written by tests/golden/make_golden.py) and against published known-answer vectors."""

import numpy as np
import pytest
import torch

from flashsampling_b200 import testing as T
from flashsampling_b200.tp_info import TPInfo
from oracle import fmms_oracle as O


def _bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.copy()).view(torch.bfloat16)


@pytest.mark.parametrize("nh", [1, 2])
@pytest.mark.parametrize("V", [100, 256, 512])
def test_synthetic_inputs_match_reference(golden, V, nh):
    inp = T.make_synthetic_inputs(vocab_size=V, hidden_size=10, n_hidden_states=nh, device="cpu")
    tag = f"syn_V{V}_H{nh}"
    assert torch.equal(inp.weights, _bf16(golden[f"{tag}_weights_bf16"]))
    assert torch.equal(inp.hidden_states, _bf16(golden[f"{tag}_hidden_bf16"]))
    assert torch.equal(inp.logits, torch.from_numpy(golden[f"{tag}_logits"]))
    assert inp.hidden_size % 8 == 0


@pytest.mark.parametrize("nh", [1, 2])
@pytest.mark.parametrize("V", [100, 256, 512])
def test_oracle_sample_and_greedy_match_reference(golden, V, nh):
    tag = f"syn_V{V}_H{nh}"
    w, h = _bf16(golden[f"{tag}_weights_bf16"]), _bf16(golden[f"{tag}_hidden_bf16"])
    ids = O.sample(w, h, 64, torch.tensor(V / 20.0), seed=7)
    assert np.array_equal(ids.numpy(), golden[f"{tag}_sample_seed7"])
    assert np.array_equal(O.greedy(w, h).numpy(), golden[f"{tag}_greedy"])


def test_oracle_sample_small_gaussian_head(golden):
    w, h = T.gaussian_head(4096, 256, 4, 0.05, seed=11)
    assert np.allclose([w.double().sum().item(), w.double().abs().sum().item()], golden["small_w_checksum"], rtol=0, atol=0)
    assert np.allclose([h.double().sum().item(), h.double().abs().sum().item()], golden["small_h_checksum"], rtol=0, atol=0)
    ids = O.sample(w, h, 16, torch.tensor(0.7), seed=3)
    assert np.array_equal(ids.numpy(), golden["small_sample_seed3_T0p7"])


def test_oracle_config1_qwen_head_on_cpu(golden):
    """The CPU-runnable benchmark configuration: V=151936, d=4096, B=4, fp32 hidden states, T=1, 1 draw per row."""
    w, h = T.gaussian_head(151936, 4096, 4, 0.02, seed=0, hidden_dtype=torch.float32)
    w32 = w.float()
    assert [w32.double().sum().item(), w32.double().abs().sum().item()] == list(golden["cfg1_w_checksum"])
    ids = O.sample(w32, h, 1, torch.tensor(1.0), seed=0)
    assert np.array_equal(ids.numpy(), golden["cfg1_sample_seed0_T1"])
    assert np.array_equal(O.greedy(w32, h).numpy(), golden["cfg1_greedy"])
    # the Gumbel-max form with T=1 and zero noise is the greedy answer, every row decisive
    logits = O.logits_fp32(w32, h)
    idx, decisive, _ = O.gumbel_argmax(logits, 1.0, None)
    assert np.array_equal(idx.numpy(), golden["cfg1_greedy"])
    stats = torch.stack([logits.max(-1).values, logits.min(-1).values, logits.sum(-1)]).numpy()
    assert np.allclose(stats, golden["cfg1_logits_rowstats"], rtol=1e-4, atol=1e-3)


def test_local_reduce_matches_reference(golden):
    s, v = O.local_reduce(
        torch.from_numpy(golden["local_reduce_maxs"]), torch.from_numpy(golden["local_reduce_maxs_idx"]), 1234
    )
    assert np.array_equal(s.numpy(), golden["local_reduce_samples"])
    assert np.array_equal(v.numpy(), golden["local_reduce_values"])


def test_shard_rows_match_reference(golden):
    for V, size, rank, begin, end in golden["shard_rows"]:
        marker = torch.arange(int(V), dtype=torch.int32)[:, None]
        sh = T.shard_weights(marker, TPInfo(rank=int(rank), size=int(size)))
        assert (int(sh[0, 0]), int(sh[-1, 0]) + 1) == (begin, end)
        b, e = TPInfo(rank=int(rank), size=int(size)).shard_rows(int(V))
        assert b == begin
        # the reference drops V % size trailing rows; here the last rank keeps them
        assert e == (V if rank == size - 1 else end)


def test_philox_known_answers():
    """Random123 known-answer vectors for philox4x32_10."""
    kat = [
        ([0, 0, 0, 0], [0, 0], [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]),
        ([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2, [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]),
        (
            [0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344],
            [0xA4093822, 0x299F31D0],
            [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1],
        ),
    ]
    for ctr, key, want in kat:
        got = O.philox4x32_10(np.array(ctr, dtype=np.uint32), np.array(key, dtype=np.uint32))
        assert [int(x) for x in got] == want


def test_kernel_noise_is_standard_gumbel_and_shard_invariant():
    g = O.kernel_gumbel_from_bits(O.kernel_noise_bits(123, 0, 8, 0, 100_000)).astype(np.float64)
    assert abs(g.mean() - 0.5772156649) < 0.01
    assert abs(g.var() - np.pi**2 / 6) < 0.02
    assert np.isfinite(g).all()
    # keyed by global coordinates: a slice of the full stream equals the stream of the slice
    full = O.kernel_noise_bits(5, 2, 3, 0, 4096)
    part = O.kernel_noise_bits(5, 2, 3, 1001, 3003)
    assert np.array_equal(full[:, 1001:3003], part)
    # the draw index adds to the seed (the reference's seed + sample_idx stream id, core.py:644)
    assert np.array_equal(O.kernel_noise_bits(7, 3, 2, 0, 64), O.kernel_noise_bits(10, 0, 2, 0, 64))


def test_gumbel_tails():
    bits = np.array([0, 1, 2**25, 2**31, 2**32 - 1], dtype=np.uint32)
    g = O.kernel_gumbel_from_bits(bits)
    assert abs(g[0] - (-np.log(2.0**-33))) < 1e-4  # smallest w: largest finite Gumbel ~ 22.87
    assert np.all(np.diff(g[:4]) < 0)  # decreasing in w
    assert g[4] == -np.inf  # w rounds to 1: never wins


def test_gumbel_argmax_oracle_distribution():
    """Gumbel-max with the kernel's noise stream reproduces softmax (chi-square, p > 0.01)."""
    torch.manual_seed(0)
    V, draws = 64, 20_000
    logits = torch.randn(1, V) * 2
    counts = np.zeros(V)
    for s0 in range(0, draws, 1000):
        noise = O.kernel_noise(seed=s0, num_samples=1000, batch_rows=1, v_begin=0, v_end=V)
        idx, _, _ = O.gumbel_argmax(logits, 0.8, noise)
        counts += np.bincount(idx[0].numpy(), minlength=V)
    p, *_ = O.chi_square_pvalue(counts, O.softmax_probs(logits[0], 0.8), draws)
    assert p > 0.01


def test_bsz_h_table_recorded(golden):
    """The reference's batch-tile heuristic (core.py:876-881) is recorded for completeness; the
    kernels here plan their tiles in fmms_plan (see test_host_logic.py)."""
    table = dict(zip(golden["bsz_h_in"].tolist(), golden["bsz_h_out"].tolist()))
    assert (table[1], table[16], table[17], table[32], table[33], table[64], table[65]) == (16, 16, 32, 32, 64, 64, 64)


def test_topk_topp_oracle_matches_reference_merge():
    """The reference's own top-k/top-p second stage, run on exact per-tile top-k lists
    (tests/golden/make_golden_topk.py), against the oracle's restatement on the full logits."""
    from pathlib import Path

    data = np.load(Path(__file__).resolve().parent / "golden" / "reference_topk_golden.npz")
    n = 0
    while f"case{n}_logits" in data:
        logits = torch.from_numpy(data[f"case{n}_logits"])
        V, H, k, top_p, temp, seed, draws = data[f"case{n}_params"].tolist()
        got = O.topk_topp_sample(logits, temp, int(k), None if top_p < 0 else top_p, int(draws), seed=int(seed))
        want = torch.from_numpy(data[f"case{n}_samples"])
        assert torch.equal(got, want), f"case {n}"
        ids, probs = O.topk_topp_probs(logits, temp, int(k), None if top_p < 0 else top_p)
        assert ids.shape == (int(H), int(k)) and torch.allclose(probs.sum(-1), torch.ones(int(H)))
        if top_p >= 0:  # the kept prefix holds at least top_p of the top-k mass, and no more tokens than needed
            full = (logits / temp).topk(int(k), dim=-1).values.softmax(-1)
            kept = probs > 0
            assert bool(((full * kept).sum(-1) >= min(top_p, 1.0) - 1e-6).all())
        n += 1
    assert n == 4
