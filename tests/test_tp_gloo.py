"""World-size-2 (and 4) tensor-parallel logic on CPU ranks over gloo: every rank computes the oracle's
winners on its own vocabulary block, the collective exchange merges them, and the result must equal
the unsharded oracle draw."""

import numpy as np
import pytest
import torch


def _tp_worker(world, seed):
    import torch.distributed as dist

    from flashsampling_b200.tensor_parallel import CollectiveExchange
    from flashsampling_b200.testing import gaussian_head, shard_weights
    from flashsampling_b200.tp_info import TPInfo
    from oracle import fmms_oracle as O

    tp = TPInfo.from_world()
    assert tp.size == world
    V, D, B, S = 1024, 64, 5, 3
    w, h = gaussian_head(V, D, B, 0.2, seed=seed)
    noise = O.kernel_noise(seed, S, B, 0, V)  # keyed by global ids: identical on every rank
    full_idx, decisive, full_val = O.gumbel_argmax(O.logits_fp32(w, h), 0.9, noise)
    lo, hi = tp.shard_rows(V)
    w_local = shard_weights(w, tp)
    assert w_local.shape[0] == hi - lo
    loc_idx, _, loc_val = O.gumbel_argmax(O.logits_fp32(w_local, h), 0.9, noise[:, :, lo:hi])
    ex = CollectiveExchange(tp, torch.device("cpu"))
    assert ex.vocab_offset(hi - lo) == lo
    ids, vals = ex.reduce(loc_idx + lo, loc_val)
    assert torch.equal(ids, full_idx), (tp.rank, ids, full_idx)
    assert torch.equal(vals, full_val)
    # every rank holds the same answer
    gathered = [torch.empty_like(ids) for _ in range(world)]
    dist.all_gather(gathered, ids)
    assert all(torch.equal(g, ids) for g in gathered)

    # a vocabulary that does not divide by the world size: the last rank holds the remainder rows
    # and every rank takes its offset from the total size carried by TPInfo
    V = 1024 + world - 1
    w, h = gaussian_head(V, D, B, 0.2, seed=seed + 1)
    noise = O.kernel_noise(seed, S, B, 0, V)
    full_idx, _, full_val = O.gumbel_argmax(O.logits_fp32(w, h), 0.9, noise)
    tpv = TPInfo.from_world(vocab_size=V)
    lo, hi = tpv.shard_rows()
    w_local = shard_weights(w, tpv, keep_remainder=True)
    assert w_local.shape[0] == hi - lo and (tp.rank < world - 1 or hi == V)
    loc_idx, _, loc_val = O.gumbel_argmax(O.logits_fp32(w_local, h), 0.9, noise[:, :, lo:hi])
    ex2 = CollectiveExchange(tpv, torch.device("cpu"))
    assert ex2.vocab_offset(hi - lo, tpv) == lo
    ids, vals = ex2.reduce(loc_idx + ex2.vocab_offset(hi - lo, tpv), loc_val)
    assert torch.equal(ids, full_idx) and torch.equal(vals, full_val)
    # the same unequal blocks without the total size: refused on every rank, not silently mis-keyed
    ex3 = CollectiveExchange(tp, torch.device("cpu"))
    with pytest.raises(ValueError, match="vocab_size"):
        ex3.vocab_offset(hi - lo, tp)
    # and a block size that contradicts the declared total
    with pytest.raises(ValueError):
        ex2.vocab_offset(hi - lo + 1, tpv)


@pytest.mark.parametrize("world", [2, 4])
def test_vocab_sharded_draw_equals_unsharded_draw_gloo(world):
    from flashsampling_b200.tp_info import run_maybe_distributed

    run_maybe_distributed(_tp_worker, world, world, 17)


def _tp_logprob_worker(world, seed):
    """Every rank reports its block's winner, that winner's log-probability under the block's own
    normaliser, and the normaliser; after the all-gather all ranks hold the unsharded values."""
    from flashsampling_b200.tensor_parallel import CollectiveExchange, reduce_gathered_logprobs
    from flashsampling_b200.testing import gaussian_head, shard_weights
    from flashsampling_b200.tp_info import TPInfo
    from oracle import fmms_oracle as O

    tp = TPInfo.from_world()
    V, D, B, S, T = 1024, 64, 5, 3, 0.9
    w, h = gaussian_head(V, D, B, 0.2, seed=seed)
    noise = O.kernel_noise(seed, S, B, 0, V)
    logits = O.logits_fp32(w, h)
    full_idx, _, _ = O.gumbel_argmax(logits, T, noise)
    full_lp, _ = O.log_probs(logits, T, full_idx)
    lo, hi = tp.shard_rows(V)
    loc_logits = O.logits_fp32(shard_weights(w, tp), h)
    loc_idx, _, loc_val = O.gumbel_argmax(loc_logits, T, noise[:, :, lo:hi])
    loc_lp, loc_lse = O.log_probs(loc_logits, T, loc_idx)
    ex = CollectiveExchange(tp, torch.device("cpu"))
    ids, vals, lp = reduce_gathered_logprobs(ex, loc_idx + lo, loc_val, loc_lp.float(), loc_lse.float())
    assert torch.equal(ids, full_idx)
    assert (lp.double() - full_lp).abs().max() < 1e-5, (tp.rank, lp, full_lp)


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_log_probabilities_renormalise_gloo(world):
    from flashsampling_b200.tp_info import run_maybe_distributed

    run_maybe_distributed(_tp_logprob_worker, world, world, 23)


def test_shard_rows_cover_vocab_without_overlap():
    from flashsampling_b200.tp_info import TPInfo

    for V in (100, 151936, 128256, 262208, 1001):
        for size in (1, 2, 4, 8):
            spans = [TPInfo(r, size).shard_rows(V) for r in range(size)]
            assert spans[0][0] == 0 and spans[-1][1] == V
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
