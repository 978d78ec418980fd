"""Tensor-parallel sampling on real GPUs (needs >= 2) and the bounded wait of the exchange kernel
(1 GPU).  With the noise keyed by global vocabulary ids, a sharded draw must equal the unsharded one
bit for bit, on every rank."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _tp_worker(world):
    import os

    import torch.distributed as dist

    import flashsampling_b200 as fs
    from flashsampling_b200 import tensor_parallel as TPX
    from flashsampling_b200.testing import assert_sampling_distribution, gaussian_head, shard_weights
    from flashsampling_b200.tp_info import TPInfo

    tp = TPInfo.from_world()
    dev = torch.device("cuda", torch.cuda.current_device())
    for (V, D, B, S, kernel) in [(8192, 256, 4, 2, "gemv"), (16384, 512, 64, 1, "mma"), (12000, 264, 200, 2, "mma")]:
        V -= V % world
        w, h = gaussian_head(V, D, B, 0.08, seed=V + B)
        t = (torch.rand(B, generator=torch.Generator().manual_seed(1)) + 0.5).to(dev)
        full = fs.fused_mm_sample(w.to(dev), h.to(dev), S, t, seed=42, kernel=kernel)  # unsharded, on this GPU
        w_local = shard_weights(w, tp).contiguous().to(dev)
        for mode in ("p2p", "p2p-unfused", "nccl"):
            os.environ["FMMS_TP_EXCHANGE"] = mode
            for rep in range(3):  # repeated steps exercise epochs and slot parities
                got = fs.fused_mm_sample(w_local, h.to(dev), S, t, seed=42, tp=tp, kernel=kernel)
                assert torch.equal(got, full), (mode, rep, tp.rank, (got != full).sum().item())
        fs.check_status()
    # a vocabulary that does not divide by the number of ranks: the last rank holds the remainder rows and
    # every rank takes the global id of its first row (ids and noise keys) from the total size in TPInfo
    V, D, B, S = 16384 + 5, 256, 33, 2
    tpv = TPInfo.from_world(vocab_size=V)
    w, h = gaussian_head(V, D, B, 0.08, seed=V)
    t = (torch.rand(B, generator=torch.Generator().manual_seed(2)) + 0.5).to(dev)
    full = fs.fused_mm_sample(w.to(dev), h.to(dev), S, t, seed=43)
    w_local = shard_weights(w, tpv, keep_remainder=True).contiguous().to(dev)
    assert w_local.shape[0] == tpv.shard_rows()[1] - tpv.shard_rows()[0]
    for mode in ("p2p", "nccl"):
        os.environ["FMMS_TP_EXCHANGE"] = mode
        got = fs.fused_mm_sample(w_local, h.to(dev), S, t, seed=43, tp=tpv)
        assert torch.equal(got, full), (mode, tp.rank, (got != full).sum().item())
    fs.check_status()
    os.environ["FMMS_TP_EXCHANGE"] = "p2p"
    # a captured tensor-parallel step replays: the exchange keeps its step counter on the device
    V, D, B, S = 16384 - 16384 % world, 256, 32, 1
    w, h = gaussian_head(V, D, B, 0.08, seed=3)
    t = torch.tensor(0.9, device=dev)
    full = fs.fused_mm_sample(w.to(dev), h.to(dev), S, t, seed=5, kernel="mma")
    w_local = shard_weights(w, tp).contiguous().to(dev)
    hd = h.to(dev)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        fs.fused_mm_sample(w_local, hd, S, t, seed=5, tp=tp, kernel="mma")
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        captured = fs.fused_mm_sample(w_local, hd, S, t, seed=5, tp=tp, kernel="mma")
    for _ in range(4):
        captured.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(captured, full), (tp.rank, (captured != full).sum().item())
    got = fs.fused_mm_sample(w_local, hd, S, t, seed=5, tp=tp, kernel="mma")  # eager again, same counter
    assert torch.equal(got, full)
    fs.check_status()
    # log-probabilities: every rank reports on its block, the results are renormalised after an all-gather
    V, D, B, S = 16384 - 16384 % world, 256, 48, 2
    w, h = gaussian_head(V, D, B, 0.08, seed=11)
    hd = h.to(dev)
    full_ids, full_lp = fs.fused_mm_sample(w.to(dev), hd, S, t, seed=7, return_logprobs=True)
    ids, lp = fs.fused_mm_sample(shard_weights(w, tp).contiguous().to(dev), hd, S, t, seed=7, tp=tp,
                                 return_logprobs=True)
    assert torch.equal(ids, full_ids), (tp.rank, (ids != full_ids).sum().item())
    assert float((lp - full_lp).abs().max()) < 1e-3
    fs.check_status()
    # e4m3 weights with per-row scales, sharded: the ids of the unsharded e4m3 draw
    from flashsampling_b200.quant import quantize_rows_e4m3

    V, D, B, S = 16384 - 16384 % world, 256, 48, 1
    w, h = gaussian_head(V, D, B, 0.08, seed=21)
    wq, wsc = quantize_rows_e4m3(w)
    hd = h.to(dev)
    full = fs.fused_mm_sample(wq.to(dev), hd, S, t, seed=11, weight_scale=wsc.to(dev))
    lo, hi = tp.shard_rows(V)
    got = fs.fused_mm_sample(wq[lo:hi].contiguous().to(dev), hd, S, t, seed=11, tp=tp,
                             weight_scale=wsc[lo:hi].contiguous().to(dev))
    assert torch.equal(got, full), (tp.rank, (got != full).sum().item())
    fs.check_status()
    # the reference's distributed protocol: chi-square per rank on sharded ramps (testing.py:264-275)
    for V, nh in ((256, 2), (512, 1)):
        assert_sampling_distribution("fused-triton", V, nh, tp=tp)
    TPX.get_exchange(tp, dev).check_status()
    dist.barrier()
    TPX.close_exchanges()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_sharded_draw_equals_unsharded_tp2():
    from flashsampling_b200.tp_info import run_maybe_distributed

    run_maybe_distributed(_tp_worker, 2, 2)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs >= 4 GPUs")
def test_sharded_draw_equals_unsharded_tp4():
    from flashsampling_b200.tp_info import run_maybe_distributed

    run_maybe_distributed(_tp_worker, 4, 4)


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_sharded_draw_equals_unsharded_tp8():
    from flashsampling_b200.tp_info import run_maybe_distributed

    run_maybe_distributed(_tp_worker, 8, 8)


def test_exchange_wait_is_bounded_and_reports_timeout():
    """A peer that never signals: the kernel gives up after the limit, sets the status word and
    returns ids of -1; the context stays usable."""
    from flashsampling_b200 import _lib, build

    build.build_library()
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    world, max_items, n = 2, 64, 8
    nbytes = ctypes.c_size_t()
    assert lib.fmms_tp_buffer_bytes(world, max_items, ctypes.byref(nbytes)) == 0
    bufs = [torch.zeros(nbytes.value, dtype=torch.uint8, device=dev) for _ in range(world)]  # "rank 1" never runs
    ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    ids = torch.arange(n, dtype=torch.int64, device=dev)
    vals = torch.ones(n, dtype=torch.float32, device=dev)
    out = torch.zeros(n, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = lib.fmms_tp_exchange(ids.data_ptr(), vals.data_ptr(), n, max_items, 0, world, ptrs, 1, 50_000_000,
                              out.data_ptr(), None, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == _lib.ERR_TIMEOUT
    assert (out == -1).all()
    # world of one on the same buffers: completes, and the device still works
    status.zero_()
    ptr1 = (ctypes.c_void_p * 1)(bufs[0].data_ptr())
    rc = lib.fmms_tp_exchange(ids.data_ptr(), vals.data_ptr(), n, max_items, 0, 1, ptr1, 2, 50_000_000,
                              out.data_ptr(), None, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == 0 and torch.equal(out, ids)
