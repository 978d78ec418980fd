"""GPU parity: the CUDA kernels (through the C ABI) against the CPU oracle.

Bit-exact for indices wherever the decision is not within fp32 accumulation noise:
a draw is compared only if the oracle's two largest perturbed logits differ by more
than 1e-3 relative (the tolerance the task states); logits are compared with
atol = rtol = 1e-4 as the reference's own test does (tests/test_core.py:213-215).
"""

import numpy as np
import pytest
import torch

from oracle import fmms_oracle as O

pytestmark = pytest.mark.gpu

REL_GAP = 1e-3


@pytest.fixture(scope="module")
def fs():
    import flashsampling_b200 as fs
    from flashsampling_b200 import build

    build.build_library()
    assert torch.cuda.is_available(), "GPU tests need a B200"
    return fs


def _dev():
    return torch.device("cuda", 0)


def _head(V, D, B, w_std=0.05, seed=0):
    from flashsampling_b200.testing import gaussian_head

    w, h = gaussian_head(V, D, B, w_std, seed)
    return w, h


def _check_indices(ids_gpu, logits_cpu, temperature, noise_cpu, label, vals_gpu=None, min_decisive=0.75):
    want, decisive, ymax = O.gumbel_argmax(logits_cpu, temperature, noise_cpu, rel_gap=REL_GAP)
    got = ids_gpu.cpu()
    assert got.shape == want.shape, (label, got.shape, want.shape)
    bad = (got != want) & decisive
    assert not bad.any(), f"{label}: {int(bad.sum())} decisive draws differ, e.g. {bad.nonzero()[:4].tolist()}"
    assert decisive.float().mean() >= min_decisive, f"{label}: too few decisive draws to mean anything"
    if vals_gpu is not None:
        torch.testing.assert_close(vals_gpu.cpu()[decisive], ymax[decisive], atol=2e-3, rtol=2e-4)
    return int(decisive.sum())


@pytest.mark.parametrize("kernel", ["gemv", "mma"])
@pytest.mark.parametrize("nh", [1, 2])
@pytest.mark.parametrize("V", [100, 200, 256])
def test_return_logits_matches_fp32_matmul(fs, kernel, V, nh):
    """tests/test_core.py:197-215 of the reference, for both kernels."""
    from flashsampling_b200.testing import make_synthetic_inputs

    inp = make_synthetic_inputs(vocab_size=V, n_hidden_states=nh, device=_dev())
    ids, logits = fs.fused_mm_sample_triton(
        weights=inp.weights, hidden_states=inp.hidden_states, num_samples=1,
        temperature=torch.tensor(1.0, device=_dev()), seed=0, return_logits=True, kernel=kernel,
    )
    assert fs.last_path() == kernel
    ref = inp.hidden_states.float() @ inp.weights.float().T
    assert logits.shape == ref.shape
    torch.testing.assert_close(logits, ref, atol=1e-4, rtol=1e-4)
    assert ids.shape == (nh, 1) and ids.dtype == torch.int64
    fs.check_status()


@pytest.mark.parametrize("kernel", ["gemv", "mma"])
@pytest.mark.parametrize("nh", [1, 2])
@pytest.mark.parametrize("V", [100, 200, 256, 512])
def test_greedy_is_argmax(fs, kernel, V, nh):
    """tests/test_core.py:218-236 of the reference."""
    from flashsampling_b200.testing import make_synthetic_inputs

    inp = make_synthetic_inputs(vocab_size=V, n_hidden_states=nh, device=_dev())
    ids = fs.fused_mm_sample_triton(
        weights=inp.weights, hidden_states=inp.hidden_states, num_samples=1,
        temperature=torch.empty((), device=_dev()), seed=0, greedy_sampling=True, kernel=kernel,
    )
    ref = (inp.hidden_states.float() @ inp.weights.float().T).argmax(dim=-1)
    assert ids.shape == (nh, 1)
    torch.testing.assert_close(ids[:, 0], ref)
    fs.check_status()


@pytest.mark.parametrize("V,D", [(128, 264), (129, 264), (512, 72), (262208, 64)])
def test_greedy_and_logits_over_ragged_batches(fs, V, D):
    """Deterministic modes over the ragged grid of batch sizes (one below, at and above every tile and
    kernel boundary) and vocabularies (128, 129, 512, and 262208 = 2048 * 128 + 64)."""
    for B in (1, 2, 3, 15, 16, 17, 63, 64, 65, 128, 129, 256):
        w, h = _head(V, D, B, w_std=1.0 / np.sqrt(D), seed=B)
        ref = O.logits_fp32(w, h)
        ids, logits = fs.fused_mm_sample(w.to(_dev()), h.to(_dev()), 1, torch.empty((), device=_dev()), seed=0,
                                         greedy_sampling=True, return_logits=True)
        torch.testing.assert_close(logits.cpu(), ref, atol=1e-4, rtol=1e-4)
        top2 = ref.topk(2, dim=-1).values
        clear = (top2[:, 0] - top2[:, 1]) > 1e-3 * top2[:, 0].abs()
        assert clear.float().mean() > 0.9
        assert torch.equal(ids.cpu()[clear, 0], ref.argmax(-1)[clear]), (V, D, B)
    fs.check_status()


GEMV_SHAPES = [  # V, D, B, S
    (100, 16, 1, 1), (129, 72, 2, 3), (1000, 256, 3, 2), (4097, 520, 4, 1), (5000, 1024, 5, 1),
    (6151, 264, 8, 4), (33, 8, 7, 1), (20000, 4096, 4, 2), (18992, 4096, 1, 1), (9000, 768, 5, 1), (5, 8, 3, 2),
]
MMA_SHAPES = [
    (5, 8, 3, 2), (100, 16, 1, 1), (129, 72, 2, 3), (1000, 256, 15, 2), (4097, 520, 16, 1), (5000, 1024, 17, 1),
    (6151, 264, 63, 2), (3000, 64, 64, 1), (2049, 128, 65, 1), (33, 8, 128, 1), (4500, 200, 129, 2),
    (9000, 512, 256, 1), (70000, 320, 33, 1), (50000, 4096, 8, 1),
    (3000, 64, 300, 2), (2000, 128, 513, 1),  # more than 256 rows: consecutive launches over blocks of 256 rows
    (40000, 512, 256, 1), (70000, 320, 200, 2),  # CTA-pair kernel (cta_group::2): more than 128 rows, large vocabulary
    (18992, 4096, 64, 1), (16032, 2048, 8, 1), (18992, 1024, 130, 1),  # shard-sized: tiles of two heights, several K slabs per stage
]


@pytest.mark.parametrize("shape", GEMV_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_external_noise_parity_gemv(fs, shape):
    _external_noise_case(fs, shape, "gemv")


@pytest.mark.parametrize("shape", MMA_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_external_noise_parity_mma(fs, shape):
    _external_noise_case(fs, shape, "mma")


def _external_noise_case(fs, shape, kernel):
    V, D, B, S = shape
    w, h = _head(V, D, B, w_std=1.0 / np.sqrt(D), seed=V + B)
    g = torch.Generator().manual_seed(1 + S)
    u = torch.rand(S, B, V, generator=g).clamp_min(1e-30)
    noise = O.gumbel_from_uniform(u)
    temp = torch.rand(B, generator=g) * 1.2 + 0.4  # per-row temperatures
    ids, vals = fs.fused_mm_sample(
        w.to(_dev()), h.to(_dev()), S, temp.to(_dev()), seed=0, noise=noise.to(_dev()), kernel=kernel,
        return_values=True,
    )
    assert fs.last_path() == kernel
    fs.check_status()
    _check_indices(ids, O.logits_fp32(w, h), temp, noise, f"{kernel} {shape}", vals)


@pytest.mark.parametrize("kernel,B", [("gemv", 1), ("gemv", 4), ("mma", 4), ("mma", 40), ("mma", 200)])
def test_seeded_draw_replays_on_cpu(fs, kernel, B):
    """The in-kernel Philox/Gumbel stream is a pure function of (seed, draw, row, global vocab id):
    the oracle regenerates it and must pick the same winners."""
    V, D, S = 3000, 128, 3
    w, h = _head(V, D, B, w_std=0.1, seed=3)
    temp = torch.tensor(0.7)
    ids = fs.fused_mm_sample(w.to(_dev()), h.to(_dev()), S, temp.to(_dev()), seed=1234, kernel=kernel)
    fs.check_status()
    noise = O.kernel_noise(1234, S, B, 0, V)
    _check_indices(ids, O.logits_fp32(w, h), 0.7, noise, f"seeded {kernel} B={B}")


def test_both_kernels_draw_the_same_ids(fs):
    V, D, B, S = 8192, 256, 4, 4
    w, h = _head(V, D, B, w_std=0.08, seed=9)
    w, h = w.to(_dev()), h.to(_dev())
    t = torch.tensor(0.9, device=_dev())
    a = fs.fused_mm_sample(w, h, S, t, seed=77, kernel="gemv")
    b = fs.fused_mm_sample(w, h, S, t, seed=77, kernel="mma")
    assert (a == b).float().mean() >= 0.9  # identical noise; only fp32 summation order differs
    c = fs.fused_mm_sample(w, h, S, t, seed=78, kernel="mma")
    assert (b != c).any()  # another seed, another draw


def test_vocab_offset_shifts_ids_and_noise(fs):
    """A vocabulary block sampled with its global offset reproduces the unsharded noise stream."""
    from flashsampling_b200 import _lib

    V, D, B, S = 4096, 128, 3, 2
    w, h = _head(V, D, B, w_std=0.1, seed=5)
    noise = O.kernel_noise(99, S, B, 0, V)
    logits = O.logits_fp32(w, h)
    for kernel, flag in (("gemv", _lib.FLAG_FORCE_GEMV), ("mma", _lib.FLAG_FORCE_MMA)):
        best_v, best_i = None, None
        for lo, hi in ((0, 1001), (1001, 2048), (2048, 4096)):  # 1001: a block that does not start on a multiple of 4
            ws = w[lo:hi].contiguous().to(_dev())
            out = torch.empty((B, S), dtype=torch.int64, device=_dev())
            val = torch.empty((B, S), dtype=torch.float32, device=_dev())
            wsz = _lib.query_workspace(hi - lo, D, B, S)
            ws_buf = torch.zeros(wsz, dtype=torch.uint8, device=_dev())  # zeroed once, as the header asks
            t = torch.tensor([0.8], device=_dev())
            hd = h.to(_dev())
            rc = _lib.load().fmms_sample(
                ws.data_ptr(), hd.data_ptr(), t.data_ptr(), 0, hi - lo, D, B, S, 99, lo, flag, None, 0, None,
                out.data_ptr(), val.data_ptr(), ws_buf.data_ptr(), wsz, None,
                torch.cuda.current_stream().cuda_stream,
            )
            assert rc == 0
            torch.cuda.synchronize()
            assert int(out.min()) >= lo and int(out.max()) < hi
            if best_v is None:
                best_v, best_i = val.cpu(), out.cpu()
            else:
                take = val.cpu() > best_v
                best_i = torch.where(take, out.cpu(), best_i)
                best_v = torch.where(take, val.cpu(), best_v)
        _check_indices(best_i, logits, 0.8, noise, f"sharded {kernel}")


def test_qwen_head_full_size_external_noise(fs):
    """The headline benchmark shape (Qwen3-8B head: V=151936, d=4096, T=0.7) at B=4 (weight-streaming kernel) and B=64
    (tensor-core kernel) against the fp32 CPU oracle with the same noise."""
    V, D = 151936, 4096
    w, h = _head(V, D, 64, w_std=0.02, seed=0)
    wd = w.to(_dev())
    logits = O.logits_fp32(w, h)
    g = torch.Generator().manual_seed(1)
    noise = O.gumbel_from_uniform(torch.rand(64, V, generator=g).clamp_min(1e-30))
    t = torch.tensor(0.7, device=_dev())
    ids = fs.fused_mm_sample(wd, h.to(_dev()), 1, t, seed=0, noise=noise.to(_dev()))
    assert fs.last_path() == "mma"
    _check_indices(ids, logits, 0.7, noise, "qwen B=64")
    ids4 = fs.fused_mm_sample(wd, h[:4].contiguous().to(_dev()), 1, t, seed=0, noise=noise[:4].contiguous().to(_dev()),
                              kernel="gemv")
    _check_indices(ids4, logits[:4], 0.7, noise[:4], "qwen B=4")
    ids2 = fs.fused_mm_sample(wd, h[:2].contiguous().to(_dev()), 1, t, seed=0, noise=noise[:2].contiguous().to(_dev()))
    assert fs.last_path() == "gemv"
    _check_indices(ids2, logits[:2], 0.7, noise[:2], "qwen B=2", min_decisive=0.5)
    # seeded full-size draws: the two kernels see the same noise stream
    a = fs.fused_mm_sample(wd, h[:4].contiguous().to(_dev()), 1, t, seed=5, kernel="gemv")
    b = fs.fused_mm_sample(wd, h[:4].contiguous().to(_dev()), 1, t, seed=5, kernel="mma")
    assert torch.equal(a, b)
    fs.check_status()


def test_two_stage_mode_gives_the_same_ids(fs):
    """FMMS_FLAG_TWO_STAGE: winners decoded by a separate second-stage kernel (the reference's
    stage 2) instead of the last CTA of the sampling kernel."""
    for kernel, (V, D, B, S) in (("gemv", (5000, 256, 3, 2)), ("mma", (9000, 264, 70, 3))):
        w, h = _head(V, D, B, w_std=0.08, seed=4)
        w, h = w.to(_dev()), h.to(_dev())
        t = torch.tensor(0.9, device=_dev())
        a = fs.fused_mm_sample(w, h, S, t, seed=31, kernel=kernel)
        b = fs.fused_mm_sample(w, h, S, t, seed=31, kernel=kernel, two_stage=True)
        c = fs.fused_mm_sample(w, h, S, t, seed=31, kernel=kernel)
        assert torch.equal(a, b) and torch.equal(a, c)
    fs.check_status()


@pytest.mark.parametrize("kernel,B", [("gemv", 4), ("mma", 48), ("mma", 200)])
def test_rows_with_zero_temperature_are_greedy(fs, kernel, B):
    """Per-row temperatures: rows with T = 0 take the argmax (an engine mixes greedy and sampled
    requests in one batch); the other rows still follow their noise."""
    V, D = 6000, 256
    w, h = _head(V, D, B, w_std=0.08, seed=12)
    temp = torch.full((B,), 0.8)
    temp[::2] = 0.0
    ids = fs.fused_mm_sample(w.to(_dev()), h.to(_dev()), 2, temp.to(_dev()), seed=9, kernel=kernel)
    fs.check_status()
    logits = O.logits_fp32(w, h)
    noise = O.kernel_noise(9, 2, B, 0, V)
    noise[:, ::2, :] = 0.0
    t_eff = temp.clone()
    t_eff[::2] = 1.0
    _check_indices(ids, logits, t_eff, noise, f"mixed greedy {kernel}")
    top2 = logits.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 1e-3 * top2[:, 0].abs()
    greedy_rows = torch.arange(B)[::2]
    assert torch.equal(ids.cpu()[greedy_rows][clear[greedy_rows]][:, 0], logits.argmax(-1)[greedy_rows][clear[greedy_rows]])


def test_engine_style_sampler_adapter(fs):
    from flashsampling_b200.vllm_adapter import FMMSSampler, SamplingMetadata

    V, D, B = 5000, 256, 6
    w, h = _head(V, D, B, w_std=0.08, seed=2)
    sampler = FMMSSampler(seed=100)
    meta = SamplingMetadata(temperature=torch.tensor([0.0, 0.7, 1.0, 0.0, 1.3, 0.9], device=_dev()))
    a = sampler(w.to(_dev()), h.to(_dev()), meta)
    b = sampler(w.to(_dev()), h.to(_dev()), meta)
    assert a.dtype == torch.int32 and a.shape == (B,)
    ref = O.logits_fp32(w, h).argmax(-1)
    assert int(a[0]) == int(ref[0]) and int(a[3]) == int(ref[3]) and int(b[0]) == int(ref[0])
    greedy = sampler(w.to(_dev()), h.to(_dev()), SamplingMetadata(temperature=meta.temperature, all_greedy=True))
    assert torch.equal(greedy.cpu().long(), ref)
    fs.check_status()


@pytest.mark.parametrize("kernel,B", [("gemv", 2), ("mma", 40), ("mma", 160)])
def test_step_replays_inside_a_cuda_graph(fs, kernel, B):
    """Engines replay decode steps as CUDA graphs: a captured sampling call must give the eager ids
    on every replay (the kernels leave their workspace ready for the next launch by themselves)."""
    V, D, S = 40000, 256, 2
    w, h = _head(V, D, B, w_std=0.08, seed=6)
    w, h = w.to(_dev()), h.to(_dev())
    t = torch.tensor(0.8, device=_dev())
    eager = fs.fused_mm_sample(w, h, S, t, seed=21, kernel=kernel)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        fs.fused_mm_sample(w, h, S, t, seed=21, kernel=kernel)  # warm-up on the capture stream
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        captured = fs.fused_mm_sample(w, h, S, t, seed=21, kernel=kernel)
    for _ in range(3):
        captured.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(captured, eager)
    fs.check_status()


def test_device_seed_gives_fresh_draws_on_graph_replay(fs):
    """FMMS_FLAG_SEED_DEVICE: the seed is read from device memory, so a captured step draws new noise
    on every replay; each replay equals the eager call with that seed."""
    V, D, B = 20000, 256, 24
    w, h = _head(V, D, B, w_std=0.08, seed=8)
    w, h = w.to(_dev()), h.to(_dev())
    t = torch.tensor(1.0, device=_dev())
    seed_t = torch.tensor([100], dtype=torch.int64, device=_dev())
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        fs.fused_mm_sample(w, h, 1, t, seed=seed_t)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        seed_t += 1
        captured = fs.fused_mm_sample(w, h, 1, t, seed=seed_t)
    seen = []
    for k in range(3):
        graph.replay()
        torch.cuda.synchronize()
        want = fs.fused_mm_sample(w, h, 1, t, seed=int(seed_t.item()))
        assert torch.equal(captured, want)
        seen.append(captured.clone())
    assert not torch.equal(seen[0], seen[1]) and not torch.equal(seen[1], seen[2])
    fs.check_status()


def test_argument_errors(fs):
    w = torch.zeros(64, 16, dtype=torch.bfloat16, device=_dev())
    h = torch.zeros(2, 24, dtype=torch.bfloat16, device=_dev())
    with pytest.raises(ValueError):
        fs.fused_mm_sample(w, h, 1, torch.tensor(1.0, device=_dev()), seed=0)
    with pytest.raises(TypeError):
        fs.fused_mm_sample(w.float(), h[:, :16].float(), 1, torch.tensor(1.0, device=_dev()), seed=0)
    with pytest.raises(RuntimeError):
        fs.fused_mm_sample(w.cpu(), h.cpu(), 1, torch.tensor(1.0), seed=0)
    with pytest.raises(NotImplementedError):
        fs.get_sampler("naive-pt", w)
