"""The prepared sampler (``get_sampler(...).prepare()``) and the host-buffer call of the C ABI.

Both must return exactly the ids of the general entry point for the same seed: they are other
routes to the same kernels."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fs():
    import flashsampling_b200 as fs
    from flashsampling_b200 import build

    build.build_library()
    return fs


def _dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("V,D,B,S,per_row", [(8192, 256, 2, 1, False), (20000, 512, 48, 1, True), (9000, 264, 200, 2, True)])
def test_prepared_sampler_equals_general_entry_point(fs, V, D, B, S, per_row):
    from flashsampling_b200.testing import gaussian_head

    w, h = gaussian_head(V, D, B, 0.08, seed=V, device=_dev())
    t = (torch.rand(B, device=_dev()) + 0.5) if per_row else torch.tensor(0.8, device=_dev())
    sampler = fs.get_sampler("fused-b200", w).prepare()
    assert isinstance(sampler, fs.PreparedSampler)
    for seed in (3, 4, 5):
        want = fs.fused_mm_sample(w, h, S, t, seed=seed)
        got = sampler.sample(weights=w, hidden_states=h, num_samples=S, temperature=t, seed=seed)
        assert torch.equal(got, want)
    # a fresh hidden-state tensor on every step, as an engine hands them over (new device addresses)
    keep = []
    for step in range(40):
        h2 = h.clone()
        keep.append(h2)
        got = sampler.sample(weights=w, hidden_states=h2, num_samples=S, temperature=t, seed=7)
        assert torch.equal(got, fs.fused_mm_sample(w, h, S, t, seed=7)), step
    # arguments outside the prepared pattern fall through to the general path with the same results
    ids, vals = sampler.sample(weights=w, hidden_states=h, num_samples=S, temperature=t, seed=9, return_values=True)
    assert torch.equal(ids, fs.fused_mm_sample(w, h, S, t, seed=9)) and vals.shape == (B, S)
    fs.check_status()


@pytest.mark.parametrize("V,D,B,S,per_row", [(8192, 256, 2, 2, False), (20000, 512, 64, 1, True)])
def test_host_buffer_call_equals_device_call(fs, V, D, B, S, per_row):
    from flashsampling_b200.testing import gaussian_head

    w, h = gaussian_head(V, D, B, 0.08, seed=V + 1, device=_dev())
    t = (torch.rand(B, device=_dev()) + 0.5) if per_row else torch.tensor([0.8], device=_dev())
    sampler = fs.get_sampler("fused-b200", w).prepare()
    h_host, t_host = h.cpu().pin_memory(), t.cpu().pin_memory()
    for seed in (11, 12):
        want = fs.fused_mm_sample(w, h, S, t, seed=seed).cpu()
        got = sampler.sample_host(h_host, S, t_host, seed=seed)
        assert got.device.type == "cpu" and got.dtype == torch.int64 and torch.equal(got, want)
    # pageable host memory works as well (the driver stages the copy)
    got = sampler.sample_host(h.cpu(), S, t.cpu(), seed=11)
    assert torch.equal(got, fs.fused_mm_sample(w, h, S, t, seed=11).cpu())
    fs.check_status()


def test_descriptor_entry_point_rejects_a_foreign_layout(fs):
    from flashsampling_b200 import _lib

    lib = _lib.load()
    c = _lib.FmmsCall()
    c.struct_bytes = ctypes.sizeof(_lib.FmmsCall) - 8  # a caller built against another header
    assert lib.fmms_run(ctypes.byref(c)) == _lib.ERR_BAD_ARG
    assert lib.fmms_run(None) == _lib.ERR_BAD_ARG
