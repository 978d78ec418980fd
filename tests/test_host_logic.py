"""CPU tests: the C ABI loads and exports every declared symbol, host-side planning and argument
checks (no compute call needs a GPU here), and the tensor-parallel host logic."""

import re
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol(lib):
    from flashsampling_b200 import _lib

    header = (ROOT / "include" / "fmms_b200.h").read_text()
    declared = set(re.findall(r"\b(fmms_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in the header"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/fmms_b200.h but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert lib.fmms_version() >= 1000
    assert _lib.strerror(0) == "ok" and "timed out" in _lib.strerror(1)


def test_workspace_query_and_bad_arguments(lib):
    from flashsampling_b200 import _lib

    assert _lib.query_workspace(151936, 4096, 64, 1) >= 256 + 593 * 64 * 8
    assert _lib.query_workspace(100, 16, 2, 10_000) >= 592 * 2 * 10_000 * 8
    import ctypes

    n = ctypes.c_size_t()
    assert lib.fmms_query_workspace(0, 16, 1, 1, ctypes.byref(n)) == _lib.ERR_BAD_ARG
    # argument checks come before any CUDA call, so they are testable without a GPU
    rc = lib.fmms_sample(None, None, None, 0, 10, 8, 1, 1, 0, 0, 0, None, 0, None, None, None, None, 0, None, None)
    assert rc == _lib.ERR_BAD_ARG
    rc = lib.fmms_sample_static(None, None, None, 0, 10, 8, 64, 64, 0, 0, 0, None, 0, None, None, None, None, None)
    assert rc == _lib.ERR_TOO_LARGE
    # the log-probability entry point: same checks, plus its required output and the modes it excludes
    fake = ctypes.c_void_p(4096)  # never dereferenced: the checks below fail before any CUDA call
    base = (fake, fake, fake, 0, 10, 8, 1, 1, 0, 0)
    rest = (None, 0, None, fake, None, fake, 1 << 20, None, None)
    assert lib.fmms_sample_logprobs(None, None, None, 0, 10, 8, 1, 1, 0, 0, 0, *rest, fake, None) == _lib.ERR_BAD_ARG
    assert lib.fmms_sample_logprobs(*base, 0, *rest, None, None) == _lib.ERR_BAD_ARG
    assert lib.fmms_sample_logprobs(*base, _lib.FLAG_TWO_STAGE, *rest, fake, None) == _lib.ERR_UNSUPPORTED
    assert lib.fmms_sample(*base, _lib.FLAG_LOGPROB, *rest) == _lib.ERR_BAD_ARG  # the flag needs the outputs
    # the workspace head (CTA counter and log-sum-exp scratch) is part of every size
    assert _lib.query_workspace(10, 8, 1, 1) >= 256 + (16 + 160) * 256 * 8


@pytest.mark.parametrize("V,D", [(151936, 4096), (128256, 8192), (262208, 5376), (16032, 8192), (32776, 5376), (100, 16), (513, 64)])
@pytest.mark.parametrize("B", [1, 4, 8, 16, 64, 128, 129, 256])
def test_launch_plan_covers_the_vocabulary(lib, V, D, B):
    from flashsampling_b200 import _lib

    for flags in (0, _lib.FLAG_FORCE_MMA):
        pl = _lib.plan(V, D, B, 1, flags=flags)
        assert 1 <= pl["grid"] <= 148
        # the busiest CTA's tiles cover at least its share of the vocabulary
        pair = pl["path"] == _lib.PATH_MMA and B > 128 and D % 64 == 0 and V >= 32768  # CTA pairs share each tile
        assert (pl["grid"] // 2 if pair else pl["grid"]) * pl["tiles_per_cta"] * pl["tile_rows"] >= V
        assert pl["smem_bytes"] <= 232448
        assert pl["candidate_rows"] <= 640
        if pl["path"] == _lib.PATH_MMA:
            assert pl["tile_rows"] % 16 == 0 and 16 <= pl["tile_rows"] <= 256
            assert pl["m_tiles"] == (2 if B > 128 else 1)
            # balance: the tiles of the busiest CTA stay within one granule per tile of the even share
            workers = pl["grid"] // 2 if pair else pl["grid"]
            assert pl["tiles_per_cta"] * pl["tile_rows"] < V / workers + (32 if pair else 16) * (pl["tiles_per_cta"] + 1)
        else:
            assert B <= 8 and pl["tile_rows"] == (64 if 2 <= B <= 4 else 32) and pl["stages"] >= 3


def test_plan_dispatch_rules(lib):
    from flashsampling_b200 import _lib

    assert _lib.plan(151936, 4096, 1, 1)["path"] == _lib.PATH_GEMV
    assert _lib.plan(151936, 4096, 64, 1)["path"] == _lib.PATH_MMA
    assert _lib.plan(512, 16, 1, 10_000)["path"] == _lib.PATH_MMA  # too many draws for register candidates
    assert _lib.plan(151936, 4096, 8, 4, flags=_lib.FLAG_FORCE_GEMV)["path"] == _lib.PATH_GEMV
    with pytest.raises(_lib.FmmsError):
        _lib.plan(151936, 4096, 9, 1, flags=_lib.FLAG_FORCE_GEMV)
    with pytest.raises(_lib.FmmsError):
        _lib.plan(1000, 12, 1, 1)  # D not a multiple of 8 (16-byte rows)


def test_plan_details_of_the_tensor_core_kernel(lib):
    from flashsampling_b200 import _lib

    mma = _lib.FLAG_FORCE_MMA
    # hidden-state boxes are at least 16 rows high: up to 16 rows plan alike
    assert _lib.plan(151936, 4096, 3, 1, flags=mma) == _lib.plan(151936, 4096, 16, 1, flags=mma)
    # 65..128 rows: 8 KiB of slack behind the ring leave room for a fifth stage on the Qwen head
    p128 = _lib.plan(151936, 4096, 128, 1)
    assert p128["stages"] == 5 and p128["smem_bytes"] <= 232448
    # more than 128 rows on a full-size vocabulary: CTA pairs (an even grid), on a short shard two M tiles
    assert _lib.plan(151936, 4096, 256, 1)["grid"] % 2 == 0 and _lib.plan(151936, 4096, 256, 1)["m_tiles"] == 2
    assert _lib.plan(18992, 4096, 256, 1)["m_tiles"] == 2


def test_python_entry_point_rejects_cpu_tensors_and_bad_shapes():
    import flashsampling_b200 as fs

    w = torch.zeros(64, 16, dtype=torch.bfloat16)
    h = torch.zeros(2, 16, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        fs.fused_mm_sample_triton(w, h, 1, torch.tensor(1.0), seed=0)
    with pytest.raises(NotImplementedError):
        fs.get_sampler("flashinfer:sampling_from_logits", w)
    assert {"fused-triton", "fused-b200"} <= set(fs.PROVIDERS)
    s = fs.get_sampler("fused-triton", w)
    assert s.prepare() is s


def test_reduce_gathered_prefers_value_then_lowest_id():
    from flashsampling_b200.tensor_parallel import reduce_gathered

    vals = torch.tensor([[1.0, 5.0, 2.0], [3.0, 5.0, -1.0], [3.0, 4.0, 2.0]])
    ids = torch.tensor([[10, 99, 7], [20, 50, 8], [15, 1, 3]])
    win, best = reduce_gathered(vals, ids)
    assert win.tolist() == [15, 50, 3] and best.tolist() == [3.0, 5.0, 2.0]


def test_tp_buffer_size(lib):
    import ctypes

    n = ctypes.c_size_t()
    assert lib.fmms_tp_buffer_bytes(8, 1024, ctypes.byref(n)) == 0
    # two slot parities x 8 ranks x (winner records + logit records + 256 log-sum-exp records) x 16 B, + counters
    assert n.value == 2 * 8 * (2 * 1024 + 256) * 16 + 8 * 128
    assert lib.fmms_tp_buffer_bytes(9, 1024, ctypes.byref(n)) != 0


def test_reference_import_names_resolve_through_the_shim():
    import sys

    sys.path.insert(0, str(ROOT / "flashsampling_b200" / "compat"))
    try:
        from fused_mm_sampling.core import fused_mm_sample_triton, get_sampler  # noqa: F401
        from fused_mm_sampling.testing import make_synthetic_inputs
        from fused_mm_sampling.tp_info import TP1, TPInfo

        import flashsampling_b200 as fs

        assert fused_mm_sample_triton is fs.fused_mm_sample and TP1 == TPInfo(0, 1)
        inp = make_synthetic_inputs(vocab_size=100, n_hidden_states=1, device="cpu")
        assert inp.weights.shape == (100, 16)
    finally:
        sys.path.pop(0)
        for m in [k for k in sys.modules if k.startswith("fused_mm_sampling")]:
            del sys.modules[m]


def test_header_is_plain_c_and_links_from_a_c_program(lib, tmp_path):
    """A C89-style consumer (tests/c_abi/consumer.c) compiled with gcc against the header and the
    shared library: the drop-in boundary must not need C++ or torch."""
    import shutil
    import subprocess
    from pathlib import Path

    from flashsampling_b200 import _lib

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc on this machine")
    root = Path(__file__).resolve().parent.parent
    exe = tmp_path / "consumer"
    libdir = _lib.LIB_PATH.parent
    subprocess.run(
        [gcc, "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", str(root / "include"),
         str(root / "tests" / "c_abi" / "consumer.c"), "-o", str(exe), "-L", str(libdir), "-lfmms_b200",
         f"-Wl,-rpath,{libdir}"],
        check=True, capture_output=True, text=True,
    )
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0, (res.returncode, res.stdout, res.stderr)
    assert "c-abi ok" in res.stdout
