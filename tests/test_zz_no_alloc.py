"""fmms_sample_static: the entry point for hosts that cannot allocate device memory.

Some embedders of this library have no way to give it a workspace: the serving process
reserved the whole GPU for its own pool at start-up, or the host is plain C without an
allocator, or device allocation is forbidden once the decode loop runs.  For them the
library carries its candidate scratch inside its own device image.  This test calls that
entry point through the C ABI and requires exactly the ids and winning values of the
regular fmms_sample() (same kernels, same noise stream: bit-equal), on two calls in a
row that share the built-in scratch, and checks that an oversized problem is refused.

Kept in a file that pytest collects last, so a run that stops at the first failure has
already been through every other test.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, fn_name, w, h, t, B, S, seed, flags, workspace=None):
    V, D = w.shape
    out = torch.full((B, S), -1, dtype=torch.int64, device=w.device)
    val = torch.full((B, S), float("nan"), dtype=torch.float32, device=w.device)
    stream = torch.cuda.current_stream().cuda_stream
    head = (w.data_ptr(), h.data_ptr(), t.data_ptr(), 0, V, D, B, S, seed, 0, flags, None, 0, None,
            out.data_ptr(), val.data_ptr())
    if fn_name == "fmms_sample":
        rc = lib.fmms_sample(*head, workspace.data_ptr(), workspace.numel(), None, stream)
    else:
        rc = lib.fmms_sample_static(*head, None, stream)
    torch.cuda.synchronize()
    return rc, out, val


def test_static_scratch_entry_point_matches_workspace_entry_point():
    from flashsampling_b200 import _lib, build
    from flashsampling_b200.testing import gaussian_head

    build.build_library()
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    t = torch.tensor([0.8], device=dev)
    # two calls in a row on the shared scratch: a small batch on the weight-streaming kernel,
    # then a larger one on the tensor-core kernel whose candidate rows overlap the first call's
    # ... then more than 256 rows (consecutive launches through the same array), then a small batch again
    cases = [(6000, 256, 3, 4, 11, _lib.FLAG_FORCE_GEMV), (9000, 512, 200, 2, 12, _lib.FLAG_FORCE_MMA),
             (5000, 128, 600, 1, 13, 0), (6000, 256, 2, 3, 14, _lib.FLAG_FORCE_GEMV)]
    for V, D, B, S, seed, flags in cases:
        w, h = gaussian_head(V, D, B, 0.06, seed=seed, device=dev)
        ws = torch.zeros(_lib.query_workspace(V, D, B, S), dtype=torch.uint8, device=dev)
        rc_a, ids_a, val_a = _call(lib, "fmms_sample", w, h, t, B, S, seed, flags, ws)
        rc_b, ids_b, val_b = _call(lib, "fmms_sample_static", w, h, t, B, S, seed, flags)
        assert rc_a == 0 and rc_b == 0, (rc_a, rc_b, _lib.strerror(rc_b))
        assert int(ids_b.min()) >= 0 and int(ids_b.max()) < V
        assert torch.equal(ids_a, ids_b)
        assert torch.equal(val_a, val_b)  # same kernels and noise: tolerance zero
    # the reset entry point (for use after a reported time-out) leaves the array usable
    assert lib.fmms_static_reset(torch.cuda.current_stream().cuda_stream) == 0
    V, D, B, S, seed, flags = cases[1]
    w, h = gaussian_head(V, D, B, 0.06, seed=seed, device=dev)
    ws = torch.zeros(_lib.query_workspace(V, D, B, S), dtype=torch.uint8, device=dev)
    _, ids_a, _ = _call(lib, "fmms_sample", w, h, t, B, S, seed, flags, ws)
    rc_b, ids_b, _ = _call(lib, "fmms_sample_static", w, h, t, B, S, seed, flags)
    assert rc_b == 0 and torch.equal(ids_a, ids_b)
    # beyond the built-in scratch: refused with its own status, nothing launched
    limit = lib.fmms_static_max_items()
    B, S = 256, limit // 256 + 1
    w, h = gaussian_head(512, 64, B, 0.1, seed=1, device=dev)
    rc, ids, _ = _call(lib, "fmms_sample_static", w, h, t, B, S, 0, 0)
    assert rc == _lib.ERR_TOO_LARGE and "scratch" in _lib.strerror(rc)
    assert int(ids.max()) == -1  # output untouched
