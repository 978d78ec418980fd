"""Generate tests/golden/reference_golden.npz by running the reference itself on the CPU.

Usage (only where a checkout of the reference is available; the fixtures it
writes are committed, the reference is never needed at test time):

    python tests/golden/make_golden.py /path/to/reference

The reference package imports ``nvtx`` (absent here) and queries the CUDA
device capability at import time, so both are stubbed before the import; the
functions that are called afterwards (``sample``, ``greedy_sample``,
``bsz_h``, ``_local_reduce`` and the helpers of ``testing.py``) are plain
torch and run unmodified on the CPU.

What is recorded
* make_synthetic_inputs(V, n_hidden_states) for V in {100, 256, 512} x {1, 2}:
  weights, hidden states (bf16 bit patterns) and the exact logits;
* sample(...) token ids for fixed seeds on those inputs and on a small
  Qwen-shaped Gaussian head, plus on the benchmark's CPU-runnable configuration itself
  (V=151936, d=4096, B=4, fp32 hidden states, T=1);
* greedy_sample(...) ids, the bsz_h table, shard_weights row ranges and
  _local_reduce on random candidates.
"""

from __future__ import annotations

import sys
import types
from pathlib import Path

import numpy as np
import torch


def import_reference(ref_root: str):
    nv = types.ModuleType("nvtx")

    def annotate(*a, **k):
        if len(a) == 1 and callable(a[0]) and not k:
            return a[0]
        return lambda f: f

    nv.annotate = annotate
    sys.modules.setdefault("nvtx", nv)
    torch.cuda.get_device_capability = lambda *a, **k: (10, 0)
    sys.path.insert(0, str(Path(ref_root) / "src"))
    import fused_mm_sampling.core as core
    import fused_mm_sampling.testing as rtesting
    from fused_mm_sampling.tp_info import TPInfo

    return core, rtesting, TPInfo


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().copy()


def gaussian_head(vocab: int, hidden: int, batch: int, w_std: float, seed: int, hidden_dtype):
    """Seeded inputs shaped like an LM head (the small and the CPU-runnable benchmark configurations)."""
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(vocab, hidden, generator=g) * w_std).bfloat16()
    h = torch.randn(batch, hidden, generator=g).to(hidden_dtype)
    return w, h


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference")
    ref_root = sys.argv[1]
    core, rtesting, TPInfo = import_reference(ref_root)
    cpu = torch.device("cpu")
    out: dict[str, np.ndarray] = {}

    # --- constructive inputs of the reference's statistical tests ------------------
    for V in (100, 256, 512):
        for nh in (1, 2):
            inp = rtesting.make_synthetic_inputs(vocab_size=V, hidden_size=10, n_hidden_states=nh, device=cpu)
            tag = f"syn_V{V}_H{nh}"
            out[f"{tag}_weights_bf16"] = bf16_bits(inp.weights)
            out[f"{tag}_hidden_bf16"] = bf16_bits(inp.hidden_states)
            out[f"{tag}_logits"] = inp.logits.numpy().copy()
            temp = torch.tensor(V / 20.0)
            ids = core.sample(inp.weights, inp.hidden_states, 64, temp, seed=7)
            out[f"{tag}_sample_seed7"] = ids.numpy().copy()
            out[f"{tag}_greedy"] = core.greedy_sample(inp.weights, inp.hidden_states, 1, temp).numpy().copy()

    # --- a small Gaussian head: sample() with a scalar temperature -----------------
    w, h = gaussian_head(4096, 256, 4, 0.05, seed=11, hidden_dtype=torch.bfloat16)
    out["small_sample_seed3_T0p7"] = core.sample(w, h, 16, torch.tensor(0.7), seed=3).numpy().copy()
    out["small_w_checksum"] = np.array([w.double().sum().item(), w.double().abs().sum().item()])
    out["small_h_checksum"] = np.array([h.double().sum().item(), h.double().abs().sum().item()])

    # --- the CPU-runnable benchmark configuration: Qwen3-8B-shaped head ---------------
    w, h = gaussian_head(151936, 4096, 4, 0.02, seed=0, hidden_dtype=torch.float32)
    w32 = w.float()
    out["cfg1_sample_seed0_T1"] = core.sample(w32, h, 1, torch.tensor(1.0), seed=0).numpy().copy()
    out["cfg1_greedy"] = core.greedy_sample(w32, h, 1, torch.tensor(1.0)).numpy().copy()
    out["cfg1_w_checksum"] = np.array([w32.double().sum().item(), w32.double().abs().sum().item()])
    out["cfg1_h_checksum"] = np.array([h.double().sum().item(), h.double().abs().sum().item()])
    logits = h @ w32.T
    out["cfg1_logits_rowstats"] = torch.stack([logits.max(-1).values, logits.min(-1).values, logits.sum(-1)]).numpy().copy()
    del w, w32, logits

    # --- bsz_h table (tests/test_core.py:40-55) ------------------------------------
    hs = np.arange(1, 300)
    out["bsz_h_in"] = hs
    out["bsz_h_out"] = np.array([core.bsz_h(int(x)) for x in hs])

    # --- shard_weights row ranges (testing.py:96-104) ------------------------------
    rows = []
    for V in (100, 512, 128256, 151936, 262208):
        marker = torch.arange(V, dtype=torch.int32)[:, None].contiguous()
        for size in (1, 2, 4, 8):
            for rank in range(size):
                sh = rtesting.shard_weights(marker, TPInfo(rank=rank, size=size))
                rows.append([V, size, rank, int(sh[0, 0]), int(sh[-1, 0]) + 1])
    out["shard_rows"] = np.array(rows, dtype=np.int64)

    # --- _local_reduce (core.py:359-370), un-compiled body -------------------------
    fn = getattr(core._local_reduce, "_torchdynamo_orig_callable", None)
    if fn is None:
        raise RuntimeError("cannot reach the eager body of _local_reduce")
    g = torch.Generator().manual_seed(5)
    maxs = torch.randn(3, 9, 5, generator=g)
    maxs_idx = torch.randint(0, 10_000, (3, 9, 5), generator=g)
    samples, values = fn(maxs, maxs_idx, 1234)
    out["local_reduce_maxs"] = maxs.numpy().copy()
    out["local_reduce_maxs_idx"] = maxs_idx.numpy().copy()
    out["local_reduce_samples"] = samples.numpy().copy()
    out["local_reduce_values"] = values.numpy().copy()

    out["torch_version"] = np.array([torch.__version__])
    dst = Path(__file__).parent / "reference_golden.npz"
    np.savez_compressed(dst, **out)
    print(f"wrote {dst} ({dst.stat().st_size/1024:.1f} KiB, {len(out)} arrays)")


if __name__ == "__main__":
    main()
