"""Generate tests/golden/reference_topk_golden.npz from the reference's top-k/top-p merge on the CPU.

    python tests/golden/make_golden_topk.py /path/to/reference

The reference's fused top-k path (src/fused_mm_sampling/tl_fused_mm_topk.py) has a Triton kernel
that emits, per 128-row vocabulary tile, the k largest temperature-scaled logits of every
hidden-state row (sorted, with global ids), and a plain-torch second stage
``_topk_merge_and_sample`` (:76-107: global top-k, softmax, nucleus mask, multinomial) that runs
on the CPU.  This script builds the per-tile lists exactly (``torch.topk`` of each tile of known
logits), runs the reference's second stage on them with fixed seeds, and records inputs and
outputs; tests/test_oracle_golden.py holds the oracle's restatement to them.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
from make_golden import import_reference  # noqa: E402  (nvtx stub, capability patch)


def per_tile_topk(scaled_logits: torch.Tensor, top_k: int, tile: int = 128):
    """What the Triton kernel stores (:216-238): [tiles, H, k] values and global ids."""
    H, V = scaled_logits.shape
    vals, ids = [], []
    for v0 in range(0, V, tile):
        blk = scaled_logits[:, v0:v0 + tile]
        if blk.shape[1] < top_k:  # ragged last tile: the kernel pads with -inf rows
            pad = torch.full((H, top_k - blk.shape[1]), -float("inf"))
            blk = torch.cat([blk, pad], dim=1)
        v, i = blk.topk(top_k, dim=-1)
        vals.append(v)
        ids.append(i + v0)
    return torch.stack(vals), torch.stack(ids)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden_topk.py /path/to/reference")
    ref_root = sys.argv[1]
    import_reference(ref_root)
    import fused_mm_sampling.tl_fused_mm_topk as rtopk

    merge = getattr(rtopk._topk_merge_and_sample, "_torchdynamo_orig_callable", rtopk._topk_merge_and_sample)
    out: dict[str, np.ndarray] = {}
    g = torch.Generator().manual_seed(11)
    cases = [(1000, 3, 8, None, 0.8), (1000, 3, 8, 0.9, 0.8), (777, 2, 20, 0.5, 1.3), (4096, 5, 50, 0.95, 0.7)]
    for n, (V, H, k, top_p, temp) in enumerate(cases):
        logits = torch.randn(H, V, generator=g) * 2.0
        scaled = logits / temp
        tv, ti = per_tile_topk(scaled, k)
        torch.manual_seed(100 + n)
        samples = merge(tv, ti, k, top_p, 64)
        tag = f"case{n}"
        out[f"{tag}_logits"] = logits.numpy().copy()
        out[f"{tag}_params"] = np.array([V, H, k, -1.0 if top_p is None else top_p, temp, 100 + n, 64], dtype=np.float64)
        out[f"{tag}_samples"] = samples.numpy().copy()
    path = Path(__file__).resolve().parent / "reference_topk_golden.npz"
    np.savez_compressed(path, **out)
    print(path, sum(v.nbytes for v in out.values()), "bytes")


if __name__ == "__main__":
    main()
