"""Row-wise e4m3 quantisation of an LM-head weight (the storage format of the fp8 path).

``weight[v, :] ≈ q[v, :] * scale[v]`` with ``q`` in ``torch.float8_e4m3fn`` and
``scale[v] = max|weight[v, :]| / 448`` (448 is the largest finite e4m3 value).  The sampling
kernels quantise the hidden states the same way, per row, on the way in; this module is what a
user runs once on the weight.  Plain torch: works on CPU and CUDA tensors.
"""

from __future__ import annotations

import torch

E4M3_MAX = 448.0


def round_to_e4m3(y: torch.Tensor) -> torch.Tensor:
    """fp32 values rounded to the nearest e4m3 value, ties to the even mantissa, saturating at +-448 - the
    rounding of the CUDA conversion the kernels use for the hidden states (``torch``'s own cast resolves exact
    ties differently).  Returns fp32 holding exactly representable values."""
    a = y.float().abs()
    _, ex = torch.frexp(a)  # a = m * 2^ex, m in [0.5, 1)
    e = (ex - 1).clamp_min(-6)  # exponent of the value; below 2^-6 the format is denormal with a fixed step
    step = torch.ldexp(torch.ones_like(a), e - 3)  # three mantissa bits
    q = (torch.round(a / step) * step).clamp_max(E4M3_MAX)  # torch.round: half to even
    return torch.copysign(q, y.float())


def quantize_rows_e4m3(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``(q [R, C] float8_e4m3fn, scale [R] fp32)`` of a 2-D floating-point tensor, processed in
    blocks of rows so that a 1e9-element weight needs no fp32 copy of itself."""
    if x.ndim != 2:
        raise ValueError("expected a [rows, columns] tensor")
    q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    scale = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
    step = 8192
    for r0 in range(0, x.shape[0], step):
        blk = x[r0:r0 + step].float()
        amax = blk.abs().amax(dim=1).clamp_min(1e-12)
        # one correctly rounded fp32 division, then one fp32 multiply: the operations of the CUDA quantiser
        # (tensor / tensor on purpose: `scalar / tensor` is evaluated as reciprocal-times-scalar)
        inv = torch.full_like(amax, E4M3_MAX) / amax
        q[r0:r0 + step] = round_to_e4m3(blk * inv[:, None]).to(torch.float8_e4m3fn)  # exact: no second rounding
        scale[r0:r0 + step] = amax / torch.full_like(amax, E4M3_MAX)
    return q, scale


def dequantize_rows(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """fp32 values that the quantised rows stand for."""
    return q.float() * scale[:, None].float()
