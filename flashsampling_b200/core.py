"""Fused LM-head sampling on B200: the Python entry point.

Drop-in for the reference's ``fused_mm_sample_triton`` (src/fused_mm_sampling/
core.py:224-348) and its provider registry ``get_sampler`` (core.py:658-801):
same argument names and meaning, same return value (int64 ``[B, num_samples]``
on the inputs' device, identical on every tensor-parallel rank), errors as
Python exceptions.  The work is done by hand-written sm_100a CUDA behind the C
ABI in ``include/fmms_b200.h``; this module only validates, caches scratch
buffers and forwards raw pointers.  There is no Triton, no other backend and
no CPU path: without the CUDA library or a GPU the call raises.
"""

from __future__ import annotations

import contextlib
import ctypes
from dataclasses import dataclass
from typing import Callable, Protocol

import torch

from . import _lib
from .tp_info import TP1, TPInfo

__all__ = [
    "fused_mm_sample",
    "fused_mm_sample_triton",
    "get_sampler",
    "Sampler",
    "SimpleSampler",
    "PreparedSampler",
    "check_status",
    "last_path",
    "PROVIDERS",
]

_nullcontext = contextlib.nullcontext()
_workspaces: dict[tuple, torch.Tensor] = {}
_all_workspaces: list[torch.Tensor] = []  # also those a larger one replaced (prepared calls may still use them)
_ws_bytes: dict[tuple, int] = {}  # (B, S) -> workspace bytes (independent of V and D)
_status: dict[int, torch.Tensor] = {}


def _workspace(device: torch.device, stream_id: int, nbytes: int) -> torch.Tensor:
    key = (device.index, stream_id)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        # zeroed once: the kernels keep the head of the workspace (packed winners, CTA counter) at zero
        ws = torch.zeros(max(nbytes, 8 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
        _all_workspaces.append(ws)
    return ws


_topk_workspaces: dict[tuple, torch.Tensor] = {}


def _topk_workspace(device: torch.device, stream_id: int, v_local: int, b: int) -> torch.Tensor:
    """Scratch of the top-k path (candidate lists and the logits of the exact second pass), zeroed once."""
    key = (device.index, stream_id)
    need = _lib.query_topk_workspace(v_local, b)[0]
    ws = _topk_workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=device)
        _topk_workspaces[key] = ws
        _all_workspaces.append(ws)
    return ws


_fp8_stagings: dict[tuple, torch.Tensor] = {}


def _fp8_staging(device: torch.device, stream_id: int, d: int, b: int, s: int) -> torch.Tensor:
    """Device scratch for the quantised hidden states of the e4m3 path."""
    key = (device.index, stream_id)
    need = _lib.query_staging(d, b, s)
    st = _fp8_stagings.get(key)
    if st is None or st.numel() < need:
        st = _fp8_stagings[key] = torch.empty(need, dtype=torch.uint8, device=device)
    return st


def _status_word(device: torch.device) -> torch.Tensor:
    st = _status.get(device.index)
    if st is None:
        st = torch.zeros(1, dtype=torch.int32, device=device)
        _status[device.index] = st
    return st


def check_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if a kernel recorded a device-side time-out.

    The sampling call itself never synchronises; call this where a sync is
    acceptable (tests, benchmarks, shutdown).
    """
    devs = [device.index] if device is not None else list(_status)
    for idx in devs:
        st = _status.get(idx)
        if st is None:
            continue
        code = int(st.item())
        if code != 0:
            st.zero_()
            for ws in _all_workspaces:
                if ws.device.index == idx:
                    ws.zero_()  # an aborted kernel may have left candidates behind
            raise _lib.FmmsError(code, "fused_mm_sample (device status word)")


def last_path() -> str:
    """Kernel the most recent call dispatched to: "gemv", "mma" or "none"."""
    return {0: "none", 1: "gemv", 2: "mma"}[_lib.load().fmms_last_path()]


def fused_mm_sample(
    weights: torch.Tensor,  # [V_local, D] bf16 (may be a vocabulary shard)
    hidden_states: torch.Tensor,  # [B, D] bf16
    num_samples: int,
    temperature: torch.Tensor,  # 0-d fp32 tensor on the device, or [B] for per-row temperatures
    seed,  # int, or a 1-element int64 CUDA tensor that the kernel reads (replayable in CUDA graphs)
    greedy_sampling: bool = False,
    tp: TPInfo = TP1,
    return_logits: bool = False,
    p2p_no_overlap: bool = False,
    noise: torch.Tensor | None = None,  # [num_samples, B, V_local] or [B, V_local] fp32: replaces the generator
    kernel: str | None = None,  # None = automatic, "gemv" or "mma" forces a kernel
    return_values: bool = False,
    two_stage: bool = False,  # decode the winners in a second kernel instead of the last CTA
    return_logprobs: bool = False,  # also return ln p(sampled id) [B, num_samples] from the same pass
    top_k: int | None = None,  # sample among the k largest logits of each row only (1..64)
    top_p: float | None = None,  # with top_k: nucleus cut of the top-k softmax
    weight_scale: torch.Tensor | None = None,  # [V_local] fp32: `weights` is float8_e4m3fn with one scale per row
):
    """Sample ``num_samples`` token ids per hidden-state row from softmax(W h / T).

    Arguments follow core.py:224-234.  Extensions: ``temperature`` may hold one
    value per row; ``noise`` supplies the Gumbel noise (parity checks);
    ``kernel`` pins the kernel; ``return_values`` also returns the winning
    perturbed logits ``[B, num_samples]``; ``return_logprobs`` also returns the
    log-probability of every sampled id under softmax(W h / T) (fp32
    ``[B, num_samples]``; T = 1 for greedy rows), computed by the same pass
    from a running log-sum-exp.  ``p2p_no_overlap`` selects the
    reference's ablation in which the exchange follows the kernel; here the
    exchange always follows the local reduction, so the flag changes nothing.

    ``top_k`` / ``top_p`` restrict every row to its k largest logits and, of those, to the nucleus
    of mass ``top_p`` (the reference's ``fused_mm_topk_and_sample``, tl_fused_mm_topk.py:25-37):
    the pass collects the few candidates at or above a running bound of the k-th largest logit
    and a second small kernel sorts, filters and samples them (``csrc/fmms_topk.cuh``).

    ``weight_scale`` selects e4m3 weights (``weights`` of dtype ``torch.float8_e4m3fn``, one fp32 scale per
    vocabulary row, e.g. from ``flashsampling_b200.quant.quantize_rows_e4m3``): half the streamed bytes; the
    hidden states are quantised per row on the way in and the logits are those of the dequantised operands.

    With ``tp.size > 1`` every rank passes its own contiguous vocabulary block
    and the same ``hidden_states``, ``temperature`` and ``seed``; all ranks
    return the same global token ids, equal to the single-GPU result.
    """
    if not (weights.is_cuda and hidden_states.is_cuda):
        raise RuntimeError("fused_mm_sample requires CUDA tensors (there is no CPU path)")
    if weights.ndim != 2 or hidden_states.ndim != 2:
        raise ValueError("weights must be [V, D] and hidden_states [B, D]")
    V, D = weights.shape
    B, D2 = hidden_states.shape
    if D2 != D:
        raise ValueError(
            f"hidden_states second dimension ({D2}) must match weights second dimension ({D})"
        )
    fp8 = weight_scale is not None
    if fp8:
        if weights.dtype != torch.float8_e4m3fn or hidden_states.dtype != torch.bfloat16:
            raise TypeError("with weight_scale, weights must be float8_e4m3fn and hidden_states bfloat16")
        if weight_scale.shape != (V,) or weight_scale.dtype != torch.float32 or weight_scale.device != weights.device:
            raise ValueError(f"weight_scale must be fp32 [{V}] on the weights' device")
        if D % 16 != 0:
            raise ValueError("e4m3 weights need a hidden size that is a multiple of 16")
        if kernel == "gemv" or two_stage:
            raise ValueError("e4m3 weights run on the tensor-core kernel only")
        weight_scale = weight_scale.contiguous()
    elif weights.dtype != torch.bfloat16 or hidden_states.dtype != torch.bfloat16:
        raise TypeError("weights and hidden_states must be bfloat16")
    if not weights.is_contiguous():
        raise ValueError("weights must be contiguous")
    if num_samples < 1:
        raise ValueError("num_samples must be >= 1")
    hidden_states = hidden_states.contiguous()
    dev = weights.device
    lib = _lib.load()

    flags = 0
    temp_ptr, temp_stride = None, 0
    if greedy_sampling:
        flags |= _lib.FLAG_GREEDY
    else:
        if not isinstance(temperature, torch.Tensor):
            temperature = torch.tensor(float(temperature), dtype=torch.float32, device=dev)
        if temperature.device != dev or temperature.dtype != torch.float32:
            temperature = temperature.to(device=dev, dtype=torch.float32)
        if temperature.numel() == 1:
            temp_stride = 0
        elif temperature.numel() == B:
            temperature = temperature.reshape(B).contiguous()
            temp_stride = 1
        else:
            raise ValueError(f"temperature must have 1 or {B} elements, got {temperature.numel()}")
        temp_ptr = temperature.data_ptr()

    noise_ptr, noise_ld = None, 0
    if noise is not None and not greedy_sampling:
        if noise.ndim == 2:
            noise = noise[None]
        if noise.shape != (num_samples, B, V) or noise.dtype != torch.float32 or noise.device != dev:
            raise ValueError(f"noise must be fp32 [{num_samples}, {B}, {V}] on {dev}")
        noise = noise.contiguous()
        flags |= _lib.FLAG_EXT_NOISE
        noise_ptr, noise_ld = noise.data_ptr(), V

    logits = None
    if return_logits:
        logits = torch.empty((B, V), dtype=torch.float32, device=dev)
        flags |= _lib.FLAG_RETURN_LOGITS
    if top_p is not None and top_k is None:
        raise ValueError("top_p needs top_k (the nucleus is cut from the top-k softmax, as in the reference)")
    if top_k is not None:
        if not 1 <= int(top_k) <= 64:
            raise ValueError("top_k must be between 1 and 64")
        if tp.size > 1 or return_logits or two_stage or kernel == "gemv":
            raise ValueError("top_k is not combined with tensor parallelism, return_logits, two_stage or the gemv kernel")
    if kernel == "gemv":
        flags |= _lib.FLAG_FORCE_GEMV
    elif kernel == "mma":
        flags |= _lib.FLAG_FORCE_MMA
    elif kernel is not None:
        raise ValueError('kernel must be None, "gemv" or "mma"')
    if two_stage:
        if return_logprobs:
            raise ValueError("return_logprobs is not available with two_stage")
        flags |= _lib.FLAG_TWO_STAGE
    if isinstance(seed, torch.Tensor):
        if seed.device != dev or seed.dtype != torch.int64 or seed.numel() != 1:
            raise ValueError("a tensor seed must be one int64 element on the weights' device")
        flags |= _lib.FLAG_SEED_DEVICE
        seed_arg = seed.data_ptr()
    else:
        seed_arg = int(seed) & 0xFFFFFFFFFFFFFFFF

    v_begin = 0
    if tp.size > 1:
        from .tensor_parallel import get_exchange

        exchange = get_exchange(tp, dev)
        v_begin = exchange.vocab_offset(V, tp)
    out = torch.empty((B, num_samples), dtype=torch.int64, device=dev)
    need_vals = return_values or tp.size > 1
    vals = torch.empty((B, num_samples), dtype=torch.float32, device=dev) if need_vals else None
    logprobs = lse = None
    if return_logprobs:
        logprobs = torch.empty((B, num_samples), dtype=torch.float32, device=dev)
        lse = torch.empty((B,), dtype=torch.float32, device=dev)

    stream = torch.cuda.current_stream(dev)
    nbytes = _ws_bytes.get((B, num_samples))
    if nbytes is None:
        nbytes = _ws_bytes[(B, num_samples)] = _lib.query_workspace(V, D, B, num_samples)
    ws = _workspace(dev, stream.cuda_stream, nbytes)
    status = _status_word(dev)
    common = (
        weights.data_ptr(), hidden_states.data_ptr(), temp_ptr, temp_stride, V, D, B, num_samples,
        seed_arg, v_begin, flags, noise_ptr, noise_ld,
        logits.data_ptr() if logits is not None else None, out.data_ptr(),
        vals.data_ptr() if vals is not None else None, ws.data_ptr(), ws.numel(),
        status.data_ptr(), stream.cuda_stream,
    )
    fused_tp = tp.size > 1 and getattr(exchange, "fused", False) and B * num_samples <= exchange.max_items \
        and not two_stage and B <= 256  # larger batches run as several launches, then one exchange
    with (_nullcontext if torch.cuda.current_device() == dev.index else torch.cuda.device(dev)):
        if top_k is not None or fp8:
            # the descriptor form carries what the positional entry points have no argument for
            c = _lib.FmmsCall()
            c.struct_bytes = ctypes.sizeof(_lib.FmmsCall)
            (c.W_bf16, c.H_bf16, c.temperature, c.temp_stride, c.V_local, c.D, c.B, c.S, c.seed, c.v_global_offset,
             c.flags, c.ext_noise, c.noise_ld, c.logits_out, c.out_idx, c.out_val, c.workspace, c.workspace_bytes,
             c.status_dev, c.stream) = common
            if return_logprobs:
                c.flags |= _lib.FLAG_LOGPROB
                c.out_logprob, c.out_lse = logprobs.data_ptr(), lse.data_ptr()
            if top_k is not None:
                tws = _topk_workspace(dev, stream.cuda_stream, V, B)
                c.top_k = int(top_k)
                c.top_p = float(top_p) if top_p is not None else 0.0
                c.topk_workspace, c.topk_workspace_bytes = tws.data_ptr(), tws.numel()
            if fp8:
                staging = _fp8_staging(dev, stream.cuda_stream, D, min(B, 256), num_samples)
                c.flags |= _lib.FLAG_W_FP8
                c.w_scale = weight_scale.data_ptr()
                c.staging, c.staging_bytes = staging.data_ptr(), staging.numel()
            if fused_tp:
                c.tp_rank, c.tp_world, c.tp_max_items = tp.rank, tp.size, exchange.max_items
                c.tp_peer_buffers, c.tp_epoch = exchange.ptrs, exchange.next_epoch()
            rc = lib.fmms_run(ctypes.byref(c))
        elif return_logprobs and fused_tp:
            # one launch: winners, their logits and the shards' log-sum-exps all travel in the kernel's exchange
            c = _lib.FmmsCall()
            c.struct_bytes = ctypes.sizeof(_lib.FmmsCall)
            (c.W_bf16, c.H_bf16, c.temperature, c.temp_stride, c.V_local, c.D, c.B, c.S, c.seed, c.v_global_offset,
             c.flags, c.ext_noise, c.noise_ld, c.logits_out, c.out_idx, c.out_val, c.workspace, c.workspace_bytes,
             c.status_dev, c.stream) = common
            c.flags |= _lib.FLAG_LOGPROB
            c.out_logprob, c.out_lse = logprobs.data_ptr(), lse.data_ptr()
            c.tp_rank, c.tp_world, c.tp_max_items = tp.rank, tp.size, exchange.max_items
            c.tp_peer_buffers, c.tp_epoch = exchange.ptrs, exchange.next_epoch()
            rc = lib.fmms_run(ctypes.byref(c))
        elif return_logprobs:
            rc = lib.fmms_sample_logprobs(*common, logprobs.data_ptr(), lse.data_ptr())
        elif fused_tp:
            # one launch: the sampling kernel's last CTA runs the NVLink exchange itself
            rc = lib.fmms_sample_tp(*common, tp.rank, tp.size, exchange.max_items, exchange.ptrs,
                                    exchange.next_epoch(), 0)
        else:
            rc = lib.fmms_sample(*common)
    _lib.check(rc, "fmms_sample_tp" if fused_tp else "fmms_sample")

    if tp.size > 1 and return_logprobs and not fused_tp:
        # every rank holds its shard's winner, that winner's log-probability under the shard's
        # own normaliser, and the normaliser: gather all three and renormalise
        from .tensor_parallel import reduce_gathered_logprobs

        out, vals, logprobs = reduce_gathered_logprobs(exchange, out, vals, logprobs, lse)
    elif tp.size > 1 and not fused_tp:
        out, vals = exchange.reduce(out, vals)

    result = (out,)
    if return_logits:
        result += (logits,)
    if return_values:
        result += (vals,)
    if return_logprobs:
        result += (logprobs,)
    return result[0] if len(result) == 1 else result


# The reference's name for the same entry point (core.py:224).
fused_mm_sample_triton = fused_mm_sample


class Sampler(Protocol):
    """core.py:658-663."""

    def prepare(self) -> "Sampler": ...

    def sample(self, **kwargs) -> torch.Tensor: ...


@dataclass
class SimpleSampler:
    """core.py:666-674.  ``prepare()`` binds the sampler to its weight matrix (``PreparedSampler``)
    when one was given to ``get_sampler``."""

    fn: Callable[..., torch.Tensor]
    weights: torch.Tensor | None = None
    defaults: dict | None = None

    def prepare(self) -> "Sampler":
        if self.weights is not None and self.weights.is_cuda and self.weights.dtype == torch.bfloat16:
            return PreparedSampler(self.weights, self.fn, dict(self.defaults or {}))
        return self

    def sample(self, **kwargs) -> torch.Tensor:
        return self.fn(**kwargs)


def _raw_stream(dev_index: int) -> int:
    return torch._C._cuda_getCurrentRawStream(dev_index)


class _PreparedCall:
    """One call descriptor (``fmms_call_t``) with everything filled in that stays the same from step
    to step; ``sample`` only rewrites the hidden-state, temperature, seed and output fields."""

    __slots__ = ("c", "ref", "keep")

    def __init__(self, c: "_lib.FmmsCall", keep: tuple):
        self.c = c
        self.ref = ctypes.byref(c)
        self.keep = keep  # tensors and ctypes arrays the descriptor points into


class PreparedSampler:
    """A sampler bound to one LM-head weight (``get_sampler(provider, weights).prepare()``).

    The decode loop of an engine calls ``sample`` with the same weight, batch shape and dtype on
    every step.  Everything that does not change is therefore resolved once per (batch rows, draws,
    temperature layout, tensor-parallel group, stream): argument checks, the scratch workspace, the
    status word, the vocabulary offset of a shard, the exchange buffers, and the C call descriptor,
    which is updated in place.  A call that does not fit this pattern (noise, logits or
    log-probabilities requested, a tensor seed, another weight ...) takes the general
    ``fused_mm_sample`` path with the same results.

    ``sample_host`` is the same step for hidden states that arrive in HOST memory: one library call
    copies them in, samples and copies the ids out (``FMMS_FLAG_HOST_IO`` of the C ABI).
    """

    _FAST_KEYS = frozenset(("weights", "hidden_states", "num_samples", "temperature", "seed", "tp"))

    def __init__(self, weights: torch.Tensor, fn: Callable[..., torch.Tensor], defaults: dict):
        if not weights.is_cuda or weights.ndim != 2 or weights.dtype != torch.bfloat16 or not weights.is_contiguous():
            raise ValueError("weights must be a contiguous [V, D] bfloat16 CUDA tensor")
        self.weights = weights
        self.fn = fn
        self.defaults = defaults
        self.V, self.D = weights.shape
        self.dev = weights.device
        self.dev_index = weights.device.index if weights.device.index is not None else torch.cuda.current_device()
        self.lib = _lib.load()
        self.run = self.lib.fmms_run
        self.w_ptr = weights.data_ptr()
        # defaults that the fast path cannot honour send every call down the general path
        self.fast_ok = not any(defaults.get(k) for k in ("return_logits", "greedy_sampling"))
        self.seed_default = int(defaults.get("seed", 0))
        self._calls: dict[tuple, _PreparedCall] = {}
        self._host_calls: dict[tuple, tuple] = {}

    def prepare(self) -> "PreparedSampler":
        return self

    # ---- device tensors in, device tensor out ---------------------------------------------
    def sample(self, **kw) -> torch.Tensor:
        if self.fast_ok and self._FAST_KEYS.issuperset(kw):
            w = kw.get("weights")
            hs = kw.get("hidden_states")
            t = kw.get("temperature")
            seed = kw.get("seed", self.seed_default)
            if (
                (w is None or w is self.weights or (w.data_ptr() == self.w_ptr and w.shape == self.weights.shape))
                and type(hs) is torch.Tensor and type(t) is torch.Tensor and type(seed) is int
                and hs.dtype is torch.bfloat16 and t.dtype is torch.float32
                and hs.ndim == 2 and hs.shape[1] == self.D and hs.is_contiguous()
                and hs.device == self.dev and t.device == self.dev
                and torch._C._cuda_getDevice() == self.dev_index
            ):
                B = hs.shape[0]
                nt = t.numel()
                S = kw["num_samples"]
                tp = kw.get("tp", TP1)
                if (nt == 1 or (nt == B and t.is_contiguous())) and S >= 1 and 0 < B <= 256:
                    stream = _raw_stream(self.dev_index)
                    key = (B, S, nt != 1, tp, stream)
                    call = self._calls.get(key)
                    if call is None:
                        call = self._make_call(B, S, 1 if nt != 1 else 0, tp, stream)
                    if call is not False:
                        out = torch.empty((B, S), dtype=torch.int64, device=self.dev)
                        c = call.c
                        c.H_bf16 = hs.data_ptr()
                        c.temperature = t.data_ptr()
                        c.seed = seed & 0xFFFFFFFFFFFFFFFF
                        c.out_idx = out.data_ptr()
                        rc = self.run(call.ref)
                        if rc:
                            raise _lib.FmmsError(rc, "fmms_run")
                        return out
        return self.fn(**kw)

    def _make_call(self, B: int, S: int, temp_stride: int, tp: TPInfo, stream: int, host: bool = False):
        """Resolve the step-invariant part of a call; ``False`` marks a shape the fast path leaves to
        the general one (a tensor-parallel call that cannot use the fused exchange)."""
        c = _lib.FmmsCall()
        c.struct_bytes = ctypes.sizeof(_lib.FmmsCall)
        c.W_bf16 = self.w_ptr
        c.temp_stride = temp_stride
        c.V_local, c.D, c.B, c.S = self.V, self.D, B, S
        c.flags = 0
        keep: list = []
        if tp.size > 1:
            from .tensor_parallel import get_exchange

            exchange = get_exchange(tp, self.dev)
            if not (getattr(exchange, "fused", False) and B * S <= exchange.max_items):
                if not host:
                    self._calls[(B, S, bool(temp_stride), tp, stream)] = False
                return False
            c.v_global_offset = exchange.vocab_offset(self.V, tp)
            c.tp_rank, c.tp_world, c.tp_max_items = tp.rank, tp.size, exchange.max_items
            c.tp_peer_buffers = exchange.ptrs
            c.tp_epoch = exchange.next_epoch()
            keep.append(exchange)
        nbytes = _ws_bytes.get((B, S))
        if nbytes is None:
            nbytes = _ws_bytes[(B, S)] = _lib.query_workspace(self.V, self.D, B, S)
        ws = _workspace(self.dev, stream, nbytes)
        status = _status_word(self.dev)
        c.workspace, c.workspace_bytes = ws.data_ptr(), ws.numel()
        c.status_dev = status.data_ptr()
        c.stream = stream
        keep += [ws, status, self.weights]
        call = _PreparedCall(c, tuple(keep))
        if not host:
            self._calls[(B, S, bool(temp_stride), tp, stream)] = call
        return call

    # ---- host tensors in, host tensor out ---------------------------------------------------
    def sample_host(self, hidden_states: torch.Tensor, num_samples: int, temperature: torch.Tensor,
                    seed: int = 0, tp: TPInfo = TP1) -> torch.Tensor:
        """The step for hidden states ``[B, D]`` (bf16) and temperature(s) (fp32, one or one per
        row) in host memory - pinned memory avoids a staging copy by the driver.  One library call
        enqueues the copies to the device, the sampling kernel and the copy of the ids back, and
        waits for the stream.  Returns an int64 ``[B, num_samples]`` CPU tensor and raises if the
        kernel reported a device-side time-out.  Same ids as ``sample`` for the same seed."""
        if hidden_states.is_cuda or temperature.is_cuda:
            raise ValueError("sample_host takes CPU tensors; use sample() for CUDA tensors")
        if hidden_states.dtype != torch.bfloat16 or hidden_states.ndim != 2 or hidden_states.shape[1] != self.D:
            raise ValueError(f"hidden_states must be bfloat16 [B, {self.D}]")
        if temperature.dtype != torch.float32:
            raise TypeError("temperature must be float32")
        hs = hidden_states if hidden_states.is_contiguous() else hidden_states.contiguous()
        B = hs.shape[0]
        nt = temperature.numel()
        if nt != 1 and nt != B:
            raise ValueError(f"temperature must have 1 or {B} elements, got {nt}")
        if not 0 < B <= 256:
            raise ValueError("sample_host handles 1..256 rows per call")
        with (_nullcontext if torch._C._cuda_getDevice() == self.dev_index else torch.cuda.device(self.dev)):
            stream = _raw_stream(self.dev_index)
            key = (B, num_samples, nt != 1, tp, stream)
            entry = self._host_calls.get(key)
            if entry is None:
                call = self._make_call(B, num_samples, 1 if nt != 1 else 0, tp, stream, host=True)
                if call is False:
                    raise ValueError("this tensor-parallel call does not fit the fused exchange")
                staging = torch.empty(_lib.query_staging(self.D, B, num_samples), dtype=torch.uint8, device=self.dev)
                out_host = torch.empty((B, num_samples), dtype=torch.int64).pin_memory()
                status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
                call.c.flags |= _lib.FLAG_HOST_IO
                call.c.staging, call.c.staging_bytes = staging.data_ptr(), staging.numel()
                call.c.out_idx = out_host.data_ptr()
                call.c.status_host = status_host.data_ptr()
                call.keep += (staging, out_host, status_host)
                entry = self._host_calls[key] = (call, out_host, status_host)
            call, out_host, status_host = entry
            c = call.c
            c.H_bf16 = hs.data_ptr()
            c.temperature = temperature.data_ptr()
            c.seed = int(seed) & 0xFFFFFFFFFFFFFFFF
            rc = self.run(call.ref)
        if rc:
            raise _lib.FmmsError(rc, "fmms_run (host buffers)")
        code = int(status_host[0])
        if code:
            status_host.zero_()
            check_status(self.dev)  # clears the device word and the workspace, raises
            raise _lib.FmmsError(code, "fmms_run (device status word)")
        return out_host.clone()


PROVIDERS = (
    "fused-b200",
    "fused-topk",
    "fused-triton",
    "fused-triton-p2p-no-overlap",
    "fused-triton-ret-logits",
    "fused-triton-greedy",
)


def get_sampler(provider: str, weights: torch.Tensor) -> Sampler:
    """Provider registry restricted to the fused path (core.py:744-767).

    The reference's names for its fused kernel resolve to the CUDA
    implementation, with the same default ``seed=0``; every other provider of
    the reference (torch, FlashInfer, Helion, top-k, JL baselines) is outside
    this library and raises ``NotImplementedError``.
    """
    if provider in ("fused-b200", "fused-triton"):
        return SimpleSampler(lambda **kw: fused_mm_sample(**{"seed": 0, **kw}), weights, {"seed": 0})
    if provider == "fused-topk":
        # the reference's provider for fused_mm_topk_and_sample (core.py registry; tests/test_core.py:102-140):
        # sample(weights, hidden_states, num_samples, temperature, top_k, top_p)
        return SimpleSampler(lambda **kw: fused_mm_sample(**{"seed": 0, **kw}))
    if provider == "fused-triton-p2p-no-overlap":
        return SimpleSampler(lambda **kw: fused_mm_sample(**{"seed": 0, "p2p_no_overlap": True, **kw}), weights,
                             {"seed": 0})
    if provider == "fused-triton-ret-logits":
        return SimpleSampler(lambda **kw: fused_mm_sample(**{"seed": 0, "return_logits": True, **kw})[0], weights,
                             {"seed": 0, "return_logits": True})
    if provider == "fused-triton-greedy":
        return SimpleSampler(lambda **kw: fused_mm_sample(**{"seed": 0, "greedy_sampling": True, **kw}), weights,
                             {"seed": 0, "greedy_sampling": True})
    raise NotImplementedError(f"Unknown provider: {provider} (this library implements {PROVIDERS})")
