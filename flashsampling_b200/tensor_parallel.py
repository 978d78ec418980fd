"""Vocabulary-sharded tensor parallelism: the cross-rank step of the sampling path.

Replaces the reference's ``tensor_parallel_reduce.py`` (symmetric-memory workspace with
``world * num_samples * tiles * B`` candidates per rank, fan-out stores inside the Triton
kernel, host-launched barrier, inductor reduce).  Here every rank first reduces to ONE
``(value, id)`` per row and draw on its own GPU; the exchange then moves 16 bytes per row
and peer.

Two interchangeable exchanges:

* ``PeerExchange`` (default on GPUs): one small CUDA kernel per step writes the records
  into every rank's buffer over NVLink peer memory, signals epoch flags and waits
  (bounded) for the peers - no NCCL, no host barrier.  Buffers are plain ``cudaMalloc``
  memory shared through CUDA IPC handles that travel once through ``torch.distributed``.
* ``CollectiveExchange``: ``all_gather`` of values and ids through ``torch.distributed``
  (NCCL on GPUs - the measured baseline - or gloo on CPU tensors for tests) followed by
  ``reduce_gathered``.

Both give every rank the same result, equal to the unsharded draw because the kernels' noise
is keyed by global vocabulary ids.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib
from .tp_info import TPInfo

MAX_ITEMS = 32768  # rows x draws per exchange step; larger calls are exchanged in chunks


def reduce_gathered(vals: torch.Tensor, ids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Winner over the leading (rank) axis of gathered ``[world, ...]`` values and ids.

    Larger value wins; equal values resolve to the smaller id, the same order the kernels
    use, so the result does not depend on the sharding.
    """
    best = vals.max(dim=0).values
    is_best = vals == best.unsqueeze(0)
    big = torch.iinfo(torch.int64).max
    win_id = torch.where(is_best, ids, torch.full_like(ids, big)).min(dim=0).values
    return win_id, best


def combine_logprobs(
    vals: torch.Tensor, ids: torch.Tensor, logprobs: torch.Tensor, lse: torch.Tensor
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Global winners and their log-probabilities from per-shard results.

    ``vals``, ``ids``, ``logprobs`` are ``[world, B, S]``: every shard's winner, and its
    log-probability under the shard's own normaliser ``lse`` ``[world, B]``.  The global
    normaliser is the log-sum-exp of the shards' normalisers; the winning shard's
    log-probability is shifted from its own normaliser to the global one.
    """
    world = vals.shape[0]
    win_id, best = reduce_gathered(vals.reshape(world, -1), ids.reshape(world, -1))
    win_id, best = win_id.view(vals.shape[1:]), best.view(vals.shape[1:])
    owner = (ids == win_id.unsqueeze(0)) & (vals == best.unsqueeze(0))  # exactly one shard per item
    shard_logit = logprobs + lse.unsqueeze(-1)  # logit / T of each shard's winner
    win_logit = torch.where(owner, shard_logit, torch.zeros_like(shard_logit)).sum(dim=0)
    lse_global = torch.logsumexp(lse.float(), dim=0)  # [B]
    return win_id, best, win_logit - lse_global.unsqueeze(-1)


def reduce_gathered_logprobs(exchange, ids, vals, logprobs, lse):
    """all_gather of the shards' winners, log-probabilities and normalisers, then
    ``combine_logprobs``; every rank ends with the same three tensors."""
    world = exchange.tp.size
    group = getattr(exchange, "group", None)
    B, S = ids.shape
    packed = torch.cat([vals.reshape(-1), logprobs.reshape(-1), lse.reshape(-1)]).contiguous()
    g_packed = torch.empty(world * packed.numel(), dtype=packed.dtype, device=packed.device)
    g_ids = torch.empty(world * ids.numel(), dtype=ids.dtype, device=ids.device)
    dist.all_gather_into_tensor(g_packed, packed, group=group)
    dist.all_gather_into_tensor(g_ids, ids.reshape(-1).contiguous(), group=group)
    g_packed = g_packed.view(world, -1)
    n = B * S
    return combine_logprobs(
        g_packed[:, :n].reshape(world, B, S), g_ids.view(world, B, S),
        g_packed[:, n:2 * n].reshape(world, B, S), g_packed[:, 2 * n:].reshape(world, B),
    )


def shard_offset(tp: TPInfo, v_local: int, state: dict, group=None) -> int:
    """Global vocabulary id of row 0 of this rank's block of ``v_local`` rows.

    With ``tp.vocab_size`` set, the block is ``tp.shard_rows()`` (the last rank also holds the
    ``vocab_size % size`` remainder rows) and ``v_local`` must match it.  Without it the blocks
    are taken to be equal, as the reference shards them (testing.py:96-104): offset
    ``rank * v_local``.  That assumption is verified once, on the first call of an exchange -
    where all ranks are present anyway because the exchange was just created collectively - by
    gathering every rank's block size; unequal blocks raise on every rank instead of silently
    sampling with wrong ids and noise keys.
    """
    if tp.vocab_size is not None:
        begin, end = tp.shard_rows()
        if end - begin != v_local:
            raise ValueError(
                f"rank {tp.rank}: weights have {v_local} rows but its block of a {tp.vocab_size}-row "
                f"vocabulary over {tp.size} ranks has {end - begin}"
            )
        return begin
    if not state.get("equal_blocks_checked"):
        sizes: list = [None] * tp.size
        dist.all_gather_object(sizes, int(v_local), group=group)
        state["equal_blocks_checked"] = True
        if any(n != sizes[0] for n in sizes):
            raise ValueError(
                f"vocabulary blocks differ across ranks ({sizes}): pass TPInfo(rank, size, vocab_size=V) "
                "so that every rank knows where its block starts"
            )
    return tp.rank * v_local


class CollectiveExchange:
    """all_gather through torch.distributed (NCCL baseline on GPUs, gloo on CPU)."""

    def __init__(self, tp: TPInfo, device: torch.device, group=None):
        self.tp, self.device, self.group = tp, device, group
        self._offset_state: dict = {}

    def vocab_offset(self, v_local: int, tp: TPInfo | None = None) -> int:
        return shard_offset(tp or self.tp, v_local, self._offset_state, self.group)

    def reduce(self, ids: torch.Tensor, vals: torch.Tensor):
        world = self.tp.size
        n = vals.numel()
        g_vals = torch.empty(world * n, dtype=vals.dtype, device=vals.device)
        g_ids = torch.empty(world * n, dtype=ids.dtype, device=ids.device)
        dist.all_gather_into_tensor(g_vals, vals.reshape(-1).contiguous(), group=self.group)
        dist.all_gather_into_tensor(g_ids, ids.reshape(-1).contiguous(), group=self.group)
        win, best = reduce_gathered(g_vals.view(world, n), g_ids.view(world, n))
        return win.view(ids.shape), best.view(vals.shape)


class PeerExchange:
    """Exchange over NVLink peer memory (CUDA IPC buffers, epoch flags).

    ``fused = True``: the sampling kernel itself performs the exchange in its last CTA
    (``fmms_sample_tp``); ``reduce`` is the stand-alone exchange kernel, used for calls that are
    too large for the buffers and by the "p2p-unfused" mode.
    """

    fused = True

    def __init__(self, tp: TPInfo, device: torch.device, max_items: int = MAX_ITEMS):
        if device.type != "cuda":
            raise RuntimeError("PeerExchange needs CUDA devices")
        if tp.size > 8:
            raise ValueError("at most 8 ranks (one NVLink domain)")
        self.tp, self.device, self.max_items = tp, device, max_items
        self.lib = _lib.load()
        self.epoch = 0
        n = ctypes.c_size_t(0)
        _lib.check(self.lib.fmms_tp_buffer_bytes(tp.size, max_items, ctypes.byref(n)), "fmms_tp_buffer_bytes")
        self.nbytes = int(n.value)
        with torch.cuda.device(device):
            own = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(64)
            _lib.check(self.lib.fmms_tp_alloc(self.nbytes, ctypes.byref(own), handle), "fmms_tp_alloc")
            self.own = own
            handles: list = [None] * tp.size
            dist.all_gather_object(handles, bytes(handle.raw))
            ptrs = (ctypes.c_void_p * tp.size)()
            self._opened = []
            for r, h in enumerate(handles):
                if r == tp.rank:
                    ptrs[r] = own.value
                else:
                    peer = ctypes.c_void_p()
                    _lib.check(self.lib.fmms_tp_open(ctypes.create_string_buffer(h, 64), ctypes.byref(peer)),
                               f"fmms_tp_open(rank {r})")
                    ptrs[r] = peer.value
                    self._opened.append(peer)
            self.ptrs = ptrs
        dist.barrier()  # every rank has mapped every buffer before the first step
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._offset_state: dict = {}

    def vocab_offset(self, v_local: int, tp: TPInfo | None = None) -> int:
        return shard_offset(tp or self.tp, v_local, self._offset_state)

    def next_epoch(self) -> int:
        """0 = the step number lives in the exchange buffer and the kernels advance it themselves,
        so a captured step can be replayed (CUDA graphs) and host and device never disagree."""
        return 0

    def reduce(self, ids: torch.Tensor, vals: torch.Tensor):
        flat_ids, flat_vals = ids.reshape(-1), vals.reshape(-1)
        out_ids, out_vals = torch.empty_like(flat_ids), torch.empty_like(flat_vals)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        n = flat_ids.numel()
        with torch.cuda.device(self.device):
            for lo in range(0, n, self.max_items):
                cnt = min(self.max_items, n - lo)
                rc = self.lib.fmms_tp_exchange(
                    flat_ids[lo:].data_ptr(), flat_vals[lo:].data_ptr(), cnt, self.max_items, self.tp.rank,
                    self.tp.size, self.ptrs, self.next_epoch(), 0, out_ids[lo:].data_ptr(), out_vals[lo:].data_ptr(),
                    self.status.data_ptr(), stream,
                )
                _lib.check(rc, "fmms_tp_exchange")
        return out_ids.reshape(ids.shape), out_vals.reshape(vals.shape)

    def check_status(self) -> None:
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise _lib.FmmsError(code, "fmms_tp_exchange (device status word)")

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        for p in self._opened:
            self.lib.fmms_tp_close(p)
        self._opened = []
        if self.own:
            self.lib.fmms_tp_free(self.own)
            self.own = None


class _UnfusedView:
    """A PeerExchange whose exchange always runs as its own kernel after the sampling kernel."""

    fused = False

    def __init__(self, inner: PeerExchange):
        self.inner = inner
        self.max_items = inner.max_items

    def vocab_offset(self, v_local: int, tp: TPInfo | None = None) -> int:
        return self.inner.vocab_offset(v_local, tp)

    def reduce(self, ids, vals):
        return self.inner.reduce(ids, vals)

    def check_status(self) -> None:
        self.inner.check_status()


_exchanges: dict = {}


def exchange_mode() -> str:
    """FMMS_TP_EXCHANGE: "p2p" (default: exchange inside the sampling kernel), "p2p-unfused"
    (separate exchange kernel) or "nccl" (all_gather baseline)."""
    return os.environ.get("FMMS_TP_EXCHANGE", "p2p")


def get_exchange(tp: TPInfo, device: torch.device):
    """The exchange of this process for (tp, device); created collectively on first use."""
    mode = exchange_mode() if device.type == "cuda" else "nccl"
    key = (tp.rank, tp.size, str(device), mode)
    ex = _exchanges.get(key)
    if ex is None:
        if mode in ("p2p", "p2p-unfused"):
            # both peer modes share one set of buffers and one epoch counter
            ex = _exchanges.get((tp.rank, tp.size, str(device), "p2p-buffers"))
            if ex is None:
                ex = PeerExchange(tp, device)
                _exchanges[(tp.rank, tp.size, str(device), "p2p-buffers")] = ex
            if mode == "p2p-unfused":
                ex = _UnfusedView(ex)
        else:
            ex = CollectiveExchange(tp, device)
        _exchanges[key] = ex
    return ex


def close_exchanges() -> None:
    for ex in set(_exchanges.values()):
        if isinstance(ex, PeerExchange):
            ex.close()
    _exchanges.clear()
