"""Tensor-parallel context of the sampling path (vocabulary sharding).

Mirrors the reference's ``tp_info.py``: ``TPInfo(rank, size)`` (tp_info.py:12-28),
``TP1`` (:31) and ``run_maybe_distributed`` (:34-56).  One process drives one GPU;
``torch.distributed`` (NCCL on GPUs, gloo on CPU) is only the bootstrap.
"""

from __future__ import annotations

import os
import socket
from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


@dataclass(frozen=True)
class TPInfo:
    """Rank and size of the vocabulary-parallel group."""

    rank: int
    size: int
    # Total vocabulary (extension; the reference's record has only rank and size).  Needed only
    # when the blocks are unequal, i.e. vocab_size % size != 0: the sampler then takes the global id
    # of the local block's first row from shard_rows() instead of assuming rank * V_local.
    vocab_size: int | None = None

    def is_rank0(self) -> bool:
        return self.rank == 0

    def rank0_print(self, *args, **kwargs) -> None:
        if self.is_rank0():
            print(*args, **kwargs)

    @classmethod
    def from_world(cls, vocab_size: int | None = None) -> "TPInfo":
        return cls(rank=dist.get_rank(), size=dist.get_world_size(), vocab_size=vocab_size)

    def shard_rows(self, vocab_size: int | None = None) -> tuple[int, int]:
        """[begin, end) of this rank's contiguous vocabulary block.

        Blocks have ``vocab_size // size`` rows (testing.py:96-104); unlike the
        reference, which drops ``vocab_size % size`` trailing rows, the last
        rank also takes the remainder.
        """
        if vocab_size is None:
            vocab_size = self.vocab_size
        if vocab_size is None:
            raise ValueError("shard_rows needs the total vocabulary size")
        per = vocab_size // self.size
        begin = self.rank * per
        end = vocab_size if self.rank == self.size - 1 else begin + per
        return begin, end


TP1 = TPInfo(rank=0, size=1)


def _is_torchrun() -> bool:
    return "RANK" in os.environ and "WORLD_SIZE" in os.environ


def _find_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init_group(rank: int, world_size: int, init_method: str, local_rank: int) -> None:
    use_cuda = torch.cuda.is_available() and torch.cuda.device_count() >= world_size
    if use_cuda:
        torch.cuda.set_device(local_rank)
        dist.init_process_group(
            backend="nccl", init_method=init_method, rank=rank, world_size=world_size,
            device_id=torch.device("cuda", local_rank),
        )
    else:
        dist.init_process_group(backend="gloo", init_method=init_method, rank=rank, world_size=world_size)


def _spawn_worker(rank: int, world_size: int, port: int, fn: Callable, args: tuple) -> None:
    _init_group(rank, world_size, f"tcp://127.0.0.1:{port}", rank)
    try:
        fn(*args)
    finally:
        dist.destroy_process_group()


def run_maybe_distributed(fn: Callable, n_procs: int, *args) -> None:
    """Run ``fn(*args)`` in this process or in ``n_procs`` ranks.

    Under torchrun (RANK/WORLD_SIZE set) the process group is created from the
    environment; otherwise ``n_procs > 1`` spawns workers that rendezvous on
    127.0.0.1.  ``fn`` and ``args`` must be picklable.
    """
    if _is_torchrun():
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        _init_group(rank, world, "env://", int(os.environ.get("LOCAL_RANK", rank)))
        try:
            fn(*args)
        finally:
            dist.destroy_process_group()
    elif n_procs > 1:
        mp.spawn(_spawn_worker, args=(n_procs, _find_free_port(), fn, args), nprocs=n_procs, join=True)
    else:
        fn(*args)
