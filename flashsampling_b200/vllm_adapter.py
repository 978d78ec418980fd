"""Sampler adapter in the shape an inference engine calls it (the caller side of the boundary).

The reference is wired into its vLLM fork through a small class that receives the LM-head weight,
the hidden states of the step and per-request sampling parameters and returns one token id per
request (findings/vllm-integration.md:205-330, ``FMMSSampler.__call__``).  This mirrors that call
without importing vLLM: per-request temperatures live in one device tensor, requests with
temperature 0 are decoded greedily by the same kernel launch (their rows skip the noise), seeds
advance per step, and nothing synchronises with the host.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .core import fused_mm_sample
from .tp_info import TP1, TPInfo


@dataclass
class SamplingMetadata:
    """The subset of an engine's per-step sampling state that this path consumes."""

    temperature: torch.Tensor  # [num_requests] fp32 on the device; 0 = greedy for that request
    all_greedy: bool = False  # every request greedy: skip temperature and noise altogether
    logprobs: bool = False  # also report ln p(sampled token) per request (the engine's `logprobs` field)


class FMMSSampler:
    """``sampler(lm_head_weight, hidden_states, metadata) -> int32 [num_requests]`` token ids.

    With ``metadata.logprobs`` the call returns ``(token ids, fp32 [num_requests] log-probabilities)``:
    the engine's ``SamplerOutput(sampled_token_ids, logprobs)`` pair
    (findings/vllm-integration.md:220), which the reference's hook leaves as ``None`` because it
    has no logits to compute it from (:99, :325).
    """

    def __init__(self, seed: int = 0, tp: TPInfo = TP1, device_seed: bool = False):
        """``device_seed=True`` keeps the step's seed in a device tensor that is advanced by a tiny
        device op before every call, so the whole call can be captured in a CUDA graph and still
        draw fresh noise on every replay."""
        self.seed = int(seed)
        self.step = 0
        self.tp = tp
        self.device_seed = device_seed
        self._seed_t = None
        if tp.size > 1 and torch.cuda.is_available():
            # The exchange buffers are created collectively (IPC handles travel through the process
            # group, cudaMalloc): do it here, at engine start-up on every rank, not inside the first
            # sampling call, which may already run under CUDA-graph capture.
            from .tensor_parallel import get_exchange

            get_exchange(tp, torch.device("cuda", torch.cuda.current_device()))

    @property
    def status(self) -> torch.Tensor:
        """The device status word (int32, one element) that a kernel sets when one of its bounded waits
        runs out - e.g. a tensor-parallel peer that is more than the wait limit late; the ids of that
        step are then -1.  Nothing on the sampling path synchronises, so the engine tests this word at
        its own synchronisation point (or calls ``flashsampling_b200.check_status()``, which raises)."""
        from .core import _status_word

        return _status_word(torch.device("cuda", torch.cuda.current_device()))

    def __call__(self, lm_head_weight: torch.Tensor, hidden_states: torch.Tensor,
                 sampling_metadata: SamplingMetadata) -> torch.Tensor:
        self.step += 1
        if self.device_seed:
            if self._seed_t is None:
                self._seed_t = torch.full((1,), self.seed, dtype=torch.int64, device=lm_head_weight.device)
            self._seed_t += 1  # enqueued on the stream (captured with the call)
            seed = self._seed_t
        else:
            seed = self.seed + self.step  # draw s of a call uses stream seed + s: one fresh stream per step
        out = fused_mm_sample(
            weights=lm_head_weight,
            hidden_states=hidden_states,
            num_samples=1,
            temperature=sampling_metadata.temperature,
            seed=seed,
            greedy_sampling=sampling_metadata.all_greedy,
            tp=self.tp,
            return_logprobs=sampling_metadata.logprobs,
        )
        if sampling_metadata.logprobs:
            ids, logprobs = out
            return ids[:, 0].to(torch.int32), logprobs[:, 0]
        return out[:, 0].to(torch.int32)
