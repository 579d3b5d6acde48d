"""Sampling: greedy and seeded temperature draws from float32 logits, on the device.

The reference samples greedily only (src/runner.ts:38-42: the first index with a strictly
greater value wins, so ties go to the lowest index; its device kernel refuses non-finite logits,
native/cuda-device.inc:97-115).  Temperature sampling is this engine's own: a row with
temperature T > 0 is drawn from softmax(logits / T) by inverse CDF at one uniform number, and that
number is a function of (seed, request id, output index) alone (``uniform_for``), so batching,
chunking, preemption and recomputation cannot change what a request generates.

``sample`` is the one place that launches the sampling kernels (csrc/sampling.cu).
"""
from __future__ import annotations

import hashlib

import torch

from .. import kernels


def uniform_for(seed: int, request_id: str, index: int) -> float:
    """The uniform number in [0, 1) that draws output token ``index`` of a request: a function of
    (seed, request id, index) alone.  24 bits, so that it is exact in float32 and below 1."""
    digest = hashlib.blake2b(f"{seed}:{request_id}:{index}".encode(), digest_size=8).digest()
    return (int.from_bytes(digest, "little") >> 40) / float(1 << 24)


def sample(logits: torch.Tensor, status: torch.Tensor, temperatures: torch.Tensor | None = None,
           uniforms: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Token ids (int32, on the device) from float32 logits [rows, vocab].

    Without ``temperatures`` every row is greedy; with them (float32 device tensors, one value per
    row, like ``uniforms``) a row is greedy where its temperature is 0 and drawn otherwise.  A
    non-finite logit sets a bit in the device ``status`` word instead of yielding a token."""
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    kernels.sample(logits, out, status, temperatures, uniforms)
    return out


__all__ = ["sample", "uniform_for"]
