"""Choosing the next token from logits: greedy and temperature.

The reference samples greedily only: arg max with ties to the lowest id
(src/metal/kernels/sampling.metal:55-60,145-149); its server refuses a
temperature other than 0 (src/server.cc:128-132).  Temperature sampling is an
addition: p = softmax(logits / T) in 32-bit, inverse CDF with one uniform per
(sampler seed, request, index of the generated token).  The uniform is a hash
of those three numbers, so what a request samples does not depend on the batch
it was in or on the order of steps.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch


@dataclass(frozen=True)
class SamplingParams:
    """``max_new_tokens`` and ``ignore_eos`` as in the reference
    (src/seq.h:59-62); ``temperature`` 0 means greedy."""

    max_new_tokens: int = 64
    ignore_eos: bool = False
    temperature: float = 0.0
    seed: int = 0


def uniform_for(seed: int, request_key: int, index: int) -> float:
    """A number in [0, 1) that depends on its three arguments only."""
    digest = hashlib.sha256(f"{seed}/{request_key}/{index}".encode()).digest()
    return (int.from_bytes(digest[:8], "little") >> 40) / float(1 << 24)


class PendingTokens:
    """Tokens that the device has chosen and is sending to the host.
    ``device_ids`` (int32, one per row) can be used on the device at once;
    ``result()`` waits for the copy and returns them as a list."""

    def __init__(self, device_ids: torch.Tensor, host: Optional[torch.Tensor], event):
        self.device_ids, self._host, self._event = device_ids, host, event
        self._list: Optional[List[int]] = None

    def result(self) -> List[int]:
        if self._list is None:
            if self._host is None:
                self._list = self.device_ids.tolist()
            else:
                self._event.synchronize()
                self._list = self._host[:self.device_ids.numel()].tolist()
        return self._list


class Sampler:
    def __init__(self, runtime):
        self.runtime = runtime
        self._out: Optional[torch.Tensor] = None
        self._host = [None, None]        # pinned arrays, taken in turn
        self._turn = 0

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               request_keys: Sequence[int], indices: Sequence[int]) -> PendingTokens:
        """One token per row of ``logits``, chosen on the device; the copy to
        the host is started and an event marks its end, so that work queued
        after this call does not hold the tokens back.  ``indices[r]`` is how
        many tokens request r has generated before this one."""
        R = logits.shape[0]
        if not (len(params) == len(request_keys) == len(indices) == R):
            raise ValueError("one SamplingParams, key and index per row of logits")
        dev = self.runtime.device
        if self._out is None or self._out.numel() < R:
            self._out = torch.empty(max(R, 64), dtype=torch.int32, device=dev)
        out = self._out[:R]
        if all(p.temperature <= 0.0 for p in params):
            self.runtime.kernels.sample(logits, None, None, out)
        else:
            temps = torch.tensor([max(0.0, float(p.temperature)) for p in params], dtype=torch.float32)
            unis = torch.tensor([uniform_for(p.seed, k, i) for p, k, i in zip(params, request_keys, indices)],
                                dtype=torch.float32)
            self.runtime.kernels.sample(logits, temps.to(dev), unis.to(dev), out)
        if dev.type != "cuda":
            return PendingTokens(out, None, None)
        self._turn ^= 1
        host = self._host[self._turn]
        if host is None or host.numel() < R:
            host = torch.empty(max(R, 64), dtype=torch.int32, pin_memory=True)
            self._host[self._turn] = host
        host[:R].copy_(out, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return PendingTokens(out, host, event)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               request_keys: Sequence[int], indices: Sequence[int]) -> List[int]:
        """``launch`` and wait: the tokens as a list."""
        return self.launch(logits, params, request_keys, indices).result()
