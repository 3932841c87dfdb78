"""Sampling: greedy and temperature, on the device, from float32 logits.

The reference samples with ``argmax`` and one device read-back per token
(src/infurnace/sampler/greedy.py:21-22); its documents ask for a per-request random key and
counter that do not depend on batch order or slot reuse (docs/architecture.md:293-297).
Here the random number of a request's k-th token is a pure function of (seed, k), computed
on the host and handed to the kernel, which picks by inverse CDF in index order.  So a
request's tokens do not depend on what else is in the batch, on how its prompt was cut,
or on preemption.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

_M64 = (1 << 64) - 1


def _mix(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform(seed: int, counter: int) -> float:
    """A number in [0, 1) with 24 random bits (exact in float32) for draw ``counter`` of ``seed``."""
    return (_mix(_mix(seed & _M64) ^ (counter & _M64)) >> 40) / float(1 << 24)


class Sampler:
    """For callers that hold logits of their own (from ``ModelRunner.step``): the same kernel and the
    same random numbers as the engine, which samples inside ``step_and_sample`` without this class."""

    def __init__(self, kernels, device):
        self.k = kernels
        self.device = device
        self._pin = torch.device(device).type == "cuda"

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], seeds: Sequence[int],
               counters: Sequence[int]) -> List[int]:
        """One token id per row of ``logits``.  Row m uses temperatures[m] (0: greedy) and the
        random number of draw counters[m] of seeds[m]."""
        m = logits.shape[0]
        out = torch.empty(m, dtype=torch.int32, device=logits.device)
        if all(t == 0.0 for t in temperatures):
            self.k.sample(logits, None, None, out)
        else:
            host = torch.tensor([list(map(float, temperatures)),
                                 [uniform(s, c) for s, c in zip(seeds, counters)]], dtype=torch.float32)
            if self._pin:
                host = host.pin_memory()
            dev = host.to(logits.device, non_blocking=True)
            self.k.sample(logits, dev[0], dev[1], out)
        return out.tolist()
