"""Choosing the next token from logits, on the device.

Parity: runtime/engine.py:99-100 (greedy argmax on the device, one copy of the chosen
ids to the host, then a synchronisation).  Temperature sampling is added: softmax of
logits / T in float and an inverse-CDF draw whose uniform depends only on the
request's seed and on how many tokens it has sampled so far.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..ops import kernels


def sample_tokens(logits: torch.Tensor, temperature: Optional[torch.Tensor] = None, seed: Optional[torch.Tensor] = None,
                  counter: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """int32 token per row of float logits [rows, vocab]; rows with temperature <= 0 (or none given) take the argmax."""
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    return kernels.sample(logits, temperature, seed, counter, out)


def uniform(seed: int, counter: int) -> float:
    """The uniform in [0, 1) that the device sampler uses for a request's `counter`-th sampled token."""
    return kernels.uniform_host(seed, counter)


class DeviceSampler:
    """`choose(logits, requests)` of the scheduler: samples on the device, returns host ints."""

    def __init__(self, stepper):
        self.stepper = stepper

    def __call__(self, logits: torch.Tensor, requests: Sequence) -> List[int]:
        extras = self.stepper.last_extras
        if getattr(self.stepper, "last_tokens", None) is not None:
            tokens = self.stepper.last_tokens        # the step ran from a graph that samples itself
        elif extras and "temperature" in extras:
            tokens = sample_tokens(logits, extras["temperature"].view(torch.float32), extras["seed"].view(torch.int64),
                                   extras["counter"])
        else:
            tokens = sample_tokens(logits)
        return tokens.to("cpu").tolist()   # the one device-to-host read of the step; it also synchronises
