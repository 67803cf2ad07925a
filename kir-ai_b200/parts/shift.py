"""Token shift: what a mixer reads is mixed with the row of the token before.

h_t <- h_t + (h_{t-1} - h_t) * mu, element by element, with one learned weight per column and h_{t-1} the previous
token's row as it was BEFORE this replacement (zeros before a sequence's first token).  The row of a request's last
token is part of its state: it lives in the request's slot, in 32-bit, and is what the first token of the request's
next step is mixed with.  The rows come in 32-bit (from the norm) and leave in the runtime dtype.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Part, Runtime, StateNeed, WeightSpec


class TokenShift(Part):
    capture_safe = True  # slots and row boundaries are read on the device; the slot advances once per run
    kernels_only = True

    def __init__(self, weight_name: str, width: int):
        self.weight_name, self.width = weight_name, width
        self.weight: Optional[torch.Tensor] = None

    def cache_need(self) -> StateNeed:
        return StateNeed((self.width,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.width,), "bias")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.weight = weights.on_device(self.weight_name, torch.float32)

    def forward(self, rows: torch.Tensor, batch, cache) -> torch.Tensor:
        """``rows`` [T, width] (float32); ``cache`` a StateLayerView of [slots, width]."""
        return self.rt.ops.token_shift(rows, self.weight, cache.state, batch, self.rt.dtype)

    def fused_args(self, batch, cache) -> tuple:
        """What a norm's kernel needs to run this shift itself in a step of single tokens: (mu, state, slots)."""
        return (self.weight, cache.state, batch.slots)
