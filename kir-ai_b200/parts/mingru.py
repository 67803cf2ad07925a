"""minGRU: a gated recurrence whose gates read only the current token.

For the mixer's input h_t: z_t = sigmoid(W_z h_t + b_z), u_t = W_x h_t + b_x, the candidate c_t = u_t + 1/2 where
u_t >= 0 and sigmoid(u_t) below, and element by element S_t = (1 - z_t) S_{t-1} + z_t c_t.  The output is
W_o (S_t * silu(W_g h_t)).  S starts at zero, is 32-bit, and is carried from token to token in the request's state
slot.  Because no gate reads S, a run of tokens is a linear scan: S_end = A S_start + B with A the product of the
(1 - z) and B the run's end state from zero, which is how prompt portions are cut into pieces that run side by side.

The three input projections are one stacked product with a 32-bit result; gates, candidate and the recurrence are
32-bit; only what the output projection reads is rounded to the runtime dtype.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Mixer, Runtime, StateNeed, WeightSpec
from .linear import Linear


class MinGRU(Mixer):
    capture_safe = True  # slots and row boundaries are read on the device; a step of single tokens walks one token
    kernels_only = True

    def __init__(self, prefix: str, hidden_size: int, width: int, names: Optional[Dict[str, str]] = None,
                 out_dtype: Optional[torch.dtype] = None):
        n = {"z": "z", "x": "x", "g": "g", "o": "o", "z_bias": "z.b", "x_bias": "x.b"}
        n.update(names or {})
        self.hidden_size, self.width, self.out_dtype = hidden_size, width, out_dtype
        self.inputs = Linear([(prefix + n["z"], width), (prefix + n["x"], width), (prefix + n["g"], width)], hidden_size)
        self.out = Linear([(prefix + n["o"], hidden_size)], width)
        self.z_bias_name, self.x_bias_name = prefix + n["z_bias"], prefix + n["x_bias"]
        self.z_bias = self.x_bias = None

    def cache_need(self) -> StateNeed:
        return StateNeed((self.width,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {**self.inputs.weight_specs(), **self.out.weight_specs(),
                self.z_bias_name: WeightSpec((self.width,), "bias"), self.x_bias_name: WeightSpec((self.width,), "bias")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.inputs.load(weights, rt)
        self.out.load(weights, rt)
        self.z_bias = weights.on_device(self.z_bias_name, torch.float32)
        self.x_bias = weights.on_device(self.x_bias_name, torch.float32)

    def forward(self, x, batch, cache, write_cache: bool = True) -> torch.Tensor:
        zxg = self.inputs.forward(x, torch.float32)
        gated = self.rt.ops.mingru(zxg, self.z_bias, self.x_bias, cache.state, batch, self.rt.dtype)
        return self.out.forward(gated, self.out_dtype)
