"""A feed-forward made of small experts, of which every token uses a few.

Router logits z = W_router x in 32-bit; the ``top`` experts with the largest
logits are chosen and weighted by the softmax over the chosen logits alone;
an expert is down(act(up x)) without biases, act(z) = relu(z)^2; the result is
the weighted sum of the chosen experts' outputs.

How it runs: the experts' up matrices are stacked along the output axis and
their down matrices laid side by side along the input axis at load.  One
product gives every expert's hidden rows, one kernel applies the activation
and multiplies by the token's routing weight of the column's expert (zero for
an expert that was not chosen), and the down product then sums the chosen
experts' outputs in its own accumulation.  Nothing depends on how many tokens
an expert drew, so a step of single tokens can be captured in a graph; the
price is that every expert's rows are computed for every token, experts / top
times the arithmetic that the chosen experts alone would need.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import FeedForward, Runtime, WeightSpec
from .linear import Linear

ACTIVATIONS = ("relu2",)


class RoutedExperts(FeedForward):
    capture_safe = True
    kernels_only = True

    def __init__(self, prefix: str, hidden_size: int, expert_size: int, experts: int, top: int, *,
                 activation: str = "relu2", names: Optional[Dict[str, str]] = None,
                 out_dtype: Optional[torch.dtype] = None):
        if activation not in ACTIVATIONS:
            raise ValueError(f"unknown expert activation {activation!r}; known: {ACTIVATIONS}")
        if not 0 < top <= experts:
            raise ValueError(f"every token uses {top} of {experts} experts")
        n = {"router": "router.weight", "up": "experts.{e}.up_proj.weight", "down": "experts.{e}.down_proj.weight"}
        n.update(names or {})
        self.hidden_size, self.expert_size, self.experts, self.top = hidden_size, expert_size, experts, top
        self.activation = activation
        self.out_dtype = out_dtype
        self.router_name = prefix + n["router"]
        self.up = Linear([(prefix + n["up"].format(e=e), expert_size) for e in range(experts)], hidden_size)
        self.down = Linear([(prefix + n["down"].format(e=e), expert_size) for e in range(experts)], hidden_size,
                           side_by_side=True)
        self.router: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.router_name: WeightSpec((self.experts, self.hidden_size), "linear"),
                **self.up.weight_specs(), **self.down.weight_specs()}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.router = weights.on_device(self.router_name, torch.float32)
        self.up.load(weights, rt)
        self.down.load(weights, rt)

    def forward(self, x: torch.Tensor, batch=None) -> torch.Tensor:
        ops = self.rt.ops
        gates = ops.router_gates(x, self.router, self.top)
        hidden = self.up.forward(x)
        ops.relu2_gate_(hidden, gates, self.expert_size)
        return self.down.forward(hidden, self.out_dtype)
