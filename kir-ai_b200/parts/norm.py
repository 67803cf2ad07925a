"""RMSNorm and layer norm with the residual add fused in.

y = x * 1/sqrt(mean(x^2) + eps) * w, statistics in 32-bit, the scale 0 when
mean + eps is 0 (crates/llm-backend/src/core/math.rs:73-113 of the reference; the
dense model uses the plain weight, crates/llm-backend/src/core/qwen/ops/norm.rs:119-133).
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from .base import FusedNormSpec, Norm, Runtime, WeightSpec


class RMSNorm(Norm):
    capture_safe = True
    kernels_only = True

    def __init__(self, weight_name: str, width: int, eps: float):
        self.weight_name = weight_name
        self.width = width
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.width,), "norm")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.weight = weights.on_device(self.weight_name, torch.float32)

    def add_forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        return self.rt.ops.add_rmsnorm(resid, delta, self.weight, self.eps, self.rt.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.rt.ops.add_rmsnorm(x, None, self.weight, self.eps, self.rt.dtype)

    def add_normed(self, resid: torch.Tensor, y: torch.Tensor) -> Optional[torch.Tensor]:
        if y.dtype != torch.float32:
            y = y.float()
        return self.rt.ops.norm_add(resid, y, self.weight, self.eps, None if self.rt.dtype == torch.float32 else self.rt.dtype)

    def fused_spec(self) -> Optional[FusedNormSpec]:
        # the tensor-core products read and write rows in 16-byte units; KIRAI_FUSE_NORMS=0 keeps every norm a
        # kernel of its own (for comparing the two paths)
        if self.rt.dtype != torch.bfloat16 or self.width % 8 or os.environ.get("KIRAI_FUSE_NORMS", "1") == "0":
            return None
        return FusedNormSpec(self.weight, self.eps, self.width)

    def add_forward_rows(self, resid: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        """The norm of ``resid[rows] + delta[rows]`` only; the stream is left untouched."""
        out, _ = self.rt.ops.add_rmsnorm(resid, delta, self.weight, self.eps, self.rt.dtype, row_index=rows)
        return out


class LayerNorm(Norm):
    """Layer norm with a weight and no bias: y = (x - mean) / sqrt(var + eps) * w, var the mean of the squared
    deviations from the mean, statistics in 32-bit.  ``add_forward`` may also take a bias [width] of the sub-layer
    whose output it adds (``takes_delta_bias``), and can leave its rows in 32-bit for a step that goes on in 32-bit
    (``wide``: a token shift).  It is a kernel of its own: no product takes it over."""

    capture_safe = True
    kernels_only = True
    takes_delta_bias = True
    fuses_shift = True  # add_forward(shift=...) runs a token shift of single-token steps inside the norm's kernel

    def __init__(self, weight_name: str, width: int, eps: float):
        self.weight_name = weight_name
        self.width = width
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.width,), "norm")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.weight = weights.on_device(self.weight_name, torch.float32)

    def add_forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], delta_bias: Optional[torch.Tensor] = None,
                    wide: bool = False, shift: Optional[tuple] = None) -> torch.Tensor:
        return self.rt.ops.add_layernorm(resid, delta, self.weight, self.eps, self.rt.dtype, delta_bias=delta_bias, wide=wide,
                                         shift=shift)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.rt.ops.add_layernorm(x, None, self.weight, self.eps, self.rt.dtype)

    def add_forward_rows(self, resid: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        """The norm of ``resid[rows] + delta[rows]`` only; the stream is left untouched."""
        return self.rt.ops.add_layernorm(resid, delta, self.weight, self.eps, self.rt.dtype, row_index=rows)
