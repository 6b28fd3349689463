"""Normalisation parts."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.specs import NormSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm:
    """out = v * rsqrt(mean(v^2) + eps) * weight with v = x (+ delta), everything in 32-bit
    (src/layers/rms_norm.cu:77-93).  The weight multiplies directly (no 1 + w)."""

    accepts_partials = True    # `delta` may be an ops.PartialSum: the kernel adds the k-splits as it reads
    center = False             # what a kernel that applies this norm itself needs to know beside weight and eps

    def __init__(self, spec: NormSpec, size: int):
        self.eps = float(spec.eps)
        self.size = size
        self.name = getattr(spec, "weight_name", "weight")     # '' when the tensor is named like the norm itself
        self.weight: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.size,), role="scale", init=("one_plus_normal", 0.01))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name].contiguous()

    def add_normed(self, h: torch.Tensor, y, copy_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
        """h += norm(y) * weight in place (the norm of a sublayer's OUTPUT joined with the residual add);
        returns the new h in `copy_dtype` if one is asked for."""
        return ops.rmsnorm_add(h, y, self.weight, self.eps, copy_dtype)

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, delta: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None, write_sum: bool = False) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype, delta=delta, rows=rows, write_sum=write_sum)


@register_norm("layernorm")
class LayerNorm:
    """out = (v - mean(v)) * rsqrt(mean((v - mean(v))^2) + eps) * weight with v = x (+ delta), a weight and no
    bias, everything in 32-bit.  The kernel is the one that serves models with several residual streams, run on
    one stream with unit coefficients."""

    accepts_partials = True
    center = True

    def __init__(self, spec: NormSpec, size: int):
        self.eps = float(spec.eps)
        self.size = size
        self.name = getattr(spec, "weight_name", "weight")
        self.weight: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.size,), role="scale", init=("one_plus_normal", 0.01))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name].contiguous()

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, delta=None, rows: Optional[torch.Tensor] = None,
                write_sum: bool = False) -> torch.Tensor:
        if isinstance(delta, ops.PartialSum) and delta.rounds_to is not None:
            delta = ops.as_tensor(delta)
        return ops.stream_norm(x, delta, None, None, None, self.weight, self.eps, True, out_dtype, rows=rows,
                               write_back=write_sum)
