"""RMSNorm and layer norm over the hidden dimension, fused with the residual addition before them.

``y = x * rsqrt(mean(x^2) + eps) * (w + weight_offset)`` with the statistics in float32
(thinruntime/gpu_runtime.py:13028-13039; the fused add form is the reference's
_add_rms_norm_kernel, thinruntime/triton_kernels.py:2580-2614).  ``weight_offset`` is 0
for Llama (thinruntime/model_arch.py:231-233).
"""
from __future__ import annotations

import torch

from ..kernels import api
from .base import NORMS, Delta, Norm, WeightDecl


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, dim: int, eps: float, weight_offset: float = 0.0, name: str = "weight"):
        self.dim = int(dim)
        self.eps = float(eps)
        self.weight_offset = float(weight_offset)
        self.name = name                        # what the checkpoint calls the weight, behind the part's prefix
        self.weight: torch.Tensor | None = None

    def weights(self) -> dict[str, WeightDecl]:
        return {self.name: WeightDecl((self.dim,), init="norm")}

    def bind(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.name].to(torch.float32).contiguous()

    def vectors(self) -> list[torch.Tensor]:
        return [self.weight]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, residual, delta: Delta | None, out, rows=None) -> None:
        api.add_rmsnorm(residual, None if delta is None else delta.tensor, self.weight, self.eps, out, rows, self.weight_offset)   # an empty delta is already in the stream


@NORMS.register("layernorm")
class LayerNorm(Norm):
    """``y = (x - mean(x)) / sqrt(var(x) + eps) * w (+ b)`` with the variance the mean of the squared deviations,
    statistics in float32, fused with the residual addition before it like :class:`RMSNorm`.  ``bias``: whether the
    checkpoint stores one (``bias_name``)."""

    def __init__(self, dim: int, eps: float, bias: bool = False, name: str = "weight", bias_name: str = "bias"):
        self.dim, self.eps, self.bias = int(dim), float(eps), bool(bias)
        self.name, self.bias_name = name, bias_name
        self.weight: torch.Tensor | None = None
        self.shift: torch.Tensor | None = None

    def weights(self) -> dict[str, WeightDecl]:
        out = {self.name: WeightDecl((self.dim,), init="norm")}
        if self.bias:
            out[self.bias_name] = WeightDecl((self.dim,), init="zeros")
        return out

    def bind(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.name].to(torch.float32).contiguous()
        self.shift = tensors[self.bias_name].to(torch.float32).contiguous() if self.bias else None

    def vectors(self) -> list[torch.Tensor]:
        return [self.weight] + ([self.shift] if self.shift is not None else [])

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, residual, delta: Delta | None, out, rows=None) -> None:
        api.add_layernorm(residual, None if delta is None else delta.tensor, self.weight, self.shift, self.eps, out, rows)
