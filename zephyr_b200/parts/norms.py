"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, statistics in float32, the scale multiplied after
the normalisation and not as (1 + w) (reference: src/layer/normalization.cpp:10-18,
deps/ttl/src/kernels/normalization/normalization.cu:76-139)."""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.spec import NormSpec
from ..kernels import ops
from ..weights.loader import ROLE_NORM, WeightDecl
from .base import Norm, register_norm


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, spec: NormSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype):
        self.size = spec.size
        self.eps = float(spec.eps)
        self.weight = weights[spec.weight]

    @staticmethod
    def weight_decls(spec: NormSpec) -> dict[str, WeightDecl]:
        return {spec.weight: WeightDecl((spec.size,), ROLE_NORM)}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps)

    def add_forward(self, residual: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps)

    def as_rms_scale(self) -> tuple[torch.Tensor, float]:
        return self.weight, self.eps


register_norm("rmsnorm", RMSNorm)
