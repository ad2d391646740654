"""The dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases.

Gate and up run as one product over the row-concatenated weight [2I, H] (rows 0..I-1 gate), as the
reference packs them at load (src/layer/mlp.cpp:16-36).  silu and the product are one float32
pass with a single rounding; the reference rounds between them (src/layer/activation.cu:31-33).
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.spec import FeedForwardSpec
from ..kernels import ops
from ..weights.loader import ROLE_LINEAR, WeightDecl
from .base import FeedForward, register_feed_forward


class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, spec: FeedForwardSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.intermediate = int(p["intermediate_size"])
        self.w_gate_up = torch.cat([weights[p["gate_proj"]], weights[p["up_proj"]]], dim=0).contiguous()
        self.w_down = weights[p["down_proj"]]

    @staticmethod
    def weight_decls(spec: FeedForwardSpec) -> dict[str, WeightDecl]:
        p = spec.params
        hidden, inter = int(p["hidden_size"]), int(p["intermediate_size"])
        return {
            p["gate_proj"]: WeightDecl((inter, hidden), ROLE_LINEAR),
            p["up_proj"]: WeightDecl((inter, hidden), ROLE_LINEAR),
            p["down_proj"]: WeightDecl((hidden, inter), ROLE_LINEAR),
        }

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(ops.silu_mul(ops.linear(x, self.w_gate_up)), self.w_down)


register_feed_forward("swiglu", SwiGLU)
