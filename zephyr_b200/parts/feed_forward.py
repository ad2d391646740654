"""The dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases.

Gate and up run as one product over one packed weight [2I, H], as the reference packs them at
load (src/layer/mlp.cpp:16-36); the reference puts all gate rows first, this part alternates blocks
of 8 gate rows and 8 up rows (see ``__init__``).  silu and the product are one float32
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
        gate, up = weights[p["gate_proj"]], weights[p["up_proj"]]
        # With I a multiple of 8 the rows alternate in blocks of 8 gate rows and their 8 up rows, the
        # order in which the decode kernel applies silu(gate) * up inside the product's epilogue.
        self.blocked = self.intermediate % 8 == 0
        if self.blocked:
            k = gate.shape[1]
            self.w_gate_up = torch.stack([gate.view(-1, 8, k), up.view(-1, 8, k)], dim=1).reshape(-1, k).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
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

    def as_gated_products(self) -> tuple[torch.Tensor, torch.Tensor] | None:
        return (self.w_gate_up, self.w_down) if self.blocked else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.blocked and x.shape[0] <= ops.SMALL_GEMM_ROWS and ops.gemm_small_supported(x, self.w_gate_up):
            hidden = ops.gemm_small(x, self.w_gate_up, swiglu=True)       # product and activation in one kernel
        elif (self.blocked and (x.shape[0] >= ops.GEMM_TC_MIN_ROWS or not ops.USE_LIBRARY_PRODUCTS)
              and ops.gemm_tc_supported(x, self.w_gate_up, swiglu=True)):
            hidden = ops.gemm_tc(x, self.w_gate_up, swiglu=True)          # the same for a prompt's many rows, on tcgen05
        else:
            hidden = ops.silu_mul(ops.linear(x, self.w_gate_up), blocked=self.blocked)
        return ops.linear(hidden, self.w_down)


register_feed_forward("swiglu", SwiGLU)
