"""Position encodings applied to queries and keys.

``rope_neox``: inv_freq[i] = 1 / theta^(2i/hd) for i < hd/2, angle[p, i] = p * inv_freq[i], all in
float32; cos and sin of the float32 angle; rotation of the pairs (i, i + hd/2)
(reference: src/layer/rotary_embedding.cpp:36-55, src/layer/rotary_embedding.cu:24-47).  The
tables stay float32 on the device (the reference rounds them to the model's type).

``none``: no encoding.
"""

from __future__ import annotations

import torch

from ..config.errors import ConfigError
from ..config.spec import PositionSpec
from ..kernels import ops
from .base import PositionEncoding, register_position_encoding


def rope_tables(head_dim: int, max_positions: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin, float32 [max_positions, head_dim/2], computed on the host in float32."""
    index = torch.arange(0, head_dim // 2, dtype=torch.float32)
    exponent = (2.0 * index) / torch.tensor(float(head_dim), dtype=torch.float32)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)
    angles = torch.arange(max_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(angles).contiguous(), torch.sin(angles).contiguous()


class RopeNeox(PositionEncoding):
    graph_safe = True

    kind = "rope_neox"

    def __init__(self, spec: PositionSpec, dtype: torch.dtype, device: torch.device | str):
        if spec.head_dim <= 0 or spec.head_dim % 2 != 0:
            raise ConfigError("a rotary head size must be positive and even")
        theta = float(spec.params.get("theta", 10000.0))
        if not theta > 0.0 or theta == float("inf"):
            raise ConfigError("the rotary base must be finite and positive")
        self.head_dim = spec.head_dim
        self.max_positions = spec.max_positions
        cos, sin = rope_tables(spec.head_dim, spec.max_positions, theta)
        self.cos = cos.to(device)
        self.sin = sin.to(device)

    def apply(self, x: torch.Tensor, heads: int, positions: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        return ops.rope(x, heads, self.head_dim, self.cos, self.sin, positions, status)

    def as_rotation_tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        return self.cos, self.sin


class NoPosition(PositionEncoding):
    graph_safe = True

    kind = "none"

    def __init__(self, spec: PositionSpec, dtype: torch.dtype, device: torch.device | str):
        self.head_dim = spec.head_dim
        self.max_positions = spec.max_positions

    def apply(self, x: torch.Tensor, heads: int, positions: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        return x

    def as_rotation_tables(self) -> tuple[None, None]:
        return None, None


register_position_encoding("rope_neox", RopeNeox)
register_position_encoding("none", NoPosition)
