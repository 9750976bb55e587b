"""Rotary position encoding (NeoX halves): the constants; the rotation itself runs fused
with the bias add and the cache append in ``layer_ops.cu`` (``PositionEncoding.apply``).

``inv_freq[i] = 1 / theta^(2i / rotary_dim)`` in float32, ``angle = (float32(pos) / factor) *
inv_freq[i]``, the pair ``(i, i + rotary_dim / 2)`` is rotated by it, as
``src/turboserve/engine/model/layers.py:258-302`` builds its tables (``:214-222`` for the
halves). The reference casts cos and sin to the model dtype before the multiply; here angles,
cos, sin and the rotation are fp32 and the result is rounded once.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import PositionEncoding, register_position


class RotaryPosition(PositionEncoding):
    def __init__(self, spec: PartSpec, device: torch.device | str) -> None:
        self.rotary_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        self.factor = float(spec.get("factor", 1.0))
        if self.rotary_dim < 2 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be even and >= 2, got {self.rotary_dim}")
        if self.theta <= 0 or self.factor <= 0:
            raise ValueError("rope theta and factor must be positive")
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta ** exponent)).to(device)


class NoPosition(PositionEncoding):
    """No position encoding: queries and keys are used as projected (bias and append only)."""

    def __init__(self, spec: PartSpec | None = None, device: torch.device | str | None = None) -> None:
        pass


register_position("rotary", RotaryPosition)
register_position("none", NoPosition)
