"""RMSNorm fused with the residual sum.

``out = gain * x * rsqrt(mean(x^2) + eps)`` with ``x = residual + delta`` taken in fp32, the
statistics in fp32 and one rounding to the activation dtype at the end. The reference rounds
the normalised value to the model dtype before the gain multiply
(``src/turboserve/engine/model/layers.py:202-208``); here the product is rounded once, which
is equal in float32 and at least as close to the exact value in bfloat16.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from .base import Norm, ParamSpec, register_norm


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str) -> None:
        self.eps = float(spec["eps"])
        self.hidden_size = int(hidden_size)
        self.dtype = dtype
        self.gain: torch.Tensor | None = None

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec("weight", (self.hidden_size,), role="gain", init="one_plus_normal")]

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.gain = tensors["weight"]

    def scratch_per_token(self) -> int:
        return 0  # it writes into the block's buffer

    def forward(self, residual, delta, out, ctx):
        kernels.add_rmsnorm(residual, delta, self.gain, self.eps, out, None, ctx.batch.num_tokens)
        return out

    def forward_rows(self, residual, delta, rows, num_rows, out, ctx):
        kernels.add_rmsnorm(residual, delta, self.gain, self.eps, out, rows, num_rows)
        return out


register_norm("rms_norm", RMSNorm)
