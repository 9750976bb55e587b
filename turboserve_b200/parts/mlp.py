"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))``.

Gate and up projections are kept as one ``[2 * intermediate, hidden]`` matrix so the step runs
one product for both (the reference runs two, ``src/turboserve/engine/model/layers.py:412-440``);
the activation and the multiply are fp32 with one rounding: in the product's epilogue for small
bfloat16 batches, else in a kernel of their own (``ops.linear.gated_linear``).
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from ..ops.linear import gated_linear, interleave_gate_up, linear
from .base import FeedForward, ParamSpec, register_feed_forward


class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str) -> None:
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(spec["intermediate_size"])
        self.activation = str(spec.get("activation", "silu"))
        if self.activation not in kernels.ACTIVATION_CODES:
            raise ValueError(f"activation {self.activation!r} is not implemented; known: {sorted(kernels.ACTIVATION_CODES)}")
        self.has_bias = bool(spec.get("bias", False))
        self.dtype = dtype
        self.gate_up: torch.Tensor | None = None
        self.gate_block = 0
        self.down: torch.Tensor | None = None
        self.gate_up_bias = None
        self.down_bias = None

    def param_specs(self) -> list[ParamSpec]:
        h, i = self.hidden_size, self.intermediate_size
        specs = [
            ParamSpec("gate_proj.weight", (i, h)),
            ParamSpec("up_proj.weight", (i, h)),
            ParamSpec("down_proj.weight", (h, i)),
        ]
        if self.has_bias:
            specs += [
                ParamSpec("gate_proj.bias", (i,), role="bias", init="bias_normal"),
                ParamSpec("up_proj.bias", (i,), role="bias", init="bias_normal"),
                ParamSpec("down_proj.bias", (h,), role="bias", init="bias_normal"),
            ]
        return specs

    def scratch_per_token(self) -> int:
        return 3 * self.intermediate_size + self.hidden_size  # gate and up, their product, the output

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.gate_up, self.gate_block = interleave_gate_up(tensors["gate_proj.weight"], tensors["up_proj.weight"])
        self.down = tensors["down_proj.weight"].contiguous()
        if self.has_bias:
            self.gate_up_bias, _ = interleave_gate_up(tensors["gate_proj.bias"], tensors["up_proj.bias"])
            self.down_bias = tensors["down_proj.bias"].contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        n = ctx.batch.num_tokens
        hidden = ctx.buffer("mlp.hidden", (n, self.intermediate_size))
        gated_linear(x, self.gate_up, hidden, self.gate_up_bias, self.activation, self.gate_block, n, ctx)
        out = ctx.buffer("mlp.out", (n, self.hidden_size))
        linear(hidden, self.down, out, self.down_bias, n, ctx)
        return out


register_feed_forward("gated_mlp", GatedMLP)
