"""The two parts that stand around the layers: ids to the residual stream, final rows to logits.

``table``: a row of a ``[vocab, hidden]`` matrix per token, upcast into the float32 residual
stream (``src/turboserve/engine/model/model.py:68-69,92``). ``linear``: ``logits = rows @ W^T``
in float32 (``:220-244``), ``W`` the head's own matrix or, tied, the embedding's.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from ..ops.linear import linear
from .base import LogitHead, ParamSpec, TokenEmbedding, register_embedding, register_head


class TableEmbedding(TokenEmbedding):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, vocab_size: int, dtype: torch.dtype, device: torch.device | str) -> None:
        self.hidden_size, self.vocab_size = int(hidden_size), int(vocab_size)
        self.table = None

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec("weight", (self.vocab_size, self.hidden_size))]

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.table = tensors["weight"].contiguous()

    def scratch_per_token(self) -> int:
        return 0  # it writes into the model's residual stream

    def forward(self, residual: torch.Tensor, ctx) -> None:
        kernels.embedding(ctx.batch.token_ids, self.table, residual, ctx.status)


class LinearHead(LogitHead):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, vocab_size: int, dtype: torch.dtype, device: torch.device | str,
                 tied: bool = False) -> None:
        self.hidden_size, self.vocab_size, self.tied = int(hidden_size), int(vocab_size), bool(tied)
        self.weight: torch.Tensor | None = None

    def param_specs(self) -> list[ParamSpec]:
        return [] if self.tied else [ParamSpec("weight", (self.vocab_size, self.hidden_size))]

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = tensors["weight"].contiguous()

    def tie(self, table: torch.Tensor) -> None:
        if tuple(table.shape) != (self.vocab_size, self.hidden_size):
            raise ValueError(f"a tied head needs a [{self.vocab_size}, {self.hidden_size}] table, got {tuple(table.shape)}")
        self.weight = table

    def scratch_per_token(self) -> int:
        return 0  # the logits are the model's buffer, sized by the rows that are wanted

    def forward(self, rows_in: torch.Tensor, logits: torch.Tensor, num_rows: int, ctx) -> None:
        linear(rows_in, self.weight, logits, None, num_rows, ctx)


register_embedding("table", TableEmbedding)
register_head("linear", LinearHead)
