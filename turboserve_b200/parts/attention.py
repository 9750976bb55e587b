"""Grouped-query attention over the paged cache: the mixer of this architecture.

Per token: ``q, k, v = x Wq^T + bq, x Wk^T + bk, x Wv^T + bv`` (one fused product; the bias
is added in fp32 by the kernel that follows), position encoding of ``q`` and ``k``, append of
``k`` and ``v`` to the request's pages, attention of every query over the keys of its own
sequence up to its position (or over the last ``window`` of them), output projection.
Formulas: ``src/turboserve/engine/model/layers.py:336-391`` (projections, views, order),
``src/turboserve/engine/model/attention.py:139-148,184-209`` (mask ``key <= ctx - q_len + i``,
GQA: kv head ``j`` serves query heads ``j*g .. j*g+g-1``).

All sizes and constants are parameters of the spec: ``num_heads``, ``num_kv_heads``,
``head_dim``, ``scale``, ``qkv_bias``, ``out_bias``, ``window`` (keys seen, itself included;
``None`` = all). With ``shares_cache`` the mixer has no key and value projections and attends
over the pages another run writes.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops.attention import decode_fusion, paged_attention
from ..ops.linear import linear
from .base import MIXERS, POSITIONS, Mixer, PagedKVNeed, ParamSpec, register_mixer
from .rope import NoPosition


class PagedAttention(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str,
                 position: PartSpec | None = None, shares_cache: bool = False) -> None:
        self.hidden_size = int(hidden_size)
        self.num_heads = int(spec["num_heads"])
        self.num_kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.scale = float(spec.get("scale", self.head_dim ** -0.5))
        self.qkv_bias = bool(spec.get("qkv_bias", False))
        self.out_bias = bool(spec.get("out_bias", False))
        window = spec.get("window")
        self.window = int(window) if window else None
        self.shares_cache = bool(shares_cache)
        self.dtype = dtype
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"num_heads ({self.num_heads}) must be a multiple of num_kv_heads ({self.num_kv_heads})")
        if self.head_dim % 16 or not 16 <= self.head_dim <= 256:
            raise ValueError(f"head_dim must be a multiple of 16 between 16 and 256, got {self.head_dim}")
        self.position = POSITIONS.get(position.kind)(position, device) if position is not None else NoPosition()
        self.position.check(self.head_dim)
        self.graph_safe = bool(self.position.graph_safe)
        self.proj_kv_heads = 0 if self.shares_cache else self.num_kv_heads
        self.qkv_width = (self.num_heads + 2 * self.proj_kv_heads) * self.head_dim
        self.qkv: torch.Tensor | None = None
        self.qkv_b: torch.Tensor | None = None
        self.out_w: torch.Tensor | None = None
        self.out_b: torch.Tensor | None = None

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(self.num_kv_heads, self.head_dim, self.window)

    def scratch_per_token(self) -> int:
        return self.qkv_width + self.num_heads * self.head_dim + self.hidden_size

    def param_specs(self) -> list[ParamSpec]:
        h, d = self.hidden_size, self.head_dim
        names = [("q_proj", self.num_heads * d)]
        if not self.shares_cache:
            names += [("k_proj", self.num_kv_heads * d), ("v_proj", self.num_kv_heads * d)]
        specs = [ParamSpec(f"{name}.weight", (width, h)) for name, width in names]
        if self.qkv_bias:
            specs += [ParamSpec(f"{name}.bias", (width,), role="bias", init="bias_normal") for name, width in names]
        specs.append(ParamSpec("o_proj.weight", (h, self.num_heads * d)))
        if self.out_bias:
            specs.append(ParamSpec("o_proj.bias", (h,), role="bias", init="bias_normal"))
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        names = ["q_proj"] if self.shares_cache else ["q_proj", "k_proj", "v_proj"]
        self.qkv = torch.cat([tensors[f"{n}.weight"] for n in names], dim=0).contiguous()
        if self.qkv_bias:
            self.qkv_b = torch.cat([tensors[f"{n}.bias"] for n in names]).contiguous()
        self.out_w = tensors["o_proj.weight"].contiguous()
        if self.out_bias:
            self.out_b = tensors["o_proj.bias"].contiguous()

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        batch = ctx.batch
        n = batch.num_tokens
        table = batch.block_tables[cache.group]
        qkv = ctx.buffer("attn.qkv", (n, self.qkv_width))
        write = cache.writes and not self.shares_cache
        # a decode step may leave bias, encoding and append to the attention kernel itself
        fusion = None if self.shares_cache else decode_fusion(
            qkv, cache.k_pages, batch, self.num_heads, self.num_kv_heads, self.head_dim, self.scale, self.qkv_b,
            self.position.fused_rotation(), write)
        # that kernel is launched as thread-block clusters, which are slow to set up ahead of time
        linear(x, self.qkv, qkv, None, n, ctx, early_trigger=fusion is None)
        if fusion is None:
            self.position.apply(qkv, self.qkv_b, self.num_heads, self.proj_kv_heads, self.head_dim, ctx, cache, write)
        attended = ctx.buffer("attn.attended", (n, self.num_heads * self.head_dim))
        paged_attention(
            qkv, attended, cache.k_pages, cache.v_pages, table, batch, self.num_heads, self.num_kv_heads,
            self.head_dim, self.window, self.scale, ctx, fusion,
        )
        out = ctx.buffer("attn.out", (n, self.hidden_size))
        linear(attended, self.out_w, out, self.out_b, n, ctx)
        return out


register_mixer("attention", PagedAttention)
