"""Which attention kernel runs for which dtype, head size and step shape.

* float32, or a head size the tensor-core kernels do not take: the generic kernel
  (``attention_generic.cu``), whose result for a token is bit-identical however the sequence is
  cut into steps.
* bfloat16 with ``head_dim`` in :data:`TENSOR_CORE_HEAD_DIMS`: the split-KV decode kernel when
  every request of the step brings one token (``attention_bf16.cu``); else, for head size 128,
  the TMA + tcgen05 kernel (``attention_tc.cu``), and for head size 64 the tiled ``mma.sync``
  prefill kernel (``attention_bf16.cu``). In a mixed step the requests at the end (or the head)
  of the batch that bring one token still go to the decode kernel, the rest to the tiled one.
"""

from __future__ import annotations

import torch

from . import kernels

TENSOR_CORE_HEAD_DIMS = (64, 128)


def decode_fusion(qkv: torch.Tensor, k_pages: torch.Tensor, batch, num_heads: int, num_kv_heads: int, head_dim: int,
                  scale: float, bias: torch.Tensor | None, rotation, write: bool):
    """What to hand :func:`paged_attention` as ``fusion`` so that it does the step before attention
    (bias, rotation of queries and keys, append to the cache) inside its decode kernel, or ``None``
    when this step cannot be run that way and the position encoding has to be applied first.

    ``rotation`` is ``(inv_freq, rotary_dim, factor)`` of an encoding that is a rotation of pairs.
    """
    if qkv.dtype != torch.bfloat16 or head_dim not in TENSOR_CORE_HEAD_DIMS or rotation is None:
        return None
    from . import attention_bf16

    inv_freq, rotary_dim, factor = rotation
    if not attention_bf16.can_fuse_decode(qkv, k_pages, batch, num_heads, num_kv_heads, head_dim, scale, int(rotary_dim)):
        return None
    return attention_bf16.DecodeFusion(bias, inv_freq, int(rotary_dim), float(factor), bool(write))


def paged_attention(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                    block_table: torch.Tensor, batch, num_heads: int, num_kv_heads: int, head_dim: int,
                    window: int | None, scale: float, ctx, fusion=None) -> None:
    """``fusion`` (from :func:`decode_fusion`): ``q`` is the raw q/k/v product and the kernel encodes and appends itself."""
    if q.dtype == torch.bfloat16 and head_dim in TENSOR_CORE_HEAD_DIMS:
        from . import attention_bf16

        if attention_bf16.paged_attention_bf16(q, out, k_pages, v_pages, block_table, batch, num_heads,
                                               num_kv_heads, head_dim, window, scale, ctx, fusion):
            return
    if fusion is not None:
        raise RuntimeError("a fused decode step was refused by the kernel that agreed to it")
    kernels.paged_attention_generic(q, out, k_pages, v_pages, block_table, batch.seq_of_token, batch.positions,
                                    batch.num_tokens, num_heads, num_kv_heads, head_dim, window, scale, ctx.status)
