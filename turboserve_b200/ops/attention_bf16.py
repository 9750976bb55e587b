"""Python face of ``attention_bf16.cu``: tensor-core paged attention for bfloat16.

Rules (explicit; what they refuse goes to the generic kernel, see ``ops/attention.py``):
head size 64 or 128, page size a power of two, at most 64 query heads per kv head. A step with
prompts in it and head size 128 runs the TMA + tcgen05 kernel of ``attention_tc.cu`` when that
takes the shape (``attention_tc.supports``), else the tiled ``mma.sync`` kernel here. A decode
step (at most 16 query heads per kv head) with pages of at least 4 tokens runs the TMA-fed
decode kernel, else the register-fed one; it is cut along the keys into
``num_splits`` parts, a function of the number of tokens, kv heads and SMs only, so the same
launch shape serves a captured graph at any context length.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import attention_tc, kernels
from .kernels import KernelError, _check, _fn, _need, _ptr, _stream
from .skinny import num_sms

MAX_SPLITS = 32
TMA_DECODE = os.environ.get("TURBOSERVE_B200_DECODE_TMA", "1") != "0"
"""Decode steps fetch keys and values by TMA (``flash_decode_tma``); 0 keeps the register-fed kernel."""
CLUSTER_MAX_SPLITS = 8
"""Up to this many splits are the blocks of one thread-block cluster and are joined over
distributed shared memory, with no scratch and no second kernel."""


def available() -> bool:
    return True


def supports(head_dim: int, page_size: int, group: int, decode: bool) -> bool:
    if head_dim not in (64, 128) or page_size & (page_size - 1) or group > 64:
        return False
    return group <= 16 if decode else True


def decode_splits(num_tokens: int, num_kv_heads: int, sms: int) -> int:
    """Splits along the keys so that about two blocks per SM are in flight."""
    blocks = max(1, num_tokens * num_kv_heads)
    splits = max(1, min(MAX_SPLITS, (2 * sms) // blocks))
    # a little fewer splits that are joined inside a cluster beat more that need the join kernel
    return CLUSTER_MAX_SPLITS if CLUSTER_MAX_SPLITS < splits <= 2 * CLUSTER_MAX_SPLITS else splits


def _common(q, out, k_pages, v_pages, block_table, num_heads, num_kv_heads, head_dim):
    _need(q, torch.bfloat16, "q"); _need(out, torch.bfloat16, "out")
    _need(k_pages, torch.bfloat16, "k_pages"); _need(v_pages, torch.bfloat16, "v_pages")
    _need(block_table, torch.int32, "block_table")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or tuple(k_pages.shape[2:]) != (num_kv_heads, head_dim):
        raise KernelError("flash attention: pages must be contiguous [pages, page_size, kv_heads, head_dim]")
    if q.shape[1] < num_heads * head_dim or out.shape[1] < num_heads * head_dim:
        raise KernelError("flash attention: q or out is narrower than its heads")


def flash_prefill(q, out, k_pages, v_pages, block_table, query_start_loc, context_lens, num_seqs, num_tokens,
                  num_heads, num_kv_heads, head_dim, window, scale) -> None:
    """Attention for a step with portions of prompts in it (any mix of query lengths)."""
    _common(q, out, k_pages, v_pages, block_table, num_heads, num_kv_heads, head_dim)
    _need(query_start_loc, torch.int32, "query_start_loc"); _need(context_lens, torch.int32, "context_lens")
    tokens_per_tile = max(1, 64 // (num_heads // num_kv_heads))
    max_tiles = -(-num_tokens // tokens_per_tile) + num_seqs
    fn = _fn("attention_bf16", "ts_flash_prefill",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
              block_table.stride(0), _ptr(query_start_loc), _ptr(context_lens), num_seqs, max_tiles, k_pages.shape[1],
              num_heads, num_kv_heads, head_dim, int(window or 0), float(scale), _stream()), "flash_prefill")


SKEW_SPLIT_ROOM = 16
"""Parts of all requests together, in units of two blocks a multiprocessor per kv head, that a lopsided batch may use."""


def decode_scratch_floats(num_tokens: int, num_heads: int, num_splits: int, head_dim: int) -> int:
    return 0 if num_splits <= 1 else num_tokens * num_heads * num_splits * (head_dim + 2)


def flash_decode(q, out, k_pages, v_pages, block_table, seq_of_token, positions, num_tokens, num_heads, num_kv_heads,
                 head_dim, window, scale, num_splits, scratch, status=None) -> None:
    """Attention for a decode step; ``scratch`` is fp32 of ``decode_scratch_floats(...)`` elements.

    A page that is missing from the table inside a request's visible keys is masked out and
    raises bit 4 of ``status`` (int32, one element) when that is given."""
    _common(q, out, k_pages, v_pages, block_table, num_heads, num_kv_heads, head_dim)
    _need(seq_of_token, torch.int32, "seq_of_token"); _need(positions, torch.int32, "positions")
    if num_splits > CLUSTER_MAX_SPLITS:
        _need(scratch, torch.float32, "scratch")
        if scratch.numel() < decode_scratch_floats(num_tokens, num_heads, num_splits, head_dim):
            raise KernelError("flash_decode: scratch is too small")
    fn = _fn("attention_bf16", "ts_flash_decode",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
              block_table.stride(0), _ptr(seq_of_token), _ptr(positions), num_tokens, k_pages.shape[1], num_heads,
              num_kv_heads, head_dim, int(window or 0), float(scale), num_splits,
              _ptr(scratch if num_splits > CLUSTER_MAX_SPLITS else None), _ptr(status), _stream()), "flash_decode",
           launches=2 if num_splits > CLUSTER_MAX_SPLITS else 1)  # more splits than a cluster holds: a join kernel follows


def tma_decode_supports(head_dim: int, page_size: int, group: int) -> bool:
    """Head size 64 or 128, pages of at least 4 tokens (a power of two), at most 16 query heads per kv head."""
    return head_dim in (64, 128) and page_size >= 4 and page_size & (page_size - 1) == 0 and group <= 16


def flash_decode_tma(q, out, k_pages, v_pages, block_table, seq_of_token, positions, num_tokens, num_heads, num_kv_heads,
                     head_dim, window, scale, num_splits, scratch, status=None) -> None:
    """Attention for a decode step with keys and values fetched by TMA; arguments as :func:`flash_decode`."""
    _common(q, out, k_pages, v_pages, block_table, num_heads, num_kv_heads, head_dim)
    _need(seq_of_token, torch.int32, "seq_of_token"); _need(positions, torch.int32, "positions")
    if num_splits > CLUSTER_MAX_SPLITS:
        _need(scratch, torch.float32, "scratch")
        if scratch.numel() < decode_scratch_floats(num_tokens, num_heads, num_splits, head_dim):
            raise KernelError("flash_decode_tma: scratch is too small")
    fn = _fn("attention_bf16", "ts_flash_decode_tma",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages), k_pages.shape[0],
              _ptr(block_table), block_table.stride(0), _ptr(seq_of_token), _ptr(positions), num_tokens, k_pages.shape[1],
              num_heads, num_kv_heads, head_dim, int(window or 0), float(scale), num_splits,
              _ptr(scratch if num_splits > CLUSTER_MAX_SPLITS else None), _ptr(status), _stream()), "flash_decode_tma",
           launches=2 if num_splits > CLUSTER_MAX_SPLITS else 1)


WORK_LIST = os.environ.get("TURBOSERVE_B200_DECODE_WORK_LIST", "1") != "0"
"""A very lopsided decode step (``StepBatch.decode_skew`` >= WORK_LIST_FROM) cuts every request into parts by its
own length (a work list the TMA-fed kernel walks) instead of all requests into the same, larger, number of parts."""
WORK_LIST_FROM = 4
"""Measured at the 7B sizes: 64 requests, one at 32,768 tokens and 63 at 512 (class 16): 4.73 ms a step with
the list, 5.0 ms with 16 times the parts for everyone; 16 requests, one at 8,192 and 15 at 1,024 (class 2):
3.96 ms with the list, 3.80 ms with twice the parts, which still meet inside a cluster."""


def decode_item_target(num_kv_heads: int, sms: int) -> int:
    """Into how many parts the requests of a lopsided decode step are cut together: two rounds of
    two blocks a multiprocessor, a block being (part, kv head)."""
    return max(32, 2 * ((2 * sms) // max(1, num_kv_heads)))


def flash_decode_tma_items(q, out, k_pages, v_pages, block_table, seq_of_token, positions, num_tokens, num_heads,
                           num_kv_heads, head_dim, window, scale, items, scratch, status=None) -> None:
    """Decode attention over a work list (``engine.batch.DecodeItems``): every request cut by its own length."""
    _common(q, out, k_pages, v_pages, block_table, num_heads, num_kv_heads, head_dim)
    _need(seq_of_token, torch.int32, "seq_of_token"); _need(positions, torch.int32, "positions")
    for name in ("item_token", "item_part", "parts_of", "first_item"):
        _need(getattr(items, name), torch.int32, name)
    if items.item_token.numel() < items.num_items or items.item_part.numel() < items.num_items \
            or items.parts_of.numel() < num_tokens or items.first_item.numel() < num_tokens:
        raise KernelError("flash_decode_tma_items: the work list is shorter than it says")
    _need(scratch, torch.float32, "scratch")
    if scratch.numel() < items.num_items * num_heads * (head_dim + 2):
        raise KernelError("flash_decode_tma_items: scratch is too small")
    fn = _fn("attention_bf16", "ts_flash_decode_tma_items",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
              c_void_p, c_void_p])
    _check(fn(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages), k_pages.shape[0],
              _ptr(block_table), block_table.stride(0), _ptr(seq_of_token), _ptr(positions), num_tokens, k_pages.shape[1],
              num_heads, num_kv_heads, head_dim, int(window or 0), float(scale), _ptr(items.item_token), _ptr(items.item_part),
              _ptr(items.parts_of), _ptr(items.first_item), int(items.num_items), _ptr(scratch), _ptr(status), _stream()),
           "flash_decode_tma_items", launches=2)


FUSED_CLUSTER = os.environ.get("TURBOSERVE_B200_FUSED_CLUSTER", "1") != "0"
FUSED_DECODE = os.environ.get("TURBOSERVE_B200_FUSED_DECODE", "0") != "0"
"""With 1, decode steps let the TMA-fed attention kernel add the bias, rotate queries and keys and
append to the cache itself (one launch less a layer). Off by default: measured inside a captured
decode step at the 7B sizes (batch 8, context 4,096) the step takes 3.35 ms that way against 3.28 ms
with the rotation kernel, whose launch and angles already hide behind the product before it, while
the attention kernel, launched as clusters, cannot be set up ahead of time without costing more
than it saves (3.70 ms), and joining its parts through scratch instead of a cluster costs 3.44 ms."""


@dataclass
class DecodeFusion:
    """The step before attention, handed to the decode kernel instead of being run on its own:
    the bias of the fused q/k/v product, the rotation's constants, and whether to append."""

    bias: torch.Tensor | None
    inv_freq: torch.Tensor | None
    rotary_dim: int
    factor: float
    write: bool


def can_fuse_decode(qkv: torch.Tensor, k_pages: torch.Tensor, batch, num_heads: int, num_kv_heads: int, head_dim: int,
                    scale: float, rotary_dim: int) -> bool:
    """Whether this step's attention can take the raw q/k/v product (:func:`flash_decode_tma_fused`):
    a decode-only bfloat16 step whose shape the TMA-fed kernel takes, with the mixer's own keys and values."""
    return (FUSED_DECODE and TMA_DECODE and qkv.dtype == torch.bfloat16 and batch.is_decode_only and scale > 0
            and head_dim == 128 and tma_decode_supports(head_dim, k_pages.shape[1], num_heads // num_kv_heads)
            and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0 and qkv.shape[1] >= (num_heads + 2 * num_kv_heads) * head_dim
            and 0 <= rotary_dim <= head_dim and rotary_dim % 2 == 0)


def flash_decode_tma_fused(qkv, fusion: DecodeFusion, out, k_pages, v_pages, block_table, seq_of_token, positions, num_tokens,
                           num_heads, num_kv_heads, head_dim, window, scale, num_splits, scratch, status=None) -> None:
    """Decode attention straight from the raw q/k/v product: bias, rotation and cache append happen in the kernel."""
    _common(qkv, out, k_pages, v_pages, block_table, num_heads, num_kv_heads, head_dim)
    _need(seq_of_token, torch.int32, "seq_of_token"); _need(positions, torch.int32, "positions")
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape[1] < width:
        raise KernelError("flash_decode_tma_fused: qkv is narrower than its heads")
    if fusion.bias is not None:
        _need(fusion.bias, torch.float32, "bias")
        if fusion.bias.numel() != width:
            raise KernelError("flash_decode_tma_fused: bias length does not match the projected heads")
    if fusion.rotary_dim:
        _need(fusion.inv_freq, torch.float32, "inv_freq")
        if fusion.inv_freq.numel() * 2 != fusion.rotary_dim:
            raise KernelError("flash_decode_tma_fused: inv_freq must hold rotary_dim / 2 values")
    cluster = FUSED_CLUSTER and 2 <= num_splits <= CLUSTER_MAX_SPLITS
    if num_splits > 1 and not cluster:
        _need(scratch, torch.float32, "scratch")
        if scratch.numel() < decode_scratch_floats(num_tokens, num_heads, num_splits, head_dim):
            raise KernelError("flash_decode_tma_fused: scratch is too small")
    fn = _fn("attention_bf16", "ts_flash_decode_tma_fused",
             [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p, c_longlong, c_void_p, c_void_p,
              c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
              c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(qkv), qkv.stride(0), _ptr(fusion.bias), _ptr(fusion.inv_freq if fusion.rotary_dim else None),
              int(fusion.rotary_dim), float(fusion.factor), int(bool(fusion.write)), _ptr(out), out.stride(0),
              _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], _ptr(block_table), block_table.stride(0), _ptr(seq_of_token),
              _ptr(positions), num_tokens, k_pages.shape[1], num_heads, num_kv_heads, head_dim, int(window or 0),
              float(scale), num_splits, _ptr(scratch if num_splits > 1 and not cluster else None), _ptr(status),
              int(cluster or FUSED_CLUSTER), _stream()), "flash_decode_tma_fused",
           launches=2 if num_splits > 1 and not cluster else 1)


def paged_attention_bf16(q, out, k_pages, v_pages, block_table, batch, num_heads, num_kv_heads, head_dim, window,
                         scale, ctx, fusion: DecodeFusion | None = None) -> bool:
    """Run the tensor-core kernel that fits the step; returns False if the shape is refused.

    With ``fusion`` (only after :func:`can_fuse_decode` said yes) ``q`` is the raw q/k/v product."""
    group = num_heads // num_kv_heads
    if fusion is not None:
        _decode_tokens(q, out, k_pages, v_pages, block_table, batch, 0, batch.num_tokens, num_heads, num_kv_heads, head_dim,
                       window, scale, ctx, fusion)
        return True
    if not scale > 0:
        return False  # the tiled kernel keeps its running maximum in unscaled units
    decode = batch.is_decode_only and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
    if not supports(head_dim, k_pages.shape[1], group, decode):
        if decode and supports(head_dim, k_pages.shape[1], group, False):
            decode = False  # a group too large for the decode kernel still fits the tiled one
        else:
            return False
    n = batch.num_tokens
    if decode:
        _decode_tokens(q, out, k_pages, v_pages, block_table, batch, 0, n, num_heads, num_kv_heads, head_dim, window, scale, ctx)
        return True
    # A mixed step: the requests at the end of the batch that bring one token each (the scheduler
    # puts prompts first, then the requests that decode), or at its head, go to the decode kernel,
    # which splits their keys over many blocks; in the tiled kernel each would hold a 128-row tile,
    # nearly empty, over its whole context. Any token can go either way: its keys are in the cache.
    lead = tail = 0
    if getattr(batch, "query_lens_host", None) and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 \
            and supports(head_dim, k_pages.shape[1], group, True) and len(batch.query_lens_host) == batch.num_seqs and sum(batch.query_lens_host) == n:  # no padding
        lead, tail = batch.num_leading_decode, batch.num_trailing_decode
    if lead:
        _decode_tokens(q, out, k_pages, v_pages, block_table, batch, 0, lead, num_heads, num_kv_heads, head_dim, window, scale, ctx)
    if tail:
        _decode_tokens(q, out, k_pages, v_pages, block_table, batch, n - tail, tail, num_heads, num_kv_heads, head_dim, window, scale, ctx)
    seqs = batch.num_seqs - lead - tail
    tokens = n - lead - tail
    if seqs <= 0 or tokens <= 0:
        return True
    table, starts, lens = block_table[lead:], batch.query_start_loc[lead:], batch.context_lens[lead:]
    if attention_tc.supports(q, out, head_dim, k_pages.shape[1], group, scale):
        attention_tc.flash_prefill_tc(q, out, k_pages, v_pages, table, starts, lens, seqs, tokens, num_heads,
                                      num_kv_heads, head_dim, window, scale, ctx.status,
                                      max_context=min(batch.max_context_len, window) if window else batch.max_context_len)
    else:
        flash_prefill(q, out, k_pages, v_pages, table, starts, lens, seqs, tokens, num_heads, num_kv_heads,
                      head_dim, window, scale)
    return True


def _decode_tokens(q, out, k_pages, v_pages, block_table, batch, first, n, num_heads, num_kv_heads, head_dim, window, scale, ctx,
                   fusion: DecodeFusion | None = None) -> None:
    """Tokens ``first .. first + n`` of the batch, each against the keys of its request up to its position."""
    if first:
        q, out = q[first:], out[first:]
    seq_of_token, positions = batch.seq_of_token[first:], batch.positions[first:]
    group = num_heads // num_kv_heads
    sms = num_sms(q.device)
    # a lopsided batch (one context far above the others) cuts every request's keys into more parts,
    # so that the long one does not hold a few blocks while the device idles
    most = (n + SKEW_SPLIT_ROOM * ((2 * sms) // num_kv_heads)) // n
    splits = max(1, min(decode_splits(n, num_kv_heads, sms) * max(1, getattr(batch, "decode_skew", 1)), MAX_SPLITS, most))
    # tokens x splits never exceeds tokens + 16 x 2 * SMs / kv_heads, and that bound grows with the
    # number of tokens: the scratch a large batch reserves also serves every smaller one
    # (buffers may not grow once decode graphs have been captured)
    bound = num_heads * (head_dim + 2) * (n + SKEW_SPLIT_ROOM * ((2 * sms) // num_kv_heads) + 1)
    scratch = ctx.buffer("attn.decode_scratch", (bound,), torch.float32)
    uneven = getattr(batch, "decode_skew", 1) >= WORK_LIST_FROM and first == 0 and n == batch.num_tokens
    if fusion is not None:
        flash_decode_tma_fused(q, fusion, out, k_pages, v_pages, block_table, seq_of_token, positions, n, num_heads,
                               num_kv_heads, head_dim, window, scale, splits, scratch, ctx.status)
    elif WORK_LIST and uneven and TMA_DECODE and tma_decode_supports(head_dim, k_pages.shape[1], group):
        items = getattr(batch, "decode_items", {}).get(int(window or 0))
        if items is None:
            # a batch that brought no list of its own (not one of fixed shape): make one from its lengths
            from ..engine.batch import DecodeItems, plan_decode_items

            visible = [min(c, window) if window else c for c in batch.context_lens_host]
            target = decode_item_target(num_kv_heads, sms)
            lists = plan_decode_items(visible, target)
            count = len(lists[0])
            flat = torch.tensor(lists[0] + lists[1] + lists[2] + [1] * (n - len(visible)) + lists[3] + [0] * (n - len(visible)),
                                dtype=torch.int32).to(q.device, non_blocking=True)
            items = DecodeItems(flat[:count], flat[count:2 * count], flat[2 * count:2 * count + n], flat[2 * count + n:], count)
            if isinstance(getattr(batch, "decode_items", None), dict):
                batch.decode_items[int(window or 0)] = items  # the other layers of the step use it too
        flash_decode_tma_items(q, out, k_pages, v_pages, block_table, seq_of_token, positions, n, num_heads, num_kv_heads,
                               head_dim, window, scale, items, scratch, ctx.status)
    elif TMA_DECODE and tma_decode_supports(head_dim, k_pages.shape[1], group):
        flash_decode_tma(q, out, k_pages, v_pages, block_table, seq_of_token, positions, n, num_heads,
                         num_kv_heads, head_dim, window, scale, splits, scratch, ctx.status)
    else:
        flash_decode(q, out, k_pages, v_pages, block_table, seq_of_token, positions, n, num_heads,
                     num_kv_heads, head_dim, window, scale, splits, scratch, ctx.status)
