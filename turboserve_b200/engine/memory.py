"""How many cache pages fit: the arithmetic the engine does at start-up.

``num_blocks`` given explicitly wins. Otherwise the budget is ``gpu_memory_utilization x
total - used - activation headroom``, divided by the bytes one page id stands for over all
cache groups (every group gets the same number of pages), capped at what ``max_num_seqs``
requests of ``max_model_len`` tokens could ever use. Same rule as
``src/turboserve/engine/runtime/memory.py:208-348``, with groups and state slots added.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass

import torch

from ..cache.storage import CachePlan
from ..config.engine_config import SchedulerConfig


@dataclass
class KVCacheSizing:
    num_blocks: int
    block_size: int
    num_groups: int
    bytes_per_block: int
    state_bytes: int
    total_bytes: int
    source: str
    budget_bytes: int | None = None
    activation_bytes: int | None = None
    max_tokens: int = 0

    def to_dict(self) -> dict:
        return asdict(self)


def activation_headroom_bytes(scratch_per_token: int, vocab: int, scheduler: SchedulerConfig) -> int:
    """Scratch the step needs at its largest batch: what the model's parts declare per token
    (``DecoderModel.scratch_bytes_per_token``), fp32 logits for every request, twice (the sampler's
    scratch is as large), and the sampler's bit per vocabulary entry and request."""
    seen_bits = scheduler.max_num_seqs * ((vocab + 31) // 32) * 4
    return scheduler.max_num_batched_tokens * scratch_per_token + 2 * scheduler.max_num_seqs * vocab * 4 + seen_bits


def device_memory_info(device: torch.device | None = None) -> tuple[int, int]:
    """``(free, total)`` bytes as the sizing wants them: memory that torch's allocator holds but has
    handed to nobody (freed originals of fused weights, for instance) counts as free, since the
    cache is allocated through the same allocator and gets it."""
    free, total = torch.cuda.mem_get_info(device)
    cached = torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
    return free + max(0, cached), total


def size_kv_cache(plan: CachePlan, scheduler: SchedulerConfig, itemsize: int, *, scratch_per_token: int, vocab: int,
                  gpu_memory_utilization: float = 0.9, max_model_len: int | None = None,
                  device: torch.device | None = None, memory_info: tuple[int, int] | None = None) -> KVCacheSizing:
    block = scheduler.block_size
    per_page = sum(plan.bytes_per_page(block, itemsize))
    state = plan.state_bytes_per_slot() * scheduler.max_num_seqs
    groups = len(plan.windows)
    if per_page == 0:
        blocks = scheduler.num_blocks or 1
        return KVCacheSizing(blocks, block, groups, 0, state, state, "no paged layers", max_tokens=blocks * block)
    if scheduler.num_blocks is not None:
        blocks = scheduler.num_blocks
        return KVCacheSizing(blocks, block, groups, per_page, state, blocks * per_page + state, "explicit",
                             max_tokens=blocks * block)
    if memory_info is None:
        memory_info = device_memory_info(device)
    free, total = memory_info
    used = total - free
    activations = activation_headroom_bytes(scratch_per_token, vocab, scheduler)
    budget = int(gpu_memory_utilization * total) - used - activations - state
    blocks = budget // per_page
    if blocks < 1:
        raise RuntimeError(
            f"no memory for the cache: {gpu_memory_utilization:.2f} x {total} bytes minus {used} in use minus "
            f"{activations} of scratch leaves {budget}, one page needs {per_page}"
        )
    source = "memory"
    if max_model_len is not None:
        cap = -(-max_model_len // block) * scheduler.max_num_seqs
        if cap < blocks:
            blocks, source = cap, "max_model_len"
    return KVCacheSizing(int(blocks), block, groups, per_page, state, int(blocks) * per_page + state, source, budget,
                         activations, int(blocks) * block)
