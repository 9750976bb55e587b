"""The arithmetic that sizes the page pool (no GPU)."""

import pytest
import torch

from conftest import TINY_B
from turboserve_b200.config import SchedulerConfig, config_from_dict, lookup
from turboserve_b200.engine import memory
from turboserve_b200.engine.memory import activation_headroom_bytes, size_kv_cache


def tiny_model():
    config = config_from_dict(TINY_B)
    return lookup(config.architecture).build_model(config, torch.bfloat16, "cpu")


def test_pages_are_what_is_left_after_weights_and_scratch():
    model = tiny_model()
    scheduler = SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64, block_size=8)
    scratch = model.scratch_bytes_per_token(2)
    # residual fp32 + normed rows + attention (qkv, attended, out) + feed-forward (gate and up, product, out)
    assert scratch == 4 * 96 + 2 * (96 + (5 * 32 + 3 * 32 + 96) + (3 * 256 + 96))
    total, used = 1 << 26, 1 << 22
    sizing = size_kv_cache(model.cache_plan(), scheduler, 2, scratch_per_token=scratch, vocab=model.vocab_size,
                           gpu_memory_utilization=0.5, memory_info=(total - used, total))
    headroom = activation_headroom_bytes(scratch, model.vocab_size, scheduler)
    assert headroom == 64 * scratch + 2 * 4 * 1000 * 4 + 4 * 32 * 4  # logits twice, a bit per request and vocabulary entry
    per_page = sum(model.cache_plan().bytes_per_page(8, 2))
    assert sizing.bytes_per_block == per_page and sizing.source == "memory"
    assert sizing.num_blocks == (total // 2 - used - headroom) // per_page
    capped = size_kv_cache(model.cache_plan(), scheduler, 2, scratch_per_token=scratch, vocab=model.vocab_size,
                           gpu_memory_utilization=0.5, memory_info=(total - used, total), max_model_len=100)
    assert capped.num_blocks == 13 * 4 and capped.source == "max_model_len"
    with pytest.raises(RuntimeError, match="no memory for the cache"):
        size_kv_cache(model.cache_plan(), scheduler, 2, scratch_per_token=scratch, vocab=model.vocab_size,
                      gpu_memory_utilization=0.5, memory_info=(1 << 20, total))


def test_memory_the_allocator_holds_for_nobody_counts_as_free(monkeypatch):
    """Fusing q/k/v and gate/up leaves the unfused originals in torch's caching allocator: the
    driver sees them as used, but the cache is allocated through that allocator and gets them."""
    total = 100 << 30
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda device=None: (40 << 30, total))
    monkeypatch.setattr(torch.cuda, "memory_reserved", lambda device=None: 55 << 30)
    monkeypatch.setattr(torch.cuda, "memory_allocated", lambda device=None: 30 << 30)
    assert memory.device_memory_info() == ((40 + 25) << 30, total)


def test_a_part_that_declares_no_scratch_gets_the_stated_default():
    from turboserve_b200.parts.base import UNDECLARED_SCRATCH_WIDTHS, Part

    model = tiny_model()
    declared = model.scratch_bytes_per_token(2)
    model.blocks[0].feed_forward.scratch_per_token = Part.scratch_per_token.__get__(model.blocks[0].feed_forward)
    assert model.blocks[0].feed_forward.scratch_per_token() is None
    assert model.scratch_bytes_per_token(2) == declared  # the other layers' feed-forwards are wider
    for block in model.blocks:
        block.feed_forward.scratch_per_token = lambda: None
    assert model.scratch_bytes_per_token(2) == declared - 2 * (3 * 256 + 96) + 2 * UNDECLARED_SCRATCH_WIDTHS * 96
