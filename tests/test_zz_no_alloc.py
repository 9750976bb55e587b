"""The decode attention entry point that brings its own scratch (for callers that cannot allocate).

Some users of the kernels have given all device memory to their own arena, or run loops in
which cudaMalloc is forbidden; ``ts_flash_decode_static`` keeps the partial results of the
splits in an array inside the library instead of asking for a buffer. The test calls the
exported C symbol directly, twice in a row with different batches (the array keeps what the
first call left), and compares with the ordinary entry point. It is collected last, so a run
that stops at the first failure has run everything else by then.
"""

import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

from kernel_refs import attention_reference, pack_queries, paged_layout

pytestmark = pytest.mark.gpu
DEV = "cuda"


def static_entry():
    from turboserve_b200.ops.build import load_library

    lib = load_library("attention_bf16")
    fn = lib.ts_flash_decode_static
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]
    capacity = lib.ts_flash_decode_static_capacity_floats
    capacity.restype = c_longlong
    return fn, int(capacity())


def case(contexts, nh, nkv, d, page, window, seed):
    k_dense, v_dense, k_pages, v_pages, table = paged_layout(contexts, page, nkv, d, torch.bfloat16, DEV, seed=seed)
    q, positions, seq_of = pack_queries(contexts, [1] * len(contexts), nh, d, torch.bfloat16, DEV, seed=seed + 1)
    scale = 1.0 / math.sqrt(d)
    ref = torch.cat([attention_reference(q[s:s + 1].float(), k_dense[s], v_dense[s], positions[s:s + 1].cpu(), window, scale)
                     for s in range(len(contexts))])
    return q.to(DEV).view(len(contexts), nh * d), k_pages, v_pages, table, positions, seq_of, ref, scale


def call_static(fn, q, out, k_pages, v_pages, table, seq_of, positions, n, page, nh, nkv, d, window, scale, splits):
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    return fn(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
              table.data_ptr(), table.stride(0), seq_of.data_ptr(), positions.data_ptr(), n, page, nh, nkv, d,
              int(window or 0), scale, splits, stream)


def test_static_entry_point_matches_the_ordinary_one_on_two_calls_in_a_row():
    """Two calls in a row, a large one and then a smaller one with padding tokens at its end, so that
    slots of the array which the first call filled and the second does not use would show if they
    were read. With more splits than a cluster holds the ordinary entry point runs the same two
    kernels on its own scratch: the results must then be equal bit for bit. With fewer it joins
    inside a cluster (another order of sums): equal to a bfloat16 step of the outputs."""
    from turboserve_b200.ops import attention_bf16 as fa

    fn, capacity = static_entry()
    assert capacity == 1 << 20
    for contexts, pads, nh, nkv, d, page, window, splits, seed in [
        ([1, 37, 300, 64, 129, 1000, 65], 0, 28, 4, 128, 16, None, 12, 0),   # 12 splits: scratch on both sides
        ([513, 2, 90], 2, 28, 4, 128, 16, None, 9, 7),                       # smaller, two padding tokens, 9 splits
        ([513, 2, 90], 1, 6, 2, 64, 8, 50, 3, 5),                            # head size 64, a window, 3 splits: a cluster on the ordinary side
    ]:
        q, k_pages, v_pages, table, positions, seq_of, ref, scale = case(contexts, nh, nkv, d, page, window, seed)
        live, n = len(contexts), len(contexts) + pads
        if pads:
            q = torch.cat([q, torch.zeros(pads, nh * d, dtype=torch.bfloat16, device=DEV)])
            positions = torch.cat([positions, torch.zeros(pads, dtype=torch.int32, device=DEV)])
            seq_of = torch.cat([seq_of, torch.full((pads,), -1, dtype=torch.int32, device=DEV)])
        assert fa.decode_scratch_floats(n, nh, splits, d) <= capacity
        ordinary = torch.full((n, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        scratch = torch.empty(max(4, fa.decode_scratch_floats(n, nh, splits, d)), device=DEV)
        fa.flash_decode(q, ordinary, k_pages, v_pages, table, seq_of, positions, n, nh, nkv, d, window, scale, splits, scratch)
        out = torch.full((n, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        assert call_static(fn, q, out, k_pages, v_pages, table, seq_of, positions, n, page, nh, nkv, d, window, scale, splits) == 0
        torch.cuda.synchronize()
        assert torch.isfinite(out[:live].float()).all() and torch.isnan(out[live:].float()).all()  # padding rows are not written
        if splits > fa.CLUSTER_MAX_SPLITS:
            assert torch.equal(out[:live], ordinary[:live])
        else:
            assert (out[:live].float() - ordinary[:live].float()).abs().max().item() <= 2.0 ** -7 * max(1.0, ref.abs().max().item())
        assert (out[:live].view(live, nh, d).double().cpu() - ref).abs().max().item() < 2e-2


def test_static_entry_point_finds_one_far_key_and_takes_no_device_memory():
    """One key among 1,301 stands out (its value is 7 everywhere): a split that was lost, or a stale
    slot of the array that was read, would pull the result away from 7. And a warmed call leaves
    the device's free memory as it found it."""
    fn, _ = static_entry()
    nh, nkv, d, page, ctx, far, splits = 7, 1, 128, 16, 1301, 700, 10
    gen = torch.Generator().manual_seed(11)
    k = torch.randn(ctx, nkv, d, generator=gen) * 0.01
    v = torch.randn(ctx, nkv, d, generator=gen)
    direction = torch.randn(d, generator=gen)
    direction /= direction.norm()
    k[far, 0] = direction * 30
    v[far, 0] = 7.0
    pages = -(-ctx // page)
    order = torch.randperm(pages + 2, generator=gen).tolist()
    k_pages, v_pages = torch.zeros(pages + 2, page, nkv, d), torch.zeros(pages + 2, page, nkv, d)
    for p in range(pages):
        lo, hi = p * page, min((p + 1) * page, ctx)
        k_pages[order[p], : hi - lo], v_pages[order[p], : hi - lo] = k[lo:hi], v[lo:hi]
    k_pages, v_pages = k_pages.to(torch.bfloat16).to(DEV), v_pages.to(torch.bfloat16).to(DEV)
    table = torch.tensor([order[:pages]], dtype=torch.int32, device=DEV)
    q = (direction * 30).repeat(1, nh).to(torch.bfloat16).to(DEV)
    positions = torch.tensor([ctx - 1], dtype=torch.int32, device=DEV)
    seq_of = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty(1, nh * d, dtype=torch.bfloat16, device=DEV)
    args = (fn, q, out, k_pages, v_pages, table, seq_of, positions, 1, page, nh, nkv, d, None, 1.0, splits)
    assert call_static(*args) == 0  # the first call of this shape may load the kernels' code
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    out.fill_(0)
    assert call_static(*args) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert (out.float() - 7.0).abs().max().item() < 0.05


def test_static_entry_point_refuses_what_does_not_fit():
    fn, capacity = static_entry()
    n, nh, nkv, d, splits = 64, 32, 8, 128, 32  # 64 * 32 * 32 * 130 floats: far beyond the array
    assert n * nh * splits * (d + 2) > capacity
    q = torch.zeros(n, nh * d, dtype=torch.bfloat16, device=DEV)
    out = torch.full((n, nh * d), 3.0, dtype=torch.bfloat16, device=DEV)
    pages = torch.zeros(4, 16, nkv, d, dtype=torch.bfloat16, device=DEV)
    table = torch.zeros(n, 1, dtype=torch.int32, device=DEV)
    zeros = torch.zeros(n, dtype=torch.int32, device=DEV)
    code = fn(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), pages.data_ptr(), pages.data_ptr(), table.data_ptr(), 1,
              zeros.data_ptr(), zeros.data_ptr(), n, 16, nh, nkv, d, 0, 1.0, splits, c_void_p(torch.cuda.current_stream().cuda_stream))
    assert code == -5
    torch.cuda.synchronize()
    assert (out == 3.0).all()  # nothing was launched
