"""The packed batch on the host: how lopsided a decode batch is, and what the builders record of it."""

import torch

from turboserve_b200.engine.batch import RequestSlice, build_step_batch, skew_class


def test_skew_class_is_the_power_of_two_below_longest_over_mean():
    assert skew_class([]) == 1
    assert skew_class([4096] * 64) == 1
    assert skew_class([100, 120, 90, 150]) == 1
    assert skew_class([3000, 1000, 1000, 1000]) == 2            # 3000 / 1500
    assert skew_class([8192] + [1024] * 63) == 4                # 8192 / 1136 = 7.2
    assert skew_class([32768] + [2048] * 63) == 8               # 12.96
    assert skew_class([32768] + [256] * 63) == 16               # 42.9
    assert skew_class([10**6] + [1] * 255) == 16                # never more
    assert skew_class([0, 0]) == 1


def test_the_builder_counts_only_requests_that_decode():
    def piece(tokens, start, slot):
        pages = list(range(slot * 100, slot * 100 + (start + tokens + 15) // 16))
        return RequestSlice([1] * tokens, start, [pages], slot, [tokens - 1])

    batch = build_step_batch([piece(40, 0, 0), piece(1, 999, 1), piece(1, 9, 2), piece(1, 19, 3), piece(1, 29, 4)], 1, "cpu")
    assert batch.query_lens_host == [40, 1, 1, 1, 1] and batch.num_trailing_decode == 4 and batch.num_leading_decode == 0
    assert batch.decode_skew == skew_class([1000, 10, 20, 30]) == 2  # 1000 / 265
    assert batch.max_context_len == 1000
    whole = build_step_batch([piece(40, 0, 0), piece(7, 3, 1)], 1, "cpu")
    assert whole.decode_skew == 1 and whole.num_trailing_decode == 0
    assert isinstance(batch.context_lens, torch.Tensor)


def test_the_work_list_of_a_lopsided_step_gives_every_request_parts_by_its_own_length():
    from turboserve_b200.engine.batch import DECODE_ITEM_MAX_PARTS, plan_decode_items

    visible = [32768] + [512] * 7 + [100, 1]
    item_token, item_part, parts_of, first_item = plan_decode_items(visible, target_items=148)
    assert len(item_token) == len(item_part) == sum(parts_of) <= len(visible) + 148
    assert parts_of[0] == max(parts_of) and parts_of[-1] == parts_of[-2] == 1
    # the parts of a request lie one after the other in scratch, requests in their own order
    assert first_item == [sum(parts_of[:i]) for i in range(len(visible))]
    # every (request, part) exactly once; the longest request's items come first
    assert sorted(zip(item_token, item_part)) == [(i, p) for i in range(len(visible)) for p in range(parts_of[i])]
    assert item_token[: parts_of[0]] == [0] * parts_of[0]
    # parts are of about one length: no request's part is more than the common length, unless it is capped
    length = max(-(-v // p) for v, p in zip(visible[1:], parts_of[1:]))
    assert length <= 256 and (parts_of[0] == DECODE_ITEM_MAX_PARTS or -(-visible[0] // parts_of[0]) <= 320)
    # an even batch: the same number of parts for all
    even = plan_decode_items([4096] * 8, target_items=148)
    assert len(set(even[2])) == 1 and sum(even[2]) <= 8 + 148
    # nothing to attend to at all still gives one (empty) part each
    assert plan_decode_items([0, 0], 10)[2] == [1, 1]
