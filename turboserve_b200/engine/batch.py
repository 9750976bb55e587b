"""What one step runs on: the packed batch, the scratch buffers, and the context parts see.

A step is a flat vector of tokens: every scheduled request's next tokens one after another,
portions of prompts beside single decoded tokens, cut anywhere. The reference describes the
same batch with ``AttnMetadata`` (``src/turboserve/engine/core/types.py:244-398``) and builds
it from Python lists every step (``src/turboserve/engine/runtime/worker.py:180-201``). Here the
indices are int32, there is one block table per cache group, ``seq_of_token`` lets a kernel
find a token's request without a search, ``state_slots`` names each request's slot of
fixed-size state, and logits may be asked at any rows.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import torch


@dataclass
class RequestSlice:
    """One request's part of a step, on the host."""

    token_ids: Sequence[int]
    start_position: int
    """Number of tokens of this request already in the cache (position of the first new one)."""

    block_tables: Sequence[Sequence[int]]
    """One table per cache group, in group order; ``-1`` marks a page that was given back."""

    state_slot: int = 0
    want: Sequence[int] = ()
    """Indices among ``token_ids`` whose logits are wanted."""


@dataclass
class StepBatch:
    """Device tensors of one step (see the module docstring). Padding tokens have seq -1."""

    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    seq_of_token: torch.Tensor
    query_start_loc: torch.Tensor
    context_lens: torch.Tensor
    block_tables: list[torch.Tensor]
    state_slots: torch.Tensor
    logit_rows: torch.Tensor
    num_logit_rows: int
    query_lens_host: list[int] = field(default_factory=list)
    context_lens_host: list[int] = field(default_factory=list)
    state_slots_host: list[int] = field(default_factory=list)
    max_query_len: int = 0
    max_context_len: int = 0
    decode_skew: int = 1
    """1, 2, 4, 8 or 16: how far the longest context of the requests that decode lies above their mean
    (:func:`skew_class`). At 2 decode attention cuts every request's keys into twice the parts; from 4
    on it cuts every request into parts by its own length (a work list, :func:`plan_decode_items`), or,
    in kernels that take no list, every request's keys into that many times more parts."""

    decode_items: dict[int, "DecodeItems"] = field(default_factory=dict)
    """Work lists of a lopsided decode step that were made with the batch, by the window they are for (0: none)."""

    @property
    def is_decode_only(self) -> bool:
        return self.max_query_len == 1

    @property
    def num_leading_decode(self) -> int:
        """How many requests at the head of the batch bring exactly one token (their tokens lead too)."""
        count = 0
        for n in self.query_lens_host:
            if n != 1:
                break
            count += 1
        return count

    @property
    def num_trailing_decode(self) -> int:
        """How many requests at the end of the batch bring exactly one token (their tokens end it too)."""
        count = 0
        for n in reversed(self.query_lens_host):
            if n != 1:
                break
            count += 1
        return count


def skew_class(contexts: Sequence[int]) -> int:
    """How lopsided a decode batch is: the largest of 1, 2, 4, 8, 16 not above max / mean of its contexts.

    Decode attention gives every request the same number of blocks. One request with a context far
    above the others' then holds a few blocks for a long time while the rest of the device idles
    (64 requests, one of them at 32,768 tokens and the others at 256: 492 us a layer instead of 52).
    The class multiplies the number of parts every request's keys are cut into. It is a property of
    the batch alone, so a decode graph is captured per (batch size, class).
    """
    if not contexts:
        return 1
    longest, total = max(contexts), sum(contexts)
    if total <= 0:
        return 1
    ratio = longest * len(contexts) / total
    for cls in (16, 8, 4, 2):
        if ratio >= cls:
            return cls
    return 1


WORK_LIST_FROM = 4
"""The class of lopsidedness from which a decode step brings a work list (the attention kernels' rule, ``ops/attention_bf16.py``)."""
DECODE_ITEM_KEYS = 256
"""The fewest keys a part of a request is worth a block for."""
DECODE_ITEM_MAX_PARTS = 64


def plan_decode_items(visible: Sequence[int], target_items: int, min_keys: int = DECODE_ITEM_KEYS,
                      max_parts: int = DECODE_ITEM_MAX_PARTS, tile: int = 64):
    """Cut the requests of a decode step into parts of about equal length: the work list of decode attention.

    ``visible[i]`` is the number of keys request ``i`` attends to. All keys together are cut into
    about ``target_items`` parts of one length (a multiple of ``tile``, at least ``min_keys``);
    a request gets as many parts as its own keys fill, at least one and at most ``max_parts``.
    Returns ``(item_token, item_part, parts_of, first_item)`` as lists: item ``k`` is part
    ``item_part[k]`` of request ``item_token[k]``, the longest requests' items first (their blocks
    start first); request ``i`` has ``parts_of[i]`` parts whose partial results lie in scratch from
    slot ``first_item[i]`` on. There are never more than ``len(visible) + target_items`` items.
    """
    n = len(visible)
    total = sum(max(0, int(v)) for v in visible)
    length = max(min_keys, -(-total // max(1, target_items)))
    length = -(-length // tile) * tile
    parts_of = [min(max_parts, max(1, -(-max(0, int(v)) // length))) for v in visible]
    first_item, cursor = [0] * n, 0
    for i in range(n):
        first_item[i] = cursor
        cursor += parts_of[i]
    item_token, item_part = [], []
    for i in sorted(range(n), key=lambda r: -visible[r]):
        item_token += [i] * parts_of[i]
        item_part += list(range(parts_of[i]))
    return item_token, item_part, parts_of, first_item


@dataclass
class DecodeItems:
    """The work list of :func:`plan_decode_items` on the device (int32), padded to ``num_items`` items with -1."""

    item_token: torch.Tensor
    item_part: torch.Tensor
    parts_of: torch.Tensor
    first_item: torch.Tensor
    num_items: int


def build_step_batch(slices: Sequence[RequestSlice], num_groups: int, device: torch.device | str,
                     pad_tokens_to: int | None = None, pad_seqs_to: int | None = None,
                     table_widths: Sequence[int] | None = None, pad_rows_to: int | None = None) -> StepBatch:
    """Pack host-side slices into one :class:`StepBatch` (one host-to-device copy).

    ``pad_tokens_to`` / ``pad_seqs_to`` / ``table_widths`` give fixed shapes (for steps that
    are replayed from a captured graph); padding tokens carry ``seq_of_token == -1`` and
    padding requests a context length of 0.
    """
    ids: list[int] = []
    positions: list[int] = []
    seq_of: list[int] = []
    qsl = [0]
    ctx_lens: list[int] = []
    q_lens: list[int] = []
    slots: list[int] = []
    rows: list[int] = []
    for index, piece in enumerate(slices):
        n = len(piece.token_ids)
        if n < 1:
            raise ValueError("a request in a step must bring at least one token")
        if len(piece.block_tables) != num_groups:
            raise ValueError(f"request {index} has {len(piece.block_tables)} block tables for {num_groups} cache groups")
        base = len(ids)
        ids.extend(int(t) for t in piece.token_ids)
        positions.extend(range(piece.start_position, piece.start_position + n))
        seq_of.extend([index] * n)
        qsl.append(base + n)
        q_lens.append(n)
        ctx_lens.append(piece.start_position + n)
        slots.append(int(piece.state_slot))
        for w in piece.want:
            if not 0 <= w < n:
                raise ValueError(f"request {index} wants logits at {w}, outside its {n} tokens")
            rows.append(base + int(w))
    num_tokens, num_seqs = len(ids), len(slices)
    total_tokens = max(num_tokens, pad_tokens_to or 0)
    total_seqs = max(num_seqs, pad_seqs_to or 0)
    widths = []
    for g in range(num_groups):
        width = max([len(piece.block_tables[g]) for piece in slices] + [1])
        if table_widths is not None:
            if width > table_widths[g]:
                raise ValueError(f"block table of group {g} needs {width} entries, fixed width is {table_widths[g]}")
            width = table_widths[g]
        widths.append(width)
    # one flat int32 staging buffer, one copy
    flat: list[int] = []
    flat += ids + [0] * (total_tokens - num_tokens)
    flat += positions + [0] * (total_tokens - num_tokens)
    flat += seq_of + [-1] * (total_tokens - num_tokens)
    flat += qsl + [num_tokens] * (total_seqs - num_seqs)
    flat += ctx_lens + [0] * (total_seqs - num_seqs)
    flat += slots + [0] * (total_seqs - num_seqs)
    rows = rows + [0] * max(0, (pad_rows_to or 0) - len(rows))
    flat += rows
    for g in range(num_groups):
        for piece in slices:
            table = list(piece.block_tables[g])
            flat += table + [-1] * (widths[g] - len(table))
        flat += [-1] * (widths[g] * (total_seqs - num_seqs))
    staged = torch.tensor(flat, dtype=torch.int32).pin_memory() if torch.cuda.is_available() else torch.tensor(flat, dtype=torch.int32)
    dev = staged.to(device, non_blocking=True)
    offset = 0

    def take(count: int) -> torch.Tensor:
        nonlocal offset
        view = dev[offset:offset + count]
        offset += count
        return view

    t_ids, t_pos, t_seq = take(total_tokens), take(total_tokens), take(total_tokens)
    t_qsl, t_ctx, t_slots = take(total_seqs + 1), take(total_seqs), take(total_seqs)
    t_rows = take(len(rows))
    tables = [take(total_seqs * widths[g]).view(total_seqs, widths[g]) for g in range(num_groups)]
    return StepBatch(
        num_tokens=total_tokens, num_seqs=total_seqs, token_ids=t_ids, positions=t_pos, seq_of_token=t_seq,
        query_start_loc=t_qsl, context_lens=t_ctx, block_tables=tables, state_slots=t_slots, logit_rows=t_rows,
        num_logit_rows=len(rows), query_lens_host=q_lens, context_lens_host=ctx_lens, state_slots_host=slots,
        max_query_len=max(q_lens, default=0), max_context_len=max(ctx_lens, default=0),
        decode_skew=skew_class([c for c, n in zip(ctx_lens, q_lens) if n == 1]),
    )


class StaticBatch:
    """A batch of fixed shape at fixed device addresses, refilled in place every step.

    Used for steps that are replayed from a captured CUDA graph: ``tokens`` tokens, ``seqs``
    requests, ``seqs`` logit rows and block tables of ``table_widths`` entries, all in one
    int32 device buffer mirrored by one pinned host buffer, so that a refill is a few numpy
    slice assignments and one host-to-device copy.
    """

    def __init__(self, tokens: int, seqs: int, table_widths: Sequence[int], device: torch.device | str,
                 item_windows: Sequence[int | None] = (), item_targets: Sequence[int] = ()) -> None:
        """``item_windows`` / ``item_targets``: for each cache group whose decode attention takes a work
        list, its window (``None``: every key) and the number of parts all requests together are cut into."""
        self.tokens, self.seqs, self.widths = int(tokens), int(seqs), [int(w) for w in table_widths]
        self.item_windows = [int(w) if w else 0 for w in item_windows]
        self.item_targets = [int(t) for t in item_targets]
        counts = [tokens, tokens, tokens, seqs + 1, seqs, seqs, seqs] + [seqs * w for w in self.widths]
        self._first_item_range = len(counts)
        for target in self.item_targets:  # item_token, item_part, parts_of, first_item
            counts += [seqs + target, seqs + target, seqs, seqs]
        total = sum(counts)
        self.host = torch.zeros(total, dtype=torch.int32).pin_memory()
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)
        offsets = [0]
        for c in counts:
            offsets.append(offsets[-1] + c)
        self._ranges = list(zip(offsets[:-1], offsets[1:]))
        for a, b in self._ranges[7:self._first_item_range]:
            self.host_np[a:b] = -1
        for k in range(len(self.item_targets)):
            a, b = self._ranges[self._first_item_range + 4 * k]
            self.host_np[a:b] = -1  # no item is in use
        self._known: list[list[tuple[object, int]]] = [[(None, 0)] * seqs for _ in self.widths]
        self._uploaded: torch.cuda.Event | None = None
        views = [self.dev[a:b] for a, b in self._ranges]
        tables = [v.view(seqs, w) for v, w in zip(views[7:], self.widths)]
        self._items = {}
        for k, (window, target) in enumerate(zip(self.item_windows, self.item_targets)):
            r = self._first_item_range + 4 * k
            self._items[window] = DecodeItems(views[r], views[r + 1], views[r + 2], views[r + 3], seqs + target)
        self.batch = StepBatch(
            num_tokens=tokens, num_seqs=seqs, token_ids=views[0], positions=views[1], seq_of_token=views[2],
            query_start_loc=views[3], context_lens=views[4], block_tables=tables, state_slots=views[5],
            logit_rows=views[6], num_logit_rows=seqs,
        )

    def _host(self, index: int):
        a, b = self._ranges[index]
        return self.host_np[a:b]

    def load_decode(self, slices: Sequence[RequestSlice]) -> StepBatch:
        """Refill for a decode step: one token per request, logits for every request."""
        n = len(slices)
        if n > self.seqs or self.tokens != self.seqs:
            raise ValueError(f"{n} requests do not fit a static batch of {self.seqs}")
        if self._uploaded is not None:
            self._uploaded.synchronize()  # the copy of the step before reads the host mirror: let it finish (it has, as a rule)
        ids, pos, seq, qsl, ctx, slots, rows = (self._host(i) for i in range(7))
        ids[:n] = [piece.token_ids[0] for piece in slices]
        ids[n:] = 0
        starts = [piece.start_position for piece in slices]
        pos[:n] = starts
        pos[n:] = 0
        seq[:n] = range(n)
        seq[n:] = -1
        qsl[: n + 1] = range(n + 1)
        qsl[n + 1:] = n
        ctx[:n] = [p + 1 for p in starts]
        ctx[n:] = 0
        slots[:n] = [piece.state_slot for piece in slices]
        slots[n:] = 0
        rows[:n] = range(n)
        rows[n:] = 0
        for g, width in enumerate(self.widths):
            table = self._host(7 + g).reshape(self.seqs, width)
            known = self._known[g]
            for i, piece in enumerate(slices):
                entries = piece.block_tables[g]
                count = len(entries)
                if count > width:
                    raise ValueError(f"block table of group {g} needs {count} entries, the static batch has {width}")
                seen_list, seen_count = known[i]
                if seen_list is entries and seen_count <= count:
                    # the same live table as last step: only what was appended is new (entries that
                    # were given back since lie behind the window and are never read)
                    if seen_count < count:
                        table[i, seen_count:count] = entries[seen_count:]
                else:
                    table[i, :count] = entries
                    table[i, count:] = -1
                known[i] = (entries, count)
            for i in range(n, self.seqs):
                if known[i][0] is not None:
                    table[i] = -1
                    known[i] = (None, 0)
        uneven = skew_class([p + 1 for p in starts]) >= WORK_LIST_FROM
        if uneven:
            for k, (window, target) in enumerate(zip(self.item_windows, self.item_targets)):
                visible = [min(p + 1, window) if window else p + 1 for p in starts]
                item_token, item_part, parts_of, first_item = plan_decode_items(visible, target)
                r = self._first_item_range + 4 * k
                host = [self._host(r + j) for j in range(4)]
                host[0][: len(item_token)] = item_token
                host[0][len(item_token):] = -1
                host[1][: len(item_part)] = item_part
                host[1][len(item_part):] = 0
                host[2][:n] = parts_of
                host[2][n:] = 1
                host[3][:n] = first_item
                host[3][n:] = 0
        self.dev.copy_(self.host, non_blocking=True)
        if self._uploaded is None:
            self._uploaded = torch.cuda.Event()
        self._uploaded.record()
        batch = self.batch
        batch.decode_items = self._items if uneven else {}
        batch.query_lens_host = [1] * n
        batch.context_lens_host = [p + 1 for p in starts]
        batch.state_slots_host = [piece.state_slot for piece in slices]
        batch.max_query_len = 1
        batch.max_context_len = max(batch.context_lens_host, default=0)
        batch.decode_skew = skew_class(batch.context_lens_host)
        return batch

    @property
    def nbytes(self) -> int:
        return self.host.numel() * 4


class Workspace:
    """Named scratch buffers that live across steps, grown on demand, never shrunk.

    Activations of a step are views into these, so a step allocates nothing once the largest
    batch has been seen, and addresses stay fixed for graph replay.
    """

    def __init__(self, device: torch.device | str) -> None:
        self.device = torch.device(device)
        self._buffers: dict[str, torch.Tensor] = {}
        self.frozen = False

    def get(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        count = 1
        for s in shape:
            count *= int(s)
        key = f"{name}:{dtype}"
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < count:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would have to grow while frozen for graph capture")
            buf = torch.empty(max(count, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:count].view(*shape)

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


@dataclass
class StepContext:
    """What a part sees of the step it runs in."""

    batch: StepBatch
    workspace: Workspace
    dtype: torch.dtype
    device: torch.device
    status: torch.Tensor
    """int32[1] that kernels OR error bits into (bad token id, missing page); read after the step."""

    run_index: int = 0
    """Index in the run order of the layer that is running (names scratch uniquely if needed)."""

    def buffer(self, name: str, shape: Sequence[int], dtype: torch.dtype | None = None) -> torch.Tensor:
        return self.workspace.get(name, shape, dtype or self.dtype)
