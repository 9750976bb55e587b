"""The step function: run a batch of (request, its next tokens) against the cache.

:class:`ModelRunner` owns the model, the cache tensors and the scratch buffers, and has one
entry, :meth:`ModelRunner.step`: it runs exactly the tokens it is given, as one batch, writes
their keys and values (and state) into the cache, and returns fp32 logits at the wanted rows.
It is what the scheduler-driven engine, the replay program and the benchmark all call; the
reference splits the same work over ``ModelRunner.execute``
(``src/turboserve/engine/runtime/worker.py:237-266``), ``CausalLM.forward`` and
``compute_logits`` (``src/turboserve/engine/model/model.py:176-244``).
"""

from __future__ import annotations

from pathlib import Path
from typing import Sequence

import torch

from ..cache.manager import GroupSpec
from ..cache.storage import CachePlan, CacheStorage
from ..config.registry import config_from_dir, lookup
from ..models.decoder import DecoderModel
from ..weights.loader import load_weights
from .batch import RequestSlice, StaticBatch, StepBatch, StepContext, Workspace, build_step_batch, skew_class

STATUS_MESSAGES = {
    1: "a token id outside the vocabulary reached the embedding",
    2: "a token's position has no page in its block table (write)",
    4: "a key's position has no page in its block table (read)",
    16: "a wait on a copy or tensor-core barrier ran out in the tcgen05 matrix product",
    32: "a wait on a copy or tensor-core barrier ran out in the tcgen05 attention kernel (or its shared memory did not fit)",
    64: "a wait on a copy barrier ran out in the decode attention kernel",
}


class StepError(RuntimeError):
    """A kernel of the step flagged bad input (the step's results are not to be used)."""


def require_cuda() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError(
            "turboserve_b200 runs on an NVIDIA GPU only (its layers are CUDA kernels); "
            "no CUDA device is visible to torch"
        )
    return torch.device("cuda", torch.cuda.current_device())


def load_model(model_dir: str | Path, dtype: torch.dtype, device: torch.device | str | None = None) -> DecoderModel:
    """Build the model ``config.json`` names and load ``model.safetensors`` into it."""
    device = torch.device(device) if device is not None else require_cuda()
    config = config_from_dir(model_dir)
    model = lookup(config.architecture).build_model(config, dtype, device)
    model.config = config
    load_weights(model, model_dir)
    return model


def make_groups(plan: CachePlan, page_size: int, num_pages: int | Sequence[int]) -> list[GroupSpec]:
    counts = [num_pages] * len(plan.windows) if isinstance(num_pages, int) else list(num_pages)
    return [GroupSpec(name, window, int(count), page_size)
            for name, window, count in zip(plan.group_names(), plan.windows, counts)]


class TokenRead:
    """A copy of the step's sampled ids (with their log-probabilities and the status word) to the host that is under way."""

    def __init__(self, runner: "ModelRunner", host: torch.Tensor, event: torch.cuda.Event, count: int) -> None:
        self.runner, self.host, self.event, self.count = runner, host, event, count

    def finish(self) -> list[int]:
        self.event.synchronize()
        self.runner._raise_on(int(self.host[-1]))
        return self.host[: self.count].tolist()

    def logprobs(self) -> list[float]:
        """What the in-graph sampler left for the rows that asked for a log-probability (after :meth:`finish`)."""
        slots = (self.host.numel() - 1) // 2
        return self.host[slots: slots + self.count].view(torch.float32).tolist()


class ModelRunner:
    def __init__(self, model: DecoderModel, groups: list[GroupSpec], num_state_slots: int) -> None:
        self.model = model
        self.device = model.device
        self.dtype = model.dtype
        self.plan = model.cache_plan()
        self.groups = groups
        self.storage = CacheStorage(self.plan, groups, num_state_slots, model.dtype, model.device)
        self.workspace = Workspace(model.device)
        # sampled tokens, their log-probabilities and the kernels' status word share one buffer, so that
        # the engine reads all of it with a single device-to-host copy: [0, slots) tokens, [slots, 2 slots)
        # log-probabilities (float32 bits), last element status
        self.token_buffer = torch.zeros(2 * num_state_slots + 1, dtype=torch.int32, device=model.device)
        self.token_out = self.token_buffer[:num_state_slots]
        self.logprob_out = self.token_buffer[num_state_slots: 2 * num_state_slots].view(torch.float32)
        self.status = self.token_buffer[2 * num_state_slots:]
        self._pinned: list[torch.Tensor] | None = None  # two host buffers for the ids of a step, used in turn
        self._pinned_next = 0
        self.num_steps = 0
        self.num_graph_replays = 0
        self.num_graph_captures = 0
        self.step_sampler = None
        """A sampler with per-slot options (``Sampler.use_slots``): a step that is asked to sample, and
        every captured decode graph, then ends with its kernel, which leaves the step's token ids (and
        log-probabilities) in :attr:`token_buffer` (:attr:`sampled_in_step`)."""
        self.sampled_in_step = False
        """Whether the step that ran last sampled its own tokens."""
        self._graphs: dict[tuple[int, int], tuple[torch.cuda.CUDAGraph, StaticBatch, torch.Tensor]] = {}
        self._graph_buckets: list[int] = []
        self._graph_widths: list[int] = []

    @property
    def num_groups(self) -> int:
        return len(self.groups)

    def build_batch(self, slices: Sequence[RequestSlice], **padding) -> StepBatch:
        return build_step_batch(slices, self.num_groups, self.device, **padding)

    @torch.inference_mode()
    def run(self, batch: StepBatch) -> torch.Tensor | None:
        """Run an already packed batch; returns a view of the logits buffer or ``None``."""
        ctx = StepContext(batch=batch, workspace=self.workspace, dtype=self.dtype, device=self.device, status=self.status)
        self.num_steps += 1
        return self.model.forward(ctx, self.storage)

    def step(self, slices: Sequence[RequestSlice], device_tokens: torch.Tensor | None = None,
             sample: bool = False) -> torch.Tensor | None:
        """Pack ``slices`` and run them; logits ``[wanted rows, vocab]`` fp32, in slice order.

        ``device_tokens`` (int32, on the device) replaces the token ids of the slices, which must
        then bring one token each: slice ``i`` runs ``device_tokens[i]``. It lets a decode step be
        launched while the ids it runs on, sampled by the step before, are still on the device.

        ``sample`` asks the step to end with :attr:`step_sampler` (if there is one, and no slice
        wants more than one row): one token per wanted row, by the options of the row's state slot,
        into :attr:`token_out`; :attr:`sampled_in_step` says whether it did.
        """
        vocab = self.model.vocab_size
        if device_tokens is not None:
            if any(len(piece.token_ids) != 1 for piece in slices) or device_tokens.numel() < len(slices):
                raise ValueError("device_tokens needs one token per slice")
        else:
            for piece in slices:
                for token in piece.token_ids:
                    if not 0 <= int(token) < vocab:
                        raise ValueError(f"token id {token} is outside the vocabulary of {vocab}")
        if self._graph_buckets and self._is_plain_decode(slices):
            return self._replay_decode(slices, device_tokens)  # samples whether asked or not: it is part of the graph
        self.sampled_in_step = False
        batch = self.build_batch(slices)
        if device_tokens is not None:
            batch.token_ids[: len(slices)].copy_(device_tokens[: len(slices)])
        if self.step_sampler is not None:
            # what a repetition penalty needs: the tokens of the requests that have one, by slot
            self.step_sampler.mark_seen(batch.token_ids, batch.seq_of_token, batch.state_slots, batch.num_tokens)
        logits = self.run(batch)
        rows = batch.num_logit_rows
        if (sample and self.step_sampler is not None and logits is not None and 0 < rows <= self.token_out.numel()
                and all(len(piece.want) <= 1 for piece in slices)):
            with torch.inference_mode():
                self.step_sampler.sample_by_slot(logits, batch.state_slots, batch.seq_of_token, batch.context_lens, rows,
                                                 self.token_out, row_token=batch.logit_rows, step_tokens=batch.token_ids,
                                                 logprobs=self.logprob_out)
            self.sampled_in_step = True
        return logits

    # -- decode steps from captured graphs -------------------------------------------------------

    def reserve(self, max_tokens: int, max_rows: int) -> None:
        """Size every scratch buffer for the largest step, then forbid growth.

        A captured graph holds the addresses of the buffers it was captured with, so they
        must never be reallocated afterwards. One padded dry run (tokens that belong to no
        request touch no page) brings every buffer to its final size.
        """
        batch = self.build_batch([], pad_tokens_to=max_tokens, pad_seqs_to=1, pad_rows_to=max_rows)
        self.run(batch)
        torch.cuda.synchronize(self.device)
        self.status.zero_()
        self.workspace.frozen = True

    def enable_graphs(self, max_seqs: int, max_model_len: int, max_tokens: int | None = None) -> None:
        """Replay decode-only steps of up to ``max_seqs`` requests from CUDA graphs.

        Batch sizes are padded to the next power of two; a graph is captured the first time
        its size is needed. Block tables in a graph are ``max_model_len`` tokens wide.
        """
        if self._graph_buckets:
            return
        if not self.model.graph_safe:
            return  # a part of this model may step on the host (Part.graph_safe): it runs eagerly
        self.reserve(max(max_tokens or 0, max_seqs, 1), max_seqs)
        buckets, b = [], 1
        while b < max_seqs:
            buckets.append(b)
            b *= 2
        buckets.append(max_seqs)
        self._graph_widths = [max(1, -(-max_model_len // g.page_size)) for g in self.groups]
        # a dry decode step of the largest size brings the decode kernels' scratch to its final size
        self.workspace.frozen = False
        largest = StaticBatch(max_seqs, max_seqs, self._graph_widths, self.device)
        largest.load_decode([])
        self.run(largest.batch)
        torch.cuda.synchronize(self.device)
        self.status.zero_()
        self.workspace.frozen = True
        self._graph_buckets = buckets

    def _is_plain_decode(self, slices: Sequence[RequestSlice]) -> bool:
        if not slices or len(slices) > self._graph_buckets[-1]:
            return False
        for piece in slices:
            if len(piece.token_ids) != 1 or list(piece.want) != [0]:
                return False
            if any(len(t) > w for t, w in zip(piece.block_tables, self._graph_widths)):
                return False
        return True

    @torch.inference_mode()
    def _capture(self, bucket: int, skew: int, slices: Sequence[RequestSlice] = (),
                 device_tokens: torch.Tensor | None = None):
        """Capture the decode graph of ``bucket`` requests at lopsidedness ``skew``.

        The kernels' grids depend on the batch size and the class alone, so the capture may run on
        a batch of padding tokens (which touch no page) as well as on the step that first needs it.
        """
        static = StaticBatch(bucket, bucket, self._graph_widths, self.device, *self._decode_item_plan())
        static.load_decode(slices)
        static.batch.decode_skew = skew
        if skew >= 4 and not static.batch.decode_items:
            static.batch.decode_items = static._items  # a capture on padding tokens: the kernels still walk the (empty) lists
        if device_tokens is not None:
            static.batch.token_ids[: len(slices)].copy_(device_tokens[: len(slices)])
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            self.run(static.batch)  # warm-up outside the capture: compiles, cuBLAS handles
        torch.cuda.current_stream(self.device).wait_stream(stream)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            logits = self.run(static.batch)
            if self.step_sampler is not None:
                batch = static.batch  # row i holds the logits of token i, which is request i's (or padding)
                self.step_sampler.sample_by_slot(logits, batch.state_slots, batch.seq_of_token, batch.context_lens,
                                                 bucket, self.token_out, step_tokens=batch.token_ids,
                                                 logprobs=self.logprob_out)
        entry = (graph, static, logits)
        self._graphs[(bucket, skew)] = entry
        self.num_graph_captures += 1
        # the warm-up and the capture ran the step's side effects on this very batch already:
        # the cache holds these tokens; replaying once more writes the same values again
        return entry

    def _decode_item_plan(self) -> tuple[list[int | None], list[int]]:
        """Per cache group: its window, and into how many parts the requests of a lopsided decode
        step are cut together there (by the fewest kv heads of the group's layers)."""
        from ..ops.attention_bf16 import decode_item_target
        from ..ops.skinny import num_sms

        targets = []
        for g in range(len(self.plan.windows)):
            heads = [run.need.num_kv_heads for run in self.plan.runs if run.kind == "paged" and run.group == g]
            targets.append(decode_item_target(min(heads, default=1), num_sms(self.device)))
        return list(self.plan.windows), targets

    def capture_decode_graphs(self, skew_classes: Sequence[int] = (1,)) -> int:
        """Capture the decode graphs of every batch-size bucket for the given classes now, so that
        no request meets a capture (a warm-up step, a synchronisation and the capture itself) in
        the middle of serving. Lopsided batches of other classes are still captured when first met.
        Returns how many graphs were captured."""
        before = self.num_graph_captures
        for bucket in self._graph_buckets:
            for skew in skew_classes:
                if (bucket, skew) not in self._graphs:
                    self._capture(bucket, skew)
        self.status.zero_()
        return self.num_graph_captures - before

    @torch.inference_mode()
    def _replay_decode(self, slices: Sequence[RequestSlice], device_tokens: torch.Tensor | None = None) -> torch.Tensor:
        bucket = next(b for b in self._graph_buckets if b >= len(slices))
        # the kernels' grids are part of a graph, and decode attention has other grids for a lopsided
        # batch: one graph per (batch size, class 1, 2 or "4 and up"), captured at start-up or when first needed
        # classes 1 and 2 differ in the number of parts every request is cut into; from 4 on attention
        # walks a work list made from the lengths: one graph serves them all
        key = (bucket, min(4, skew_class([piece.start_position + 1 for piece in slices])))
        entry = self._graphs.get(key)
        if entry is None:
            entry = self._capture(bucket, key[1], slices, device_tokens)
        graph, static, logits = entry
        static.load_decode(slices)
        if device_tokens is not None:
            static.batch.token_ids[: len(slices)].copy_(device_tokens[: len(slices)])
        graph.replay()
        self.num_steps += 1
        self.num_graph_replays += 1
        self.sampled_in_step = self.step_sampler is not None
        return logits[: len(slices)]

    def start_token_read(self, count: int) -> "TokenRead":
        """Queue the copy of the sampled ids and the status word to the host; ``finish`` waits for it.

        Stream order puts the copy before anything launched later, so the next step may be
        launched (and may overwrite ``token_buffer``) before the ids have been looked at.
        """
        if self._pinned is None:
            self._pinned = [torch.zeros(self.token_buffer.numel(), dtype=torch.int32).pin_memory() for _ in range(2)]
        host = self._pinned[self._pinned_next]
        self._pinned_next ^= 1
        host.copy_(self.token_buffer, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return TokenRead(self, host, event, count)

    def read_tokens(self, count: int) -> list[int]:
        """Sampled token ids of the step (written to ``token_buffer`` by the sampler) and the status check, in one copy."""
        values = self.token_buffer.tolist()
        self._raise_on(values[-1])
        return values[:count]

    def check_status(self) -> None:
        """Raise if a kernel flagged bad input since the last check (synchronises)."""
        self._raise_on(int(self.status.item()))

    def _raise_on(self, bits: int) -> None:
        if bits:
            self.status.zero_()
            reasons = [text for bit, text in STATUS_MESSAGES.items() if bits & bit]
            raise StepError("; ".join(reasons) or f"status {bits}")

    def reset_state_slot(self, slot: int) -> None:
        self.storage.reset_state_slot(slot)
