"""Continuous batching above the step function: admit, cut prompts into portions, decode,
finish and free; recompute preemption when pages run out.

Each call of :meth:`Scheduler.schedule` builds one step under two hard budgets
(``max_num_batched_tokens`` tokens, ``max_num_seqs`` requests):

1. running requests first, in admission order: a decode token, or the next portion of a
   prompt, whatever of the token budget is left;
2. then preempted requests, then waiting ones (first come, first served, no jumping the
   queue): a request is admitted when a state slot is free and the pages its whole current
   sequence needs are free; it gets pages only for the portion it runs now.

When a running request cannot grow because its page pool is empty, the most recently admitted
running request that is not already in this step gives up all its pages and its state slot
and goes to the front of the queue (recompute preemption: its prompt and the tokens it has
generated are kept and computed again later); if nobody else can be preempted the request
preempts itself. A request samples only in the step that computes its last token, so a
recompute that is cut by the token budget never samples from the middle of its own history.

The policy follows ``src/turboserve/engine/core/scheduler.py:606-802`` (order of business
``:606-640``, admissions ``:672-711``, victim choice ``:776-790``) except for the sampling
rule: the reference defines a chunk against the prompt length (``:728-738``), which samples a
spurious token when a resumed request is split after its prompt; here the rule is
``end == num_tokens``.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import CacheManager
from ..config.engine_config import FinishReason, SamplingParams, SchedulerConfig
from .batch import RequestSlice
from .sequence import Sequence, SeqStatus


@dataclass
class ScheduledSeq:
    """One request's share of a step, fixed at schedule time."""

    seq: Sequence
    start: int
    num_new_tokens: int
    token_ids: list[int]
    block_tables: list[list[int]]
    state_slot: int
    is_prefill: bool
    samples: bool

    @property
    def context_len(self) -> int:
        return self.start + self.num_new_tokens

    def to_slice(self) -> RequestSlice:
        return RequestSlice(
            token_ids=self.token_ids, start_position=self.start, block_tables=self.block_tables,
            state_slot=self.state_slot, want=[self.num_new_tokens - 1] if self.samples else [],
        )


@dataclass
class SchedulerOutput:
    scheduled: list[ScheduledSeq] = field(default_factory=list)
    preempted: list[Sequence] = field(default_factory=list)
    admitted: list[Sequence] = field(default_factory=list)
    dropped: list[Sequence] = field(default_factory=list)
    """Requests finished by the scheduler because no cache, however empty, could hold them."""
    num_prefill_seqs: int = 0
    num_decode_seqs: int = 0
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0

    @property
    def is_empty(self) -> bool:
        return not self.scheduled

    @property
    def num_tokens(self) -> int:
        return self.num_prefill_tokens + self.num_decode_tokens

    def slices(self) -> list[RequestSlice]:
        return [item.to_slice() for item in self.scheduled]

    def sampling_seqs(self) -> list[Sequence]:
        return [item.seq for item in self.scheduled if item.samples]


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager) -> None:
        self.config = config
        self.cache = cache
        self._waiting: deque[Sequence] = deque()
        self._preempted: deque[Sequence] = deque()
        self._running: list[Sequence] = []
        self._by_request: dict[str, Sequence] = {}
        self._next_seq_id = 0
        self.copy_tables = True
        """Snapshot block tables into every ScheduledSeq (off when the step runs before anything else
        can change them, as in ``LLMEngine.step``: the runner then reads the live tables)."""
        self.num_steps = 0
        self.num_preemptions = 0
        self.num_admitted = 0
        self.num_finished = 0
        self.num_prefill_tokens = 0
        self.num_decode_tokens = 0

    # -- requests --------------------------------------------------------------------------

    def add_request(self, request_id: str, prompt_token_ids, sampling: SamplingParams | None = None,
                    arrival: float | None = None, seed: int | None = None) -> Sequence:
        if request_id in self._by_request:
            raise ValueError(f"request {request_id!r} is already in flight")
        sampling = sampling if sampling is not None else SamplingParams()
        seq = Sequence(seq_id=self._next_seq_id, request_id=request_id, prompt_token_ids=list(prompt_token_ids),
                       sampling=sampling)
        seq.seed = int(sampling.seed if sampling.seed is not None else (seed if seed is not None else seq.seq_id))
        budget = self.config.max_num_batched_tokens
        if not self.cache.fits_at_all(seq.num_prompt_tokens, budget):
            raise ValueError(
                f"request {request_id!r} has {seq.num_prompt_tokens} prompt tokens, more than the cache can "
                "ever hold; shorten the prompt or enlarge the cache"
            )
        if not self.config.enable_chunked_prefill and seq.num_tokens > budget:
            raise ValueError(
                f"request {request_id!r} has {seq.num_tokens} tokens but the step budget is {budget} and "
                "chunked prefill is disabled"
            )
        self._next_seq_id += 1
        seq.timing.t_arrival = time.perf_counter() if arrival is None else arrival
        self._by_request[request_id] = seq
        self._waiting.append(seq)
        return seq

    def get(self, request_id: str) -> Sequence | None:
        return self._by_request.get(request_id)

    def has_unfinished(self) -> bool:
        return bool(self._by_request)

    @property
    def num_waiting(self) -> int:
        return len(self._waiting) + len(self._preempted)

    @property
    def num_running(self) -> int:
        return len(self._running)

    # -- one step --------------------------------------------------------------------------

    def schedule(self, now: float | None = None) -> SchedulerOutput:
        stamp = time.perf_counter() if now is None else now
        out = SchedulerOutput()
        tokens_left = self.config.max_num_batched_tokens
        seqs_left = self.config.max_num_seqs
        in_step: set[int] = set()        # seq ids that already have their share of this step
        evicted: set[int] = set()        # seq ids preempted while this step was put together
        prefills: list[ScheduledSeq] = []
        decodes: list[ScheduledSeq] = []

        def emit(seq: Sequence, num_new: int) -> None:
            nonlocal tokens_left, seqs_left
            start = seq.num_computed_tokens
            self.cache.grow(seq.request_id, num_new)
            end = start + num_new
            item = ScheduledSeq(
                seq=seq, start=start, num_new_tokens=num_new, token_ids=seq.tokens_in_range(start, end),
                block_tables=([list(t) for t in self.cache.tables(seq.request_id)] if self.copy_tables
                              else self.cache.tables(seq.request_id)),
                state_slot=self.cache.state_slot(seq.request_id),
                is_prefill=start < seq.num_prompt_tokens, samples=end == seq.num_tokens,
            )
            seq.num_computed_tokens = end
            tokens_left -= num_new
            seqs_left -= 1
            in_step.add(seq.seq_id)
            (prefills if item.is_prefill else decodes).append(item)

        # 1. running requests
        for seq in list(self._running):
            if tokens_left <= 0 or seqs_left <= 0:
                break
            if seq.status is not SeqStatus.RUNNING:
                continue  # preempted a moment ago as somebody's victim
            num_new = min(tokens_left, seq.num_uncomputed_tokens)
            if num_new <= 0:
                continue
            if not self.config.enable_chunked_prefill and num_new < seq.num_uncomputed_tokens:
                continue
            if not self._grow_or_evict(seq, num_new, in_step, evicted, out):
                continue
            emit(seq, num_new)

        # 2. preempted, then waiting
        while tokens_left > 0 and seqs_left > 0:
            from_preempted = bool(self._preempted)
            queue = self._preempted if from_preempted else self._waiting
            if not queue:
                break
            seq = queue[0]
            if not self.cache.fits_at_all(seq.num_tokens, self.config.max_num_batched_tokens):
                # it has outgrown the whole pool: end it rather than preempt it for ever
                queue.popleft()
                self.finish(seq, FinishReason.LENGTH, now=stamp)
                out.dropped.append(seq)
                continue
            if seq.seq_id in evicted:
                break
            num_new = min(tokens_left, seq.num_uncomputed_tokens)
            if not self.config.enable_chunked_prefill and num_new < seq.num_uncomputed_tokens:
                break
            if not self.cache.can_admit(seq.num_tokens, self.config.max_num_batched_tokens):
                break
            queue.popleft()
            self.cache.admit(seq.request_id)
            seq.status = SeqStatus.RUNNING
            if seq.timing.t_first_scheduled is None:
                seq.timing.t_first_scheduled = stamp
            self._running.append(seq)
            self.num_admitted += 1
            out.admitted.append(seq)
            emit(seq, num_new)

        # Prompts first, then the requests that decode, as in the reference; among the latter the
        # longest context first, so that the attention kernel starts its longest blocks first
        # (the order inside a step changes no result: every token reads its own request's cache).
        decodes.sort(key=lambda item: -item.context_len)
        out.scheduled = [*prefills, *decodes]
        out.num_prefill_seqs, out.num_decode_seqs = len(prefills), len(decodes)
        out.num_prefill_tokens = sum(i.num_new_tokens for i in prefills)
        out.num_decode_tokens = sum(i.num_new_tokens for i in decodes)
        self.num_steps += 1
        self.num_prefill_tokens += out.num_prefill_tokens
        self.num_decode_tokens += out.num_decode_tokens
        return out

    def continue_decode(self, previous: SchedulerOutput) -> SchedulerOutput | None:
        """The step after ``previous``, planned before the tokens ``previous`` samples are known.

        Possible only when that step is certain but for the token ids: every request of
        ``previous`` samples (so each is one token on, whatever the token is), these are all the
        running requests, nobody waits, and the pages for one more token each are free, so that
        :meth:`schedule` would decide exactly this. A request that turns out to have finished with
        the token of ``previous`` runs one token too many, whose result is thrown away. The
        caller checks what it knows better (length limits, what the sampler needs). Token ids in
        the plan are placeholders: the runner takes them from the device. Returns ``None`` when
        the step cannot be planned ahead.
        """
        items = previous.scheduled
        if not items or self._waiting or self._preempted or len(items) != len(self._running):
            return None
        if len(items) > self.config.max_num_seqs or len(items) > self.config.max_num_batched_tokens:
            return None
        running = {id(seq) for seq in self._running}
        for item in items:
            seq = item.seq
            if not item.samples or id(seq) not in running or seq.status is not SeqStatus.RUNNING:
                return None
            if seq.num_computed_tokens != seq.num_tokens:
                return None
        for g, (group, pool) in enumerate(zip(self.cache.groups, self.cache.pools)):
            needed = 0
            for item in items:
                rid = item.seq.request_id
                needed += max(0, -(-(self.cache.num_tokens(rid) + 1) // group.page_size) - len(self.cache.tables(rid)[g]))
            if needed > pool.num_free:
                return None
        out = SchedulerOutput()
        for item in items:
            seq = item.seq
            start = seq.num_computed_tokens
            self.cache.grow(seq.request_id, 1)
            out.scheduled.append(ScheduledSeq(
                seq=seq, start=start, num_new_tokens=1, token_ids=[0],
                block_tables=([list(t) for t in self.cache.tables(seq.request_id)] if self.copy_tables
                              else self.cache.tables(seq.request_id)),
                state_slot=self.cache.state_slot(seq.request_id), is_prefill=False, samples=True,
            ))
            seq.num_computed_tokens = start + 1  # the token itself joins the request when it has been read
        out.num_decode_seqs = out.num_decode_tokens = len(items)
        self.num_steps += 1
        self.num_decode_tokens += len(items)
        return out

    def _grow_or_evict(self, seq: Sequence, num_new: int, in_step: set[int], evicted: set[int],
                       out: SchedulerOutput) -> bool:
        """Make sure ``seq`` can take pages for ``num_new`` more tokens; ``False`` if it had to go itself.

        While its page pools cannot serve it, the running request that was admitted last, is not
        part of this step and is not ``seq`` gives everything back and is computed again later
        (``src/turboserve/engine/core/scheduler.py:748-802`` chooses the same victim); when no
        such request is left, ``seq`` is the one that goes.
        """
        while not self.cache.can_grow(seq.request_id, num_new):
            others = [r for r in self._running
                      if r is not seq and r.seq_id not in in_step and r.status is SeqStatus.RUNNING]
            loser = max(others, key=lambda r: r.seq_id) if others else seq
            self._send_back(loser, evicted, out)
            if loser is seq:
                return False
        return True

    def _send_back(self, seq: Sequence, evicted: set[int], out: SchedulerOutput) -> None:
        """Recompute preemption of one running request: pages and slot back, progress to zero,
        tokens kept, to the end of the queue that is served before new arrivals."""
        self.cache.release(seq.request_id)
        seq.reset_for_recompute()
        self._running.remove(seq)
        self._preempted.append(seq)
        evicted.add(seq.seq_id)
        out.preempted.append(seq)
        self.num_preemptions += 1

    # -- after sampling --------------------------------------------------------------------

    def append_token(self, seq: Sequence, token_id: int, eos_token_ids=(), logprob: float | None = None,
                     now: float | None = None) -> FinishReason | None:
        seq.append_token(token_id, logprob, now)
        reason = seq.check_stop(token_id, eos_token_ids)
        if reason is not None:
            self.finish(seq, reason, now=now, stop_token_id=token_id if reason is FinishReason.STOP else None)
        return reason

    def finish(self, seq: Sequence, reason: FinishReason = FinishReason.STOP, now: float | None = None,
               stop_token_id: int | None = None) -> None:
        seq.finish(reason, now, stop_token_id)
        if seq.request_id in self.cache:
            self.cache.release(seq.request_id)
        self._detach(seq)
        self.num_finished += 1

    def abort(self, request_id: str, now: float | None = None) -> bool:
        seq = self._by_request.get(request_id)
        if seq is None:
            return False
        self.finish(seq, FinishReason.ABORT, now)
        return True

    def _detach(self, seq: Sequence) -> None:
        """Take a finished request out of whichever queue holds it, and out of the index."""
        for queue in (self._running, self._preempted, self._waiting):
            if seq in queue:
                queue.remove(seq)
                break
        self._by_request.pop(seq.request_id, None)

    def reset(self) -> None:
        self._waiting.clear()
        self._preempted.clear()
        self._running.clear()
        self._by_request.clear()
        self.cache.reset()

    # -- reporting -------------------------------------------------------------------------

    def stats(self) -> dict[str, int]:
        return {
            "num_steps": self.num_steps, "num_waiting": len(self._waiting), "num_preempted": len(self._preempted),
            "num_running": len(self._running), "num_admitted": self.num_admitted, "num_finished": self.num_finished,
            "num_preemptions": self.num_preemptions, "num_prefill_tokens": self.num_prefill_tokens,
            "num_decode_tokens": self.num_decode_tokens,
        }

    def check_invariants(self) -> None:
        self.cache.check_invariants()
        ids = [s.request_id for s in [*self._waiting, *self._preempted, *self._running]]
        if len(set(ids)) != len(ids):
            raise AssertionError("a request is in two queues")
        if set(ids) != set(self._by_request):
            raise AssertionError("the request index and the queues disagree")
        for seq in self._running:
            if seq.status is not SeqStatus.RUNNING or seq.request_id not in self.cache:
                raise AssertionError(f"{seq.request_id!r} runs without cache")
            if self.cache.num_tokens(seq.request_id) != seq.num_computed_tokens:
                raise AssertionError(f"{seq.request_id!r}: pages cover {self.cache.num_tokens(seq.request_id)} tokens, computed {seq.num_computed_tokens}")
        for seq in [*self._waiting, *self._preempted]:
            if seq.request_id in self.cache or seq.num_computed_tokens:
                raise AssertionError(f"{seq.request_id!r} waits but holds cache")
        if len(self._running) > self.config.max_num_seqs:
            raise AssertionError("more running requests than max_num_seqs")
