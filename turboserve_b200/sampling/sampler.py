"""Turns rows of logits into token ids on the device, with per-request options.

The stages and their order are the reference's (``src/turboserve/engine/core/sampler.py:
190-238``): repetition penalty, log-probabilities, temperature, top-k, top-p, then argmax for
greedy rows and a draw for the rest. The reference draws with ``torch.multinomial`` and one
``torch.Generator`` per seeded request (``:258-297``); here a draw is the Gumbel-max rule over
counter-based uniforms of (request seed, index of the generated token, vocabulary id), so a
request's tokens do not depend on its batch neighbours, on how often it was preempted, or on
any global generator. All of it is one kernel (``sampling.cu``); a batch of plain greedy rows
takes the argmax kernel, which needs no scratch.

Per-request options also live on the device, by state slot (:class:`SlotOptions`): they are
written once, when a request is admitted, and a decode step finds them through the step's
``state_slots``; the index of the token being generated follows from the request's length, so
nothing has to be sent or advanced per step, and a step ends with the sampling kernel, inside
the captured graph where there is one (:meth:`Sampler.sample_by_slot`). The history that a
repetition penalty needs is there too, as one bit per vocabulary entry and slot: the tokens a
step runs are marked by :meth:`Sampler.mark_seen` (portions of prompts, and everything that is
computed again after a preemption) or by the sampling kernel itself (the one token a request ran
in a replayed decode step), so a penalised row needs nothing from the host either.
:meth:`Sampler.sample_device` is the same sampler for callers that have no slots: options and
histories come as lists and go up with the call.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence as SequenceABC

import torch

from ..config.engine_config import SamplingParams
from ..ops import kernels


@dataclass
class SamplerOutput:
    token_ids: list[int]
    logprobs: list[float] | None = None


@dataclass
class SamplingRow:
    """What the sampler needs to know about one row."""

    params: SamplingParams
    seed: int = 0
    counter: int = 0
    history: SequenceABC[int] = ()


SLOT_CHUNKS = 8
"""Blocks a row is cut into when one pass over it is enough (greedy, or a draw without top-k and top-p)."""


class SlotOptions:
    """Sampling options of the live requests on the device, one entry per state slot.

    ``temperature``, ``top_p``, ``penalty`` (float32), ``top_k``, ``prompt_len``, ``want_logprob``
    (int32) and ``seed`` (int64) are arrays over the slots. A host mirror in pinned memory is
    changed at admission and copied over whole (a few hundred bytes, on the stream, so in order
    with the steps around it). ``seen`` (int32 ``[slots, ceil(vocab / 32)]``) is the bitmap of
    the tokens each slot's request holds; the row of a slot that goes to a request with a penalty
    is cleared by the same :meth:`flush`.
    """

    def __init__(self, num_slots: int, vocab: int, device: torch.device) -> None:
        self.num_slots, self.vocab = int(num_slots), int(vocab)
        n = self.num_slots
        pin = device.type == "cuda"
        self._host_f = torch.zeros(3 * n, dtype=torch.float32)
        self._host_i = torch.zeros(3 * n, dtype=torch.int32)
        self._host_s = torch.zeros(n, dtype=torch.int64)
        if pin:
            self._host_f, self._host_i, self._host_s = self._host_f.pin_memory(), self._host_i.pin_memory(), self._host_s.pin_memory()
        self._host_f[n:] = 1.0  # top_p, penalty
        self._dev_f = self._host_f.to(device)
        self._dev_i = self._host_i.to(device)
        self.seed = self._host_s.to(device)
        self.temperature, self.top_p, self.penalty = self._dev_f[:n], self._dev_f[n:2 * n], self._dev_f[2 * n:]
        self.top_k, self.prompt_len, self.want_logprob = self._dev_i[:n], self._dev_i[n:2 * n], self._dev_i[2 * n:]
        self.seen = torch.zeros(n, (self.vocab + 31) // 32, dtype=torch.int32, device=device)
        self._dirty = False
        self._to_clear: list[int] = []
        self._penalised: set[int] = set()

    @property
    def any_penalty(self) -> bool:
        """Whether any slot holds a request with a penalty (only then do a step's tokens have to be marked)."""
        return bool(self._penalised)

    def set(self, slot: int, params: SamplingParams, seed: int, num_prompt_tokens: int) -> None:
        n = self.num_slots
        self._host_f[slot] = params.temperature
        self._host_f[n + slot] = params.top_p
        self._host_f[2 * n + slot] = params.repetition_penalty
        self._host_i[slot] = params.top_k
        self._host_i[n + slot] = num_prompt_tokens
        self._host_i[2 * n + slot] = 1 if params.logprobs else 0
        self._host_s[slot] = seed & 0x7FFFFFFFFFFFFFFF
        if params.repetition_penalty != 1.0:
            self._to_clear.append(slot)  # what the slot's last request had seen is not this one's
            self._penalised.add(slot)
        else:
            self._penalised.discard(slot)
        self._dirty = True

    def flush(self) -> None:
        """Bring the device arrays up to date (before the step that first uses what was set)."""
        if self._dirty:
            self._dev_f.copy_(self._host_f, non_blocking=True)
            self._dev_i.copy_(self._host_i, non_blocking=True)
            self.seed.copy_(self._host_s, non_blocking=True)
            for slot in self._to_clear:
                self.seen[slot].zero_()
            self._to_clear.clear()
            self._dirty = False


class Sampler:
    def __init__(self, device: torch.device | str) -> None:
        self.device = torch.device(device)
        self._work: torch.Tensor | None = None
        self.slots: SlotOptions | None = None
        self._partial: torch.Tensor | None = None

    def use_slots(self, num_slots: int, vocab: int) -> SlotOptions:
        """Keep per-request options on the device for up to ``num_slots`` requests; sizes the scratch
        of :meth:`sample_by_slot` once, so that it can be part of a captured graph."""
        if self.slots is None or self.slots.num_slots < num_slots or self.slots.vocab != vocab:
            self.slots = SlotOptions(num_slots, vocab, self.device)
            self._partial = torch.zeros(num_slots * (4 * SLOT_CHUNKS + 1), dtype=torch.int32, device=self.device)
        self._scratch(num_slots, vocab)
        return self.slots

    def sample_by_slot(self, logits: torch.Tensor, seq_slot: torch.Tensor, seq_of_token: torch.Tensor | None,
                       seq_context: torch.Tensor, num_rows: int, out: torch.Tensor, *,
                       row_token: torch.Tensor | None = None, step_tokens: torch.Tensor | None = None,
                       logprobs: torch.Tensor | None = None) -> torch.Tensor:
        """Sample ``num_rows`` rows whose options are in :attr:`slots`; ids into ``out``. Allocates nothing.

        The arguments are a step's own index arrays: ``row_token`` (per row: the token whose logits
        it holds; without it row ``i`` is token ``i``), ``seq_of_token`` (per token: its request in the
        step, negative for padding), ``seq_slot`` and ``seq_context`` (per request: state slot, length
        after the step). ``step_tokens`` (per token: its id) joins the request's history before a
        penalty reads it; without it the history is what :meth:`mark_seen` has marked. ``logprobs``
        (float32 per row) takes the log-probability of the chosen token for the rows whose request
        asked for it; without it nobody gets one.
        """
        if self.slots is None or self._partial is None:
            raise RuntimeError("use_slots() first")
        slots = self.slots
        kernels.sample_slots(
            logits, self._scratch(num_rows, logits.shape[1]), out, num_rows, temperature=slots.temperature, top_k=slots.top_k,
            top_p=slots.top_p, seed=slots.seed, prompt_len=slots.prompt_len, seq_slot=seq_slot, seq_context=seq_context,
            partial=self._partial, chunks=SLOT_CHUNKS, row_token=row_token, seq_of_token=seq_of_token, step_tokens=step_tokens,
            penalty=slots.penalty, seen=slots.seen, want_logprob=slots.want_logprob if logprobs is not None else None,
            logprobs=logprobs,
        )
        return out[:num_rows]

    def mark_seen(self, token_ids: torch.Tensor, seq_of_token: torch.Tensor, state_slots: torch.Tensor, num_tokens: int) -> None:
        """Add a step's tokens to the histories of the requests that have a penalty (a kernel, nothing if no slot has one)."""
        if self.slots is None or not self.slots.any_penalty:
            return
        kernels.mark_seen(token_ids, seq_of_token, state_slots, self.slots.penalty, self.slots.seen, num_tokens, self.slots.vocab)

    def _scratch(self, rows: int, vocab: int) -> torch.Tensor:
        need = rows * vocab
        if self._work is None or self._work.numel() < need:
            self._work = torch.empty(need, dtype=torch.float32, device=self.device)
        return self._work

    def sample_device(self, logits: torch.Tensor, rows: SequenceABC[SamplingRow],
                      out: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor | None]:
        """Sample without leaving the device: int32 token ids ``[n]`` (into ``out`` if given) and optional logprobs."""
        n = len(rows)
        if logits.dim() != 2 or logits.shape[0] < n:
            raise ValueError(f"{n} sampling rows for logits of shape {tuple(logits.shape)}")
        tokens = out[:n] if out is not None and out.numel() >= n else torch.empty(n, dtype=torch.int32, device=self.device)
        if n == 0:
            return tokens, None
        plain_greedy = all(r.params.is_greedy and r.params.repetition_penalty == 1.0 and not r.params.logprobs for r in rows)
        if plain_greedy:
            kernels.argmax(logits, tokens, n)
            return tokens, None
        vocab = logits.shape[1]
        want_logprobs = any(r.params.logprobs for r in rows)
        use_penalty = any(r.params.repetition_penalty != 1.0 for r in rows)
        floats = [r.params.temperature for r in rows] + [r.params.top_p for r in rows] + [r.params.repetition_penalty for r in rows]
        ints = [min(r.params.top_k, vocab) for r in rows] + [r.counter & 0x7FFFFFFF for r in rows]
        starts = [0]
        history: list[int] = []
        if use_penalty:
            for r in rows:
                if r.params.repetition_penalty != 1.0:
                    history.extend(int(t) for t in r.history)
                starts.append(len(history))
            ints += starts + history
        f_dev = torch.tensor(floats, dtype=torch.float32).to(self.device, non_blocking=True)
        i_dev = torch.tensor(ints, dtype=torch.int32).to(self.device, non_blocking=True)
        seeds = [r.seed & 0x7FFFFFFFFFFFFFFF for r in rows]
        s_dev = torch.tensor(seeds, dtype=torch.int64).to(self.device, non_blocking=True)
        logprobs = torch.empty(n, dtype=torch.float32, device=self.device) if want_logprobs else None
        kernels.sample(
            logits, self._scratch(n, vocab), tokens, num_rows=n,
            temperature=f_dev[0:n], top_p=f_dev[n:2 * n], penalty=f_dev[2 * n:3 * n] if use_penalty else None,
            top_k=i_dev[0:n], counter=i_dev[n:2 * n], seed=s_dev,
            history_start=i_dev[2 * n:3 * n + 1] if use_penalty else None,
            history=i_dev[3 * n + 1:] if use_penalty and history else (i_dev[0:1] if use_penalty else None),
            logprobs=logprobs,
        )
        return tokens, logprobs

    def sample(self, logits: torch.Tensor, rows: SequenceABC[SamplingRow]) -> SamplerOutput:
        """Sample and bring the ids to the host (the step's one synchronisation)."""
        tokens, logprobs = self.sample_device(logits, rows)
        ids = tokens.tolist()
        if logprobs is None:
            return SamplerOutput(ids)
        values = logprobs.tolist()
        return SamplerOutput(ids, [v if r.params.logprobs else float("nan") for v, r in zip(values, rows)])
