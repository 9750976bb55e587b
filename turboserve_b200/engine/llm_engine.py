"""The Python entry point: requests in, tokens out, one step at a time.

``LLMEngine(EngineConfig(model=...))`` loads the model folder, sizes and allocates the paged
cache, and is then driven with :meth:`add_request` and :meth:`step` until
:meth:`has_unfinished` is false; :meth:`generate` does that for a list of prompts. Names and
meanings follow ``src/turboserve/engine/runtime/engine.py:118-508`` (``add_request`` ``:283``,
``step`` ``:340``, ``generate`` ``:414``, ``abort``, ``stats``, ``close``); every collaborator
can be injected through the constructor, as there (``:125-146``). Prompts are token ids; text
is accepted when a tokenizer object with ``encode``/``decode`` is passed in.
"""

from __future__ import annotations

import random
import time
from typing import Any, Sequence as SequenceABC

import torch

from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig, FinishReason, RequestOutput, SamplingParams
from ..sampling.sampler import Sampler, SamplerOutput, SamplingRow
from .memory import KVCacheSizing, size_kv_cache
from .runner import ModelRunner, load_model, make_groups, require_cuda
from .scheduler import Scheduler, SchedulerOutput
from .sequence import Sequence


class _Flight:
    """A step that has been launched: its plan, and how to get at the ids it samples."""

    def __init__(self, plan: SchedulerOutput, rows, read, logprobs, ids: list[int] | None = None,
                 logprobs_in_read: bool = False, in_step: bool = False) -> None:
        self.plan, self.rows, self.read, self.logprobs, self.ids = plan, rows, read, logprobs, ids
        self.logprobs_in_read = logprobs_in_read  # the step sampled itself: log-probabilities come with the ids
        self.in_step = in_step  # sampled by the step itself, from the options and histories on the device

    def result(self) -> SamplerOutput | None:
        if self.rows is None:
            return None
        ids = self.read.finish() if self.read is not None else self.ids
        if self.logprobs_in_read:
            values = self.read.logprobs()
        elif self.logprobs is not None:
            values = self.logprobs.tolist()
        else:
            return SamplerOutput(ids)
        return SamplerOutput(ids, [v if r.params.logprobs else float("nan") for v, r in zip(values, self.rows)])


class LLMEngine:
    def __init__(self, config: EngineConfig, *, model: Any = None, runner: ModelRunner | None = None,
                 cache: CacheManager | None = None, scheduler: Scheduler | None = None,
                 sampler: Sampler | None = None, tokenizer: Any = None) -> None:
        self.config = config
        self.tokenizer = tokenizer
        self.sizing: KVCacheSizing | None = None
        if runner is None:
            device = require_cuda()
            dtype = config.resolved_dtype()
            if model is None:
                model = load_model(config.model, dtype, device)
            plan = model.cache_plan()
            itemsize = torch.empty((), dtype=dtype).element_size()
            self.sizing = size_kv_cache(
                plan, config.scheduler, itemsize, scratch_per_token=model.scratch_bytes_per_token(itemsize),
                vocab=model.vocab_size, gpu_memory_utilization=config.gpu_memory_utilization,
                max_model_len=config.max_model_len, device=device,
            )
            groups = make_groups(plan, config.scheduler.block_size, self.sizing.num_blocks)
            runner = ModelRunner(model, groups, config.scheduler.max_num_seqs)
        self.runner = runner
        self.model = runner.model
        if cache is None:
            cache = scheduler.cache if scheduler is not None else CacheManager(runner.groups, config.scheduler.max_num_seqs)
        self.cache = cache
        self.scheduler = scheduler if scheduler is not None else Scheduler(config.scheduler, cache)
        self.scheduler.copy_tables = False  # a step runs before anything else can touch the tables
        if sampler is None:
            # a runner whose captured graphs already end with a sampler keeps that sampler: its options by
            # state slot are what those graphs read
            sampler = getattr(runner, "step_sampler", None) or Sampler(runner.device)
        self.sampler = sampler
        self._eos_token_ids = frozenset(int(t) for t in getattr(self.model.spec, "eos_token_ids", ()))
        self._seed_source = random.Random(config.seed)
        self._num_generated_tokens = 0
        self._num_prompt_tokens = 0
        self._step_seconds = 0.0
        self._closed = False
        self._generate_calls = 0
        self._in_flight: _Flight | None = None
        self._num_overlapped_steps = 0
        if hasattr(self.sampler, "use_slots") and hasattr(self.runner, "step_sampler"):
            captured_with = self.runner.step_sampler
            if captured_with is self.sampler or not getattr(self.runner, "_graphs", None):
                # options and histories by state slot on the device: a step samples its own tokens (inside the
                # captured graph where there is one); as many slots as the runner has (it may have been built
                # for more requests than this engine admits)
                self.sampler.use_slots(max(config.scheduler.max_num_seqs, self.runner.token_out.numel()),
                                       self.model.vocab_size)
                self.runner.step_sampler = self.sampler
            else:
                self.runner.step_sampler = None  # graphs captured with another sampler: their ids are not used
        if config.cuda_graphs and hasattr(self.runner, "enable_graphs"):
            pages = min(g.num_pages for g in self.runner.groups)
            longest = min(config.max_model_len or pages * config.block_size, pages * config.block_size)
            self.runner.enable_graphs(config.scheduler.max_num_seqs, longest, config.scheduler.max_num_batched_tokens)
            if config.capture_graphs_at_start and hasattr(self.runner, "capture_decode_graphs"):
                self.runner.capture_decode_graphs()

    # -- context manager ---------------------------------------------------------------------

    def __enter__(self) -> "LLMEngine":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    @property
    def eos_token_ids(self) -> frozenset[int]:
        return self._eos_token_ids

    @property
    def device(self) -> torch.device:
        return self.runner.device

    @property
    def dtype(self) -> torch.dtype:
        return self.runner.dtype

    # -- requests ----------------------------------------------------------------------------

    def encode(self, prompt: str) -> list[int]:
        encode = getattr(self.tokenizer, "encode", None)
        if encode is None:
            raise TypeError("text prompts need a tokenizer; pass token ids or give the engine a tokenizer")
        return [int(t) for t in encode(prompt, add_special_tokens=False)]

    def add_request(self, request_id: str, prompt: str | SequenceABC[int], sampling: SamplingParams | None = None,
                    *, arrival: float | None = None) -> Sequence:
        if self._closed:
            raise RuntimeError("the engine is closed")
        tokens = self.encode(prompt) if isinstance(prompt, str) else [int(t) for t in prompt]
        vocab = self.model.vocab_size
        for token in tokens:
            if not 0 <= token < vocab:
                raise ValueError(f"token id {token} is outside the vocabulary of {vocab}")
        seq = self.scheduler.add_request(request_id, tokens, sampling, arrival,
                                         seed=self._seed_source.getrandbits(63))
        self._num_prompt_tokens += len(tokens)
        return seq

    def abort(self, request_id: str) -> bool:
        return self.scheduler.abort(request_id)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    # -- the loop ----------------------------------------------------------------------------

    def step(self) -> list[RequestOutput]:
        """Schedule one batch, run it, sample, and report every request that made progress.

        With ``overlap_decode`` the step after this one is launched before this one's tokens are
        read, whenever it is certain to be the same requests one token on
        (:meth:`Scheduler.continue_decode`): it takes its token ids from the device, where the
        sampler of this step leaves them. The host's work between two steps then runs while the
        GPU is busy. What a call returns does not change: the tokens of one step.
        """
        started = time.perf_counter()
        outputs: list[RequestOutput] = []
        flight, self._in_flight = self._in_flight, None
        if flight is None:
            plan = self.scheduler.schedule()
            outputs = [seq.to_output(full=True) for seq in plan.dropped]
            for seq in plan.admitted:
                if seq.request_id in self.cache:
                    slot = self.cache.state_slot(seq.request_id)
                    self.runner.reset_state_slot(slot)
                    if getattr(self.sampler, "slots", None) is not None:
                        self.sampler.slots.set(slot, seq.sampling, seq.seed, seq.num_prompt_tokens)
            if plan.is_empty:
                return outputs
            flight = self._launch(plan, ahead=False)
        try:
            ahead = self._plan_ahead(flight)
            if ahead is not None:
                self._in_flight = self._launch(ahead, ahead=True)
                self._num_overlapped_steps += 1
            outputs += self._process(flight.plan, flight.result())
        except BaseException:
            self._abandon(flight)
            raise
        if self._in_flight is not None and all(seq.is_finished for seq in self._in_flight.plan.sampling_seqs()):
            self._in_flight = None  # nobody is left to take its tokens
        self._step_seconds += time.perf_counter() - started
        return outputs

    def _abandon(self, flight: "_Flight") -> None:
        """A step failed (a kernel flagged its input, a CUDA error): end its requests.

        Their tokens of this step never arrived, and what the step wrote into their pages is
        not to be trusted; the step launched ahead of it ran on the same tokens. Left alone they
        would hold their pages with nothing left to compute and never be scheduled again, so a
        caller that catches the error and goes on stepping would spin. They finish with
        ``abort`` and give everything back; other requests are untouched.
        """
        plans = [flight.plan] + ([self._in_flight.plan] if self._in_flight is not None else [])
        self._in_flight = None
        for plan in plans:
            for item in plan.scheduled:
                if not item.seq.is_finished:
                    self.scheduler.finish(item.seq, FinishReason.ABORT)

    def _plan_ahead(self, flight: "_Flight") -> SchedulerOutput | None:
        if not self.config.overlap_decode or flight.read is None:
            return None
        for seq in flight.plan.sampling_seqs():
            params = seq.sampling
            if (params.repetition_penalty != 1.0 or params.logprobs) and not flight.in_step:
                return None  # sampled from the host's copy of the history: it would need the token that is still on the device
            if seq.num_output_tokens + 1 >= params.max_tokens:
                return None  # ends with the token that is on its way: the next step has other requests
        return self.scheduler.continue_decode(flight.plan)

    def _launch(self, plan: SchedulerOutput, ahead: bool) -> "_Flight":
        """Run and sample ``plan``; the ids stay on the device until :meth:`_Flight.result`."""
        pending = 1 if ahead else 0  # tokens of a request that are sampled but not read yet: they count for the draw's index
        if getattr(self.sampler, "slots", None) is not None:
            self.sampler.slots.flush()
        logits = self.runner.step(plan.slices(), device_tokens=self.runner.token_buffer if ahead else None, sample=True)
        seqs = plan.sampling_seqs()
        if not seqs:
            return _Flight(plan, None, None, None)
        if getattr(self.runner, "sampled_in_step", False):
            # the step ended with the sampler, options and histories by state slot: the ids (and the
            # log-probabilities of the rows that want one) are in token_buffer
            rows = [SamplingRow(s.sampling, s.seed, s.num_output_tokens + pending) for s in seqs]
            return _Flight(plan, rows, self.runner.start_token_read(len(rows)), None,
                           logprobs_in_read=any(s.sampling.logprobs for s in seqs), in_step=True)
        if ahead and any(s.sampling.repetition_penalty != 1.0 for s in seqs):
            raise RuntimeError("a step launched ahead needs the histories on the device: its sampler must be the runner's step_sampler")
        rows = [SamplingRow(s.sampling, s.seed, s.num_output_tokens + pending,
                            s.token_ids if s.sampling.repetition_penalty != 1.0 else ()) for s in seqs]
        tokens, logprobs = self.sampler.sample_device(logits, rows, out=self.runner.token_out)
        if tokens.data_ptr() == self.runner.token_buffer.data_ptr():
            return _Flight(plan, rows, self.runner.start_token_read(len(rows)), logprobs)  # tokens and the status word in one copy
        ids = tokens.tolist()
        self.runner.check_status()
        return _Flight(plan, rows, None, logprobs, ids)

    def _process(self, plan: SchedulerOutput, result) -> list[RequestOutput]:
        outputs = []
        if result is None:
            return outputs
        now = time.perf_counter()
        for index, seq in enumerate(plan.sampling_seqs()):
            if seq.is_finished:
                continue  # it ended with the token before (or was aborted) while this step was under way
            token = result.token_ids[index]
            logprob = result.logprobs[index] if result.logprobs is not None else None
            self.scheduler.append_token(seq, token, self._eos_token_ids, logprob, now)
            self._num_generated_tokens += 1
            outputs.append(seq.to_output([token]))
        return outputs

    def generate(self, prompts: SequenceABC[str | SequenceABC[int]], sampling: SamplingParams | SequenceABC[SamplingParams] | None = None) -> list[RequestOutput]:
        """Run every prompt to completion; one final :class:`RequestOutput` per prompt, in order."""
        if isinstance(sampling, SamplingParams) or sampling is None:
            sampling = [sampling] * len(prompts)
        if len(sampling) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        self._generate_calls += 1
        seqs = [self.add_request(f"generate-{self._generate_calls}-{i}", p, s) for i, (p, s) in enumerate(zip(prompts, sampling))]
        while any(not s.is_finished for s in seqs):
            if not self.has_unfinished():
                break
            self.step()
        outputs = []
        for seq in seqs:
            out = seq.to_output(seq.output_token_ids, full=True)
            decode = getattr(self.tokenizer, "decode", None)
            if decode is not None:
                out.text_delta = decode(seq.output_token_ids)
            outputs.append(out)
        return outputs

    # -- reporting ---------------------------------------------------------------------------

    def stats(self) -> dict[str, Any]:
        out: dict[str, Any] = dict(self.scheduler.stats())
        out.update(
            num_generated_tokens=self._num_generated_tokens, num_prompt_tokens=self._num_prompt_tokens,
            step_seconds=self._step_seconds, num_overlapped_steps=self._num_overlapped_steps, free_pages=self.cache.free_pages(),
            num_window_releases=self.cache.num_window_releases, cache_bytes=self.runner.storage.nbytes(),
        )
        if self.sizing is not None:
            out["num_blocks"] = self.sizing.num_blocks
        return out

    def close(self) -> None:
        if self._closed:
            return
        self._in_flight = None
        self.scheduler.reset()
        self._closed = True
