"""Options of the engine, the scheduler and of one request, with the reference's names.

Field names, defaults and meanings follow ``src/turboserve/engine/core/types.py``:
``SamplingParams`` (``:97-124``), ``FinishReason`` (``:127-143``), ``RequestTiming``
(``:146-193``), ``SchedulerConfig`` (``:484-518``), ``EngineConfig`` (``:521-593``) and
``RequestOutput`` (``:596-634``). Options of subsystems this engine does not have (prefix
caching, tenant policies, LoRA, speculative decoding, stop strings) are absent rather than
accepted and ignored. ``auto`` dtype resolves to bfloat16: the engine runs on one kind of GPU.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Literal

import torch
from pydantic import BaseModel, ConfigDict, Field, model_validator

DTypeName = Literal["auto", "bfloat16", "float32"]

DTYPE_BY_NAME: dict[str, torch.dtype] = {
    "bfloat16": torch.bfloat16,
    "float32": torch.float32,
}


def resolve_dtype(dtype: str | torch.dtype) -> torch.dtype:
    """Map a dtype name onto a ``torch.dtype``; ``auto`` means bfloat16."""
    if isinstance(dtype, torch.dtype):
        if dtype not in DTYPE_BY_NAME.values():
            raise ValueError(f"unsupported dtype {dtype}; expected one of {sorted(DTYPE_BY_NAME)}")
        return dtype
    if dtype == "auto":
        return torch.bfloat16
    try:
        return DTYPE_BY_NAME[dtype]
    except KeyError:
        raise ValueError(
            f"unsupported dtype {dtype!r}; expected one of {sorted(DTYPE_BY_NAME)} or 'auto'"
        ) from None


class SamplingParams(BaseModel):
    """How one request turns logits into tokens and when it stops.

    ``temperature == 0`` is greedy; ``top_k == 0`` and ``top_p == 1`` switch those filters
    off; ``seed`` makes a request's draws independent of its batch neighbours.
    """

    model_config = ConfigDict(extra="forbid", validate_assignment=True)

    max_tokens: int = Field(default=128, ge=1)
    temperature: float = Field(default=1.0, ge=0.0)
    top_p: float = Field(default=1.0, gt=0.0, le=1.0)
    top_k: int = Field(default=0, ge=0)
    seed: int | None = None
    stop_token_ids: list[int] = Field(default_factory=list)
    repetition_penalty: float = Field(default=1.0, gt=0.0)
    ignore_eos: bool = False
    logprobs: bool = False

    @property
    def is_greedy(self) -> bool:
        return self.temperature == 0.0


class FinishReason(str, Enum):
    STOP = "stop"
    LENGTH = "length"
    ABORT = "abort"

    def __str__(self) -> str:
        return self.value


@dataclass
class RequestTiming:
    """``time.perf_counter()`` stamps of a request's life, ``None`` until reached."""

    t_arrival: float | None = None
    t_first_scheduled: float | None = None
    t_first_token: float | None = None
    t_last_token: float | None = None
    t_finished: float | None = None
    num_preemptions: int = 0

    @property
    def ttft(self) -> float | None:
        if self.t_arrival is None or self.t_first_token is None:
            return None
        return self.t_first_token - self.t_arrival


class SchedulerConfig(BaseModel):
    """Limits of one scheduler step and the geometry of the paged cache."""

    model_config = ConfigDict(extra="forbid", validate_assignment=True)

    max_num_seqs: int = Field(default=64, ge=1)
    max_num_batched_tokens: int = Field(default=2048, ge=1)
    block_size: int = Field(default=16, ge=1)
    num_blocks: int | None = Field(default=None, ge=1)
    enable_chunked_prefill: bool = True
    policy: Literal["fcfs"] = "fcfs"

    @model_validator(mode="after")
    def _check(self) -> "SchedulerConfig":
        if self.block_size & (self.block_size - 1):
            raise ValueError(f"block_size must be a power of two, got {self.block_size}")
        if self.max_num_batched_tokens < self.block_size:
            raise ValueError(
                f"max_num_batched_tokens ({self.max_num_batched_tokens}) must be at least one "
                f"block ({self.block_size})"
            )
        return self


class EngineConfig(BaseModel):
    """Everything needed to build an engine."""

    model_config = ConfigDict(extra="forbid", validate_assignment=True)

    model: str
    """Folder holding ``config.json`` and ``model.safetensors``."""

    dtype: DTypeName = "auto"
    device: Literal["auto", "cuda"] = "auto"
    gpu_memory_utilization: float = Field(default=0.9, gt=0.0, le=1.0)
    max_model_len: int | None = Field(default=None, ge=1)
    seed: int | None = None
    scheduler: SchedulerConfig = Field(default_factory=SchedulerConfig)
    cuda_graphs: bool = True
    """Replay decode-only steps from captured CUDA graphs."""

    capture_graphs_at_start: bool = True
    """Capture the decode graphs of every batch size when the engine is built, instead of when a
    batch size is first met in the middle of serving (lopsided batches, whose attention is cut
    finer, are still captured when first met)."""

    overlap_decode: bool = True
    """Launch the next decode step before the tokens of the current one have been read, when that
    step is certain to hold the same requests one token on (``LLMEngine.step``)."""

    @property
    def block_size(self) -> int:
        return self.scheduler.block_size

    @property
    def num_blocks(self) -> int | None:
        return self.scheduler.num_blocks

    def resolved_device(self) -> str:
        return "cuda"

    def resolved_dtype(self) -> torch.dtype:
        return resolve_dtype(self.dtype)


@dataclass
class RequestOutput:
    """One step's progress on one request: new tokens as a delta, counts as totals."""

    request_id: str
    new_token_ids: list[int] = field(default_factory=list)
    text_delta: str = ""
    finished: bool = False
    finish_reason: FinishReason | None = None
    timing: RequestTiming = field(default_factory=RequestTiming)
    prompt_tokens: int = 0
    output_tokens: int = 0
    token_ids: list[int] = field(default_factory=list)
    """All generated token ids so far (filled by ``LLMEngine.generate``'s final outputs)."""
    logprobs: list[float] | None = None

    @property
    def total_tokens(self) -> int:
        return self.prompt_tokens + self.output_tokens

    def usage(self) -> dict[str, int]:
        return {
            "prompt_tokens": self.prompt_tokens,
            "completion_tokens": self.output_tokens,
            "total_tokens": self.total_tokens,
        }
