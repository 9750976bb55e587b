"""Architecture-neutral description of a decoder: what the engine builds a model from.

An architecture's typed configuration (for instance :class:`Qwen2Config`) translates its own
``config.json`` keys into a :class:`ModelSpec`. Everything below the configuration layer --
parts, cache manager, step function -- sees only this description, so no part knows which
model it is in and a new architecture is a new translation, not a new engine.

A model is a list of *layers* (each a choice of mixer, feed-forward, norm and position
encoding, with that part's sizes and constants as plain parameters) and a *run order*: a list
of :class:`LayerRun` that may name a layer twice, or let a run read the cache that another run
writes.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping


def _freeze(params: Mapping[str, Any] | None) -> Mapping[str, Any]:
    return MappingProxyType(dict(params or {}))


@dataclass(frozen=True)
class PartSpec:
    """One part chosen by kind, with its sizes and constants as parameters."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        object.__setattr__(self, "params", _freeze(self.params))

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)

    def with_params(self, **changes: Any) -> "PartSpec":
        merged = dict(self.params)
        merged.update(changes)
        return PartSpec(self.kind, merged)


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: which parts it is made of and how they are arranged.

    ``position`` is handed to the mixer (a rotary encoding acts on queries and keys inside
    attention); ``None`` means the mixer receives no position encoding.
    """

    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    position: PartSpec | None = None
    block: str = "pre_norm"


@dataclass(frozen=True)
class LayerRun:
    """One entry of the run order.

    ``layer`` indexes :attr:`ModelSpec.layers`. ``cache_from`` is the index *in the run order*
    of the run whose cache this run reads instead of keeping its own; ``None`` means the run
    owns a cache (or state) of its own.
    """

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class TensorNames:
    """How an architecture's checkpoint names its tensors.

    ``layer`` is formatted with the layer index; the four part prefixes are appended to it and
    each part appends its own local names (``q_proj.weight`` and so on). ``embedding``, ``head``
    and ``final_norm`` are the prefixes of the parts around the layers. ``prefix_rewrites``
    are prefixes some exporters put in front of the decoder stack, with what the names above
    expect in their place; the first that matches a checkpoint name is applied, once
    (``src/turboserve/engine/model/weights.py:56-61,181-196``).
    """

    embedding: str = "model.embed_tokens."
    head: str = "lm_head."
    final_norm: str = "model.norm."
    layer: str = "model.layers.{index}."
    mixer: str = "self_attn."
    feed_forward: str = "mlp."
    mixer_norm: str = "input_layernorm."
    feed_forward_norm: str = "post_attention_layernorm."
    prefix_rewrites: tuple[tuple[str, str], ...] = (
        ("transformer.", "model."),
        ("language_model.model.", "model."),
        ("language_model.lm_head.", "lm_head."),
        ("model.decoder.", "model."),
    )


@dataclass(frozen=True)
class ModelSpec:
    """Everything the engine needs to build, load and step a decoder."""

    architecture: str
    hidden_size: int
    vocab_size: int
    layers: tuple[LayerSpec, ...]
    order: tuple[LayerRun, ...]
    final_norm: PartSpec
    embedding: PartSpec = PartSpec("table")
    head: PartSpec = PartSpec("linear")
    tie_word_embeddings: bool = False
    names: TensorNames = field(default_factory=TensorNames)
    eos_token_ids: tuple[int, ...] = ()
    max_position_embeddings: int = 2048
    init_std: float = 0.02

    def __post_init__(self) -> None:
        if self.hidden_size < 1 or self.vocab_size < 1:
            raise ValueError("hidden_size and vocab_size must be positive")
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.order:
            raise ValueError("the run order is empty")
        for index, run in enumerate(self.order):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"run {index} names layer {run.layer}, which does not exist")
            if run.cache_from is not None:
                if not 0 <= run.cache_from < index:
                    raise ValueError(
                        f"run {index} reads the cache of run {run.cache_from}, which must be an "
                        "earlier run"
                    )
                if self.order[run.cache_from].cache_from is not None:
                    raise ValueError(
                        f"run {index} reads the cache of run {run.cache_from}, which has none of "
                        "its own"
                    )

    @staticmethod
    def sequential(num_layers: int) -> tuple[LayerRun, ...]:
        """The ordinary order: every layer once, each with its own cache."""
        return tuple(LayerRun(layer=i) for i in range(num_layers))
