"""Interfaces of the parts a layer is put together from, and their registries.

A layer is a *mixer* (attention here), a *feed-forward*, two *norms* and optionally a
*position encoding*, arranged by a *block*; around the layers stand a *token embedding* (ids to
the residual stream) and a *logit head* (final rows to logits). Every part

* is chosen by ``PartSpec.kind`` through a registry, layer by layer, so one model can have
  different mixers and feed-forwards in different layers;
* takes its sizes and constants from ``PartSpec.params`` and from the arguments of its
  constructor, never from a model configuration: no part knows which model it is in;
* declares its tensors with :class:`ParamSpec` (local names such as ``q_proj.weight``; the
  architecture's :class:`~turboserve_b200.config.TensorNames` gives the prefixes) and receives
  them, already on the device and in their final dtype, through ``bind``;
* (mixers only) declares what it keeps per request: pages of keys and values
  (:class:`PagedKVNeed`), a fixed-size state (:class:`StateNeed`), or nothing.

Registering a new kind is one call (``register_mixer("name", cls)``); nothing else in the
framework has to change for the model builder, the loader, the cache manager and the step
function to use it.

Constructor signatures
    mixer          ``cls(spec, hidden_size, dtype, device, position=None, shares_cache=False)``
    feed-forward   ``cls(spec, hidden_size, dtype, device)``
    norm           ``cls(spec, hidden_size, dtype, device)``
    position       ``cls(spec, device)``
    block          ``cls(mixer, feed_forward, mixer_norm, feed_forward_norm)``
    embedding      ``cls(spec, hidden_size, vocab_size, dtype, device)``
    head           ``cls(spec, hidden_size, vocab_size, dtype, device, tied=False)``
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part needs from the checkpoint.

    ``role`` decides how the tensor is kept on the device: ``matrix`` in the compute dtype;
    ``bias`` and ``gain`` in float32 (exact for values stored in bfloat16, and a tensor stored
    in 32-bit stays so); ``table`` (integers) as int32. ``init`` names the rule of the
    random-weights mode: ``normal`` N(0, std), ``bias_normal`` N(0, std), ``one_plus_normal``
    1 + N(0, std / 2), ``zeros``.
    """

    name: str
    shape: tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"

    def device_dtype(self, compute_dtype: torch.dtype) -> torch.dtype:
        if self.role == "matrix":
            return compute_dtype
        if self.role in ("bias", "gain"):
            return torch.float32
        if self.role == "table":
            return torch.int32
        raise ValueError(f"unknown parameter role {self.role!r}")


@dataclass(frozen=True)
class PagedKVNeed:
    """A mixer that keeps keys and values of every position, or of a window of them."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps a state of fixed size per request (one slot per live request)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Base of every part: declared tensors in, bound tensors kept.

    ``graph_safe`` says that ``forward`` only queues work on the device from tensors whose
    addresses and shapes stay the same from step to step: it never reads a value back, never
    loops on the host over what a request brings, and takes its scratch from ``ctx.buffer``. Decode steps of a
    model are replayed from CUDA graphs only if every one of its parts says so; the default
    is the careful one, so a part written without a thought for graphs is never captured.
    """

    graph_safe = False

    def param_specs(self) -> list[ParamSpec]:
        return []

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        """Receive the tensors named by :meth:`param_specs` (device, final dtype)."""

    def scratch_per_token(self) -> int | None:
        """Elements of scratch, in the activation dtype, that ``forward`` holds per token of a step.

        The engine leaves that much room beside the cache when it sizes the page pool. ``None``
        (the default) means "not declared": the model then assumes
        :data:`UNDECLARED_SCRATCH_WIDTHS` times its hidden size for the part.
        """
        return None


UNDECLARED_SCRATCH_WIDTHS = 4
"""Hidden sizes of scratch per token assumed for a part that does not declare its own."""


class Mixer(Part):
    """Mixes information between positions of a sequence.

    ``forward(x, ctx, cache)`` takes the normed activations ``[tokens, hidden]`` of the step's
    packed tokens and returns the update to the residual stream, same shape and dtype.
    ``ctx`` is the step's :class:`~turboserve_b200.engine.batch.StepContext`; ``cache`` is the
    run's :class:`~turboserve_b200.cache.storage.RunCache` (pages and block table, or the state
    tensor and the requests' slots), ``None`` when the mixer keeps nothing.
    """

    def cache_need(self) -> PagedKVNeed | StateNeed | None:
        return None

    def forward(self, x: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    """A per-token function: ``forward(x, ctx)`` -> update to the residual stream."""

    def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    """Normalisation fused with the residual sum.

    ``forward(residual, delta, out, ctx)`` adds ``delta`` (may be ``None``) to the fp32
    residual in place and writes the normed rows to ``out``. ``forward_rows(residual, delta,
    rows, out, ctx)`` does the same for the rows listed in ``rows`` without updating the
    residual (the final norm, on the rows whose logits are wanted).
    """

    def forward(self, residual: torch.Tensor, delta: torch.Tensor | None, out: torch.Tensor, ctx: Any) -> torch.Tensor:
        raise NotImplementedError

    def forward_rows(self, residual: torch.Tensor, delta: torch.Tensor | None, rows: torch.Tensor,
                     num_rows: int, out: torch.Tensor, ctx: Any) -> torch.Tensor:
        raise NotImplementedError


class TokenEmbedding(Part):
    """Turns the step's token ids into the residual stream.

    ``forward(residual, ctx)`` fills the float32 ``residual`` ``[tokens, hidden]`` for the packed
    tokens of ``ctx.batch`` (``token_ids``, and ``positions`` or anything else of the batch it
    needs). ``table`` is the ``[vocab, hidden]`` matrix that a tied head multiplies by, if the
    embedding has one to share.
    """

    table: torch.Tensor | None = None

    def forward(self, residual: torch.Tensor, ctx: Any) -> None:
        raise NotImplementedError


class LogitHead(Part):
    """Turns the final normed rows into float32 logits.

    ``forward(rows_in, logits, num_rows, ctx)`` writes ``logits[:num_rows]`` (float32
    ``[rows, vocab]``) from ``rows_in`` (``[rows, hidden]``, activation dtype). A head built with
    ``tied=True`` declares no matrix of its own and receives the embedding's through :meth:`tie`.
    """

    def tie(self, table: torch.Tensor) -> None:
        raise NotImplementedError

    def forward(self, rows_in: torch.Tensor, logits: torch.Tensor, num_rows: int, ctx: Any) -> None:
        raise NotImplementedError


class PositionEncoding:
    """Whatever turns positions into a change of queries and keys; a mixer calls :meth:`apply`.

    ``apply`` is the whole step between a mixer's fused q/k/v product and its attention: add
    the bias, change queries and keys by their positions, and append keys and values to the
    request's pages. The mixer names no constant of the encoding; it hands over the product
    and says how it is laid out.

    The default implementation is the fused kernel of ``layer_ops.cu``: bias, then a rotation of
    the pairs ``(i, i + rotary_dim / 2)`` of every head by ``(position / factor) * inv_freq[i]``,
    then the append. An encoding that is such a rotation only sets ``inv_freq`` (float32,
    ``rotary_dim / 2`` values on the device), ``rotary_dim`` and ``factor``; with ``rotary_dim``
    0 (the class's own values) nothing is rotated. Any other encoding overrides :meth:`apply`,
    changes ``qkv`` as it likes and calls ``super().apply`` (or :meth:`append`) for the bias and
    the append.
    """

    graph_safe = True
    inv_freq: torch.Tensor | None = None
    rotary_dim = 0
    factor = 1.0

    def fused_rotation(self) -> tuple[torch.Tensor | None, int, float] | None:
        """``(inv_freq, rotary_dim, factor)`` when :meth:`apply` is the default one, else ``None``.

        A mixer may hand these constants to a kernel that does the whole of :meth:`apply` itself
        (decode attention does); an encoding that overrides :meth:`apply` is always called.
        """
        if type(self).apply is not PositionEncoding.apply:
            return None
        return self.inv_freq, self.rotary_dim, self.factor

    def check(self, head_dim: int) -> None:
        """Refuse a head size the encoding cannot act on (called once, when the mixer is built)."""
        if self.rotary_dim > head_dim:
            raise ValueError(f"rotary_dim ({self.rotary_dim}) exceeds head_dim ({head_dim})")

    def apply(self, qkv: torch.Tensor, bias: torch.Tensor | None, num_heads: int, num_kv_heads: int, head_dim: int,
              ctx: Any, cache: Any, write: bool) -> None:
        """Encode in place and append to the cache.

        ``qkv`` is ``[tokens, (num_heads + 2 * num_kv_heads) * head_dim]``: the query heads, then
        the key heads, then the value heads of every token of the step (``num_kv_heads`` is 0
        when the mixer reads another run's cache); ``bias`` (float32, same width) or ``None``;
        ``ctx.batch`` gives ``positions`` and ``seq_of_token``; ``cache`` the run's pages and
        its group, whose block table is ``ctx.batch.block_tables[cache.group]``; ``write`` says
        whether keys and values are to be appended.
        """
        from ..ops import kernels

        batch = ctx.batch
        kernels.rope_cache_write(
            qkv, bias, batch.positions, batch.seq_of_token, batch.block_tables[cache.group], cache.k_pages,
            cache.v_pages, batch.num_tokens, num_heads, num_kv_heads, head_dim, self.inv_freq, self.rotary_dim,
            self.factor, write, ctx.status,
        )

    def append(self, qkv: torch.Tensor, bias: torch.Tensor | None, num_heads: int, num_kv_heads: int, head_dim: int,
               ctx: Any, cache: Any, write: bool) -> None:
        """Bias and append alone, whatever the encoding's constants are."""
        from ..ops import kernels

        batch = ctx.batch
        kernels.rope_cache_write(
            qkv, bias, batch.positions, batch.seq_of_token, batch.block_tables[cache.group], cache.k_pages,
            cache.v_pages, batch.num_tokens, num_heads, num_kv_heads, head_dim, None, 0, 1.0, write, ctx.status,
        )


class Registry:
    def __init__(self, what: str) -> None:
        self.what = what
        self._kinds: dict[str, Callable[..., Any]] = {}

    def register(self, kind: str, factory: Callable[..., Any]) -> None:
        self._kinds[kind] = factory

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def get(self, kind: str) -> Callable[..., Any]:
        try:
            return self._kinds[kind]
        except KeyError:
            raise KeyError(f"no {self.what} of kind {kind!r} is registered; known: {sorted(self._kinds)}") from None

    def kinds(self) -> list[str]:
        return sorted(self._kinds)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("token embedding")
HEADS = Registry("logit head")


def register_mixer(kind: str, factory: Callable[..., Any]) -> None:
    MIXERS.register(kind, factory)


def register_feed_forward(kind: str, factory: Callable[..., Any]) -> None:
    FEED_FORWARDS.register(kind, factory)


def register_norm(kind: str, factory: Callable[..., Any]) -> None:
    NORMS.register(kind, factory)


def register_embedding(kind: str, factory: Callable[..., Any]) -> None:
    EMBEDDINGS.register(kind, factory)


def register_head(kind: str, factory: Callable[..., Any]) -> None:
    HEADS.register(kind, factory)


def register_position(kind: str, factory: Callable[..., Any]) -> None:
    POSITIONS.register(kind, factory)


def register_block(kind: str, factory: Callable[..., Any]) -> None:
    BLOCKS.register(kind, factory)
