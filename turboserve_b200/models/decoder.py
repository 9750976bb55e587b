"""The decoder every architecture is built as: embedding, a run order of layers, norm, head.

The model is assembled from a :class:`~turboserve_b200.config.ModelSpec` through the part
registries (the embedding and the head are parts too) and knows nothing about any particular
architecture. It replaces the reference's
``Decoder`` / ``CausalLM`` pair (``src/turboserve/engine/model/model.py:51-108,111-315``):
``forward`` runs the step's packed tokens through the layers against the cache and returns
fp32 logits only at the rows that were asked for (``compute_logits``, ``:220-244``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..cache.storage import CachePlan, CacheStorage, plan_cache
from ..config.model_spec import ModelSpec
from ..parts.base import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, UNDECLARED_SCRATCH_WIDTHS, ParamSpec, Part


@dataclass(frozen=True)
class NamedParam:
    """A tensor of the checkpoint: its full name, what it is, and the part that receives it."""

    name: str
    spec: ParamSpec
    owner: int  # index into DecoderModel.parts_list
    local: str


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device | str) -> None:
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.hidden_size, self.vocab_size = spec.hidden_size, spec.vocab_size
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding, spec.hidden_size, spec.vocab_size, dtype, self.device)
        self.parts_list: list[Part] = [self.embedding]
        self._part_prefix: list[str] = [spec.names.embedding]
        self.blocks = []
        reads_only = [True] * len(spec.layers)
        for run in spec.order:
            if run.cache_from is None:
                reads_only[run.layer] = False
        for index, layer in enumerate(spec.layers):
            prefix = spec.names.layer.format(index=index)
            mixer = MIXERS.get(layer.mixer.kind)(layer.mixer, spec.hidden_size, dtype, self.device,
                                                 position=layer.position, shares_cache=reads_only[index])
            feed_forward = FEED_FORWARDS.get(layer.feed_forward.kind)(layer.feed_forward, spec.hidden_size, dtype, self.device)
            mixer_norm = NORMS.get(layer.mixer_norm.kind)(layer.mixer_norm, spec.hidden_size, dtype, self.device)
            ff_norm = NORMS.get(layer.feed_forward_norm.kind)(layer.feed_forward_norm, spec.hidden_size, dtype, self.device)
            for part, part_prefix in ((mixer_norm, spec.names.mixer_norm), (mixer, spec.names.mixer),
                                      (ff_norm, spec.names.feed_forward_norm), (feed_forward, spec.names.feed_forward)):
                self.parts_list.append(part)
                self._part_prefix.append(prefix + part_prefix)
            self.blocks.append(BLOCKS.get(layer.block)(mixer, feed_forward, mixer_norm, ff_norm))
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, spec.hidden_size, dtype, self.device)
        self.parts_list.append(self.final_norm)
        self._part_prefix.append(spec.names.final_norm)
        self.head = HEADS.get(spec.head.kind)(spec.head, spec.hidden_size, spec.vocab_size, dtype, self.device,
                                              tied=spec.tie_word_embeddings)
        self.parts_list.append(self.head)
        self._part_prefix.append(spec.names.head)
        self.loaded = False

    # -- tensors ----------------------------------------------------------------------------

    def named_params(self) -> list[NamedParam]:
        """Every tensor the checkpoint must hold, in a fixed order (the random-weights order):
        the embedding's, the layers' in order, the final norm's, the head's."""
        out = []
        for index, (part, prefix) in enumerate(zip(self.parts_list, self._part_prefix)):
            for p in part.param_specs():
                out.append(NamedParam(prefix + p.name, p, index, p.name))
        names = [p.name for p in out]
        if len(set(names)) != len(names):
            raise ValueError("two parts declare a tensor of the same name")
        return out

    def optional_names(self) -> set[str]:
        """Names a checkpoint may hold that are not loaded (the tied head's copy of the embedding)."""
        if not self.spec.tie_word_embeddings:
            return set()
        untied = HEADS.get(self.spec.head.kind)(self.spec.head, self.hidden_size, self.vocab_size, self.dtype, self.device, tied=False)
        own = {p.name for p in self.head.param_specs()}
        return {self.spec.names.head + p.name for p in untied.param_specs() if p.name not in own}

    def bind_stream(self, fetch) -> None:
        """Hand every part its tensors, one part at a time.

        ``fetch(param)`` returns the tensor of a :class:`NamedParam` on the device in its final
        dtype; it is called once per tensor, in the order of :meth:`named_params`. A part's
        tensors are bound (and fused, where the part fuses them) and let go before the next
        part's are fetched, so that loading needs room for the model plus one part.
        """
        current: dict[str, torch.Tensor] = {}
        owner = -1

        def flush() -> None:
            if owner >= 0:
                self.parts_list[owner].bind(current)

        for p in self.named_params():
            t = fetch(p)
            if tuple(t.shape) != tuple(p.spec.shape):
                raise ValueError(f"{p.name}: shape {tuple(t.shape)} where {p.spec.shape} is declared")
            if p.owner != owner:
                flush()
                current, owner = {}, p.owner
            current[p.local] = t
        flush()
        for part in self.parts_list:
            if not part.param_specs():
                part.bind({})
        if self.spec.tie_word_embeddings:
            if self.embedding.table is None:
                raise ValueError(f"the head is tied, but the embedding of kind {self.spec.embedding.kind!r} has no table to share")
            self.head.tie(self.embedding.table)
        self.loaded = True

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        """Hand every part its tensors from a dict by full name (device, final dtypes)."""
        self.bind_stream(lambda p: tensors[p.name])

    def init_random(self, seed: int) -> None:
        """Fill the model with random weights made on the device (large shapes, benchmarks)."""
        from ..weights.random_init import draw

        generator = torch.Generator(device=self.device).manual_seed(seed)
        self.bind_stream(lambda p: draw(p.spec, self.spec.init_std, generator, self.device).to(p.spec.device_dtype(self.dtype)))

    def num_parameters(self) -> int:
        total = 0
        for p in self.named_params():
            count = 1
            for s in p.spec.shape:
                count *= s
            total += count
        return total

    # -- what the parts declare -----------------------------------------------------------------

    def scratch_bytes_per_token(self, itemsize: int) -> int:
        """Scratch a step holds per token: the fp32 residual, the normed rows, the most that any
        layer's mixer and feed-forward declare (buffers are shared between layers by name), and
        what the embedding and the head declare."""
        def declared(part: Part) -> int:
            own = part.scratch_per_token()
            return UNDECLARED_SCRATCH_WIDTHS * self.hidden_size if own is None else int(own)

        mixers = max(declared(block.mixer) for block in self.blocks)
        feed_forwards = max(declared(block.feed_forward) for block in self.blocks)
        around = declared(self.embedding) + declared(self.head)
        return 4 * self.hidden_size + itemsize * (self.hidden_size + mixers + feed_forwards + around)

    @property
    def graph_safe(self) -> bool:
        """Whether every part allows its step to be captured in a CUDA graph (``Part.graph_safe``)."""
        return all(part.graph_safe for part in self.parts_list)

    # -- cache ------------------------------------------------------------------------------

    def cache_plan(self) -> CachePlan:
        needs = [self.blocks[run.layer].mixer.cache_need() for run in self.spec.order]
        return plan_cache(needs, [run.cache_from for run in self.spec.order])

    # -- the step ---------------------------------------------------------------------------

    def forward(self, ctx, storage: CacheStorage) -> torch.Tensor | None:
        """Run the step's tokens; returns fp32 logits ``[num_logit_rows, vocab]`` or ``None``."""
        if not self.loaded:
            raise RuntimeError("the model has no weights yet")
        batch = ctx.batch
        n = batch.num_tokens
        residual = ctx.buffer("model.residual", (n, self.hidden_size), torch.float32)
        self.embedding.forward(residual, ctx)
        pending = None
        for run_index, run in enumerate(self.spec.order):
            ctx.run_index = run_index
            pending = self.blocks[run.layer].forward(residual, pending, ctx, storage.run_caches[run_index])
        rows = batch.num_logit_rows
        if rows == 0:
            return None
        final = ctx.buffer("model.final", (rows, self.hidden_size))
        self.final_norm.forward_rows(residual, pending, batch.logit_rows, rows, final, ctx)
        logits = ctx.buffer("model.logits", (rows, self.vocab_size), torch.float32)
        self.head.forward(final, logits, rows, ctx)
        return logits
