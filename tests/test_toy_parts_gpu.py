"""Toy parts defined here and nowhere else: a feed-forward with routing and another position
encoding, in different layers of one model; a position encoding that is no rotation; an
embedding and a head of their own around the layers.

They are registered by kind, named in a ``LayerSpec``, built by the random-weights mode and the
loader from their ``param_specs``, and stepped through replay whole, cut and mixed, without a
change to any file of the framework. Neither is anybody's model: the feed-forward sends each
token to the one of a few small matrices its router picks, the position encoding rotates pairs
by frequencies that are listed one by one instead of following a geometric law.
"""

import pytest
import torch

import plain_qwen2 as P
import traces

pytestmark = pytest.mark.gpu

FREQS = (0.9, 0.31, 0.07, 0.011)  # four pairs: the first 8 of 16 head dims are rotated


def register_toys():
    from dataclasses import dataclass

    from turboserve_b200.config import LayerSpec, ModelSpec, PartSpec, register_architecture
    from turboserve_b200.models import DecoderModel
    from turboserve_b200.parts import FeedForward, ParamSpec, PositionEncoding, register_feed_forward, register_position

    class RoutedFeedForward(FeedForward):
        """out = relu(W_e x) V_e with e = argmax of the fp32 router logits R x (one expert per token)."""

        def __init__(self, spec, hidden_size, dtype, device):
            self.hidden, self.experts, self.width = hidden_size, int(spec["experts"]), int(spec["width"])

        def param_specs(self):
            return [ParamSpec("router.weight", (self.experts, self.hidden)),
                    ParamSpec("experts.up", (self.experts, self.width, self.hidden)),
                    ParamSpec("experts.down", (self.experts, self.hidden, self.width))]

        def bind(self, tensors):
            self.router, self.up, self.down = tensors["router.weight"], tensors["experts.up"], tensors["experts.down"]

        def forward(self, x, ctx):
            n = ctx.batch.num_tokens
            out = ctx.buffer("toy.routed_out", (x.shape[0], self.hidden))
            choice = (x[:n].float() @ self.router.float().T).argmax(-1)
            hidden = torch.relu(torch.einsum("ewh,th->tew", self.up.float(), x[:n].float()))
            picked = hidden[torch.arange(n, device=x.device), choice]
            out[:n] = torch.einsum("thw,tw->th", self.down.float()[choice], picked).to(out.dtype)
            return out

    class ListedFrequencies(PositionEncoding):
        """Rotation of pair (i, i + rotary_dim / 2) by position * freqs[i], the frequencies given one by one."""

        def __init__(self, spec, device):
            freqs = [float(f) for f in spec["freqs"]]
            self.rotary_dim = 2 * len(freqs)
            self.factor = 1.0
            self.inv_freq = torch.tensor(freqs, dtype=torch.float32, device=device)

    register_feed_forward("toy_routed", RoutedFeedForward)
    register_position("toy_listed", ListedFrequencies)

    @dataclass(frozen=True)
    class ToyConfig:
        hidden_size: int
        vocab_size: int
        experts: int
        width: int
        architecture: str = "ToyPartsForCausalLM"

        @classmethod
        def from_dict(cls, data):
            return cls(data["hidden_size"], data["vocab_size"], data["experts"], data["width"])

        def to_dict(self):
            return dict(architectures=[self.architecture], hidden_size=self.hidden_size, vocab_size=self.vocab_size,
                        experts=self.experts, width=self.width)

        def to_model_spec(self):
            norm = PartSpec("rms_norm", {"eps": 1e-5})
            attn = PartSpec("attention", dict(num_heads=3, num_kv_heads=1, head_dim=16, qkv_bias=False, window=None))
            routed = PartSpec("toy_routed", {"experts": self.experts, "width": self.width})
            dense = PartSpec("gated_mlp", {"intermediate_size": 48})
            listed = PartSpec("toy_listed", {"freqs": list(FREQS)})
            rotary = PartSpec("rotary", dict(rotary_dim=16, theta=1e4))
            layers = (LayerSpec(attn, routed, norm, norm, listed), LayerSpec(attn, dense, norm, norm, rotary),
                      LayerSpec(attn, routed, norm, norm, None))
            return ModelSpec(self.architecture, self.hidden_size, self.vocab_size, layers, ModelSpec.sequential(3), norm)

    register_architecture("ToyPartsForCausalLM", ToyConfig,
                          lambda config, dtype, device: DecoderModel(config.to_model_spec(), dtype, device))
    return ToyConfig


def plain_attention(x, w, p, pos, inv_freq, added=None):
    """Causal attention, 3 query heads on one kv head of 16 dims, pairs (i, i + len/2... ) rotated by pos * inv_freq[i];
    ``added`` ([tokens, 16]) is added to every query and key head instead."""
    nh, d = 3, 16
    q = (x @ w[p + "q_proj.weight"].T).view(-1, nh, d)
    k = (x @ w[p + "k_proj.weight"].T).view(-1, 1, d)
    v = (x @ w[p + "v_proj.weight"].T).view(-1, 1, d)
    if added is not None:
        q, k = q + added[:, None, :], k + added[:, None, :]
    if inv_freq is not None:
        half = len(inv_freq)
        angle = pos.double()[:, None] * inv_freq.double()[None, :]
        cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]

        def rotate(t):
            a, b = t[..., :half], t[..., half:2 * half]
            return torch.cat([a * cos - b * sin, b * cos + a * sin, t[..., 2 * half:]], dim=-1)

        q, k = rotate(q), rotate(k)
    scores = torch.einsum("thd,sd->hts", q, k[:, 0]) / d ** 0.5
    mask = pos[None, :, None] >= pos[None, None, :]
    probs = torch.softmax(scores.masked_fill(~mask, float("-inf")), dim=-1)
    out = torch.einsum("hts,sd->thd", probs, v[:, 0]).reshape(-1, nh * d)
    return out @ w[p + "o_proj.weight"].T


def plain_toy(config, w, ids):
    w = {k: v.double() for k, v in w.items()}
    h = w["model.embed_tokens.weight"][torch.tensor(ids)]
    pos = torch.arange(len(ids))
    rotary = 1.0 / (1e4 ** (torch.arange(0, 16, 2, dtype=torch.float32) / 16))
    for layer, inv_freq in enumerate([torch.tensor(FREQS, dtype=torch.float32), rotary, None]):
        p = f"model.layers.{layer}."
        x = P.rms_norm(h, w[p + "input_layernorm.weight"], 1e-5)
        h = h + plain_attention(x, w, p + "self_attn.", pos, inv_freq)
        x = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], 1e-5)
        if layer == 1:
            h = h + P.mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"], "silu")
            continue
        choice = (x @ w[p + "mlp.router.weight"].T).argmax(-1)
        rows = []
        for t in range(len(ids)):
            e = int(choice[t])
            rows.append(w[p + "mlp.experts.down"][e] @ torch.relu(w[p + "mlp.experts.up"][e] @ x[t]))
        h = h + torch.stack(rows)
    return P.rms_norm(h, w["model.norm.weight"], 1e-5) @ w["lm_head.weight"].T, None


def test_toy_feed_forward_with_routing_and_another_position_encoding(tmp_path):
    from safetensors.torch import load_file

    from turboserve_b200.config import config_from_dir, unregister_architecture
    from turboserve_b200.parts import FEED_FORWARDS, POSITIONS
    from turboserve_b200.replay import Replayer
    from turboserve_b200.weights import write_random_model

    ToyConfig = register_toys()
    try:
        config = ToyConfig(hidden_size=40, vocab_size=70, experts=3, width=24)
        folder = write_random_model(config, 5, tmp_path / "toy", torch.float32)
        assert config_from_dir(folder) == config
        weights = load_file(str(folder / "model.safetensors"))
        assert weights["model.layers.0.mlp.experts.up"].shape == (3, 24, 40) and "model.layers.1.mlp.gate_proj.weight" in weights
        requests = traces.make_requests(70, [33, 8, 47, 21], seed=4)
        ref = {rid: plain_toy(config, weights, ids)[0] for rid, ids in requests.items()}
        routed_to = set()
        for rid, ids in requests.items():  # the router does send tokens to different experts
            x = P.rms_norm(weights["model.embed_tokens.weight"].double()[torch.tensor(ids)], weights["model.layers.0.input_layernorm.weight"].double(), 1e-5)
            routed_to |= set((x @ weights["model.layers.0.mlp.router.weight"].double().T).argmax(-1).tolist())
        assert len(routed_to) > 1
        for builder, kwargs in ((traces.whole, {}), (traces.changing_portions, {"sizes": (5, 2, 11, 1)}), (traces.mixed, {"seed": 3, "max_live": 3})):
            steps, max_tokens = builder(requests, **kwargs)
            replayer = Replayer(folder, "float32", max_tokens)
            got = traces.collect(requests, steps, traces.replay(replayer, steps))
            for rid in requests:
                assert torch.allclose(got[rid].double(), ref[rid], atol=3e-5), (builder.__name__, rid, (got[rid].double() - ref[rid]).abs().max())
    finally:
        unregister_architecture("ToyPartsForCausalLM")
        FEED_FORWARDS.unregister("toy_routed")
        POSITIONS.unregister("toy_listed")


WAVE_RATES = tuple(0.37 * 0.61 ** j for j in range(16))
WAVE_AMPLITUDE = 0.25


def waves(positions):
    """[tokens, 16] float64: what the toy encoding below adds to every query and key head."""
    return WAVE_AMPLITUDE * torch.sin(positions.double()[:, None] * torch.tensor(WAVE_RATES, dtype=torch.float64, device=positions.device)[None, :])


def test_toy_position_encoding_that_is_not_a_rotation(tmp_path):
    """A position encoding that adds a wave of the position to queries and keys: no pair is
    rotated, no frequency table is handed to a kernel. It overrides ``PositionEncoding.apply`` and
    is registered here; the attention part and its kernels are used as they are."""
    from dataclasses import dataclass

    from safetensors.torch import load_file

    from turboserve_b200.config import LayerSpec, ModelSpec, PartSpec, register_architecture, unregister_architecture
    from turboserve_b200.models import DecoderModel
    from turboserve_b200.parts import POSITIONS, PositionEncoding, register_position
    from turboserve_b200.replay import Replayer
    from turboserve_b200.weights import write_random_model

    calls = []

    class AddedWaves(PositionEncoding):
        def __init__(self, spec, device):
            self.heads_seen = None

        def apply(self, qkv, bias, num_heads, num_kv_heads, head_dim, ctx, cache, write):
            n = ctx.batch.num_tokens
            wave = waves(ctx.batch.positions[:n]).to(qkv.dtype)
            rotated_heads = num_heads + num_kv_heads  # queries and keys, not values
            qkv[:n, : rotated_heads * head_dim].view(n, rotated_heads, head_dim).add_(wave[:, None, :])
            calls.append((num_heads, num_kv_heads, head_dim, bool(write)))
            self.append(qkv, bias, num_heads, num_kv_heads, head_dim, ctx, cache, write)

    register_position("toy_waves", AddedWaves)

    @dataclass(frozen=True)
    class WaveConfig:
        hidden_size: int
        vocab_size: int
        architecture: str = "ToyWavesForCausalLM"

        @classmethod
        def from_dict(cls, data):
            return cls(data["hidden_size"], data["vocab_size"])

        def to_dict(self):
            return dict(architectures=[self.architecture], hidden_size=self.hidden_size, vocab_size=self.vocab_size)

        def to_model_spec(self):
            norm = PartSpec("rms_norm", {"eps": 1e-5})
            attn = PartSpec("attention", dict(num_heads=3, num_kv_heads=1, head_dim=16, qkv_bias=False, window=None))
            dense = PartSpec("gated_mlp", {"intermediate_size": 48})
            layers = (LayerSpec(attn, dense, norm, norm, PartSpec("toy_waves", {})),
                      LayerSpec(attn, dense, norm, norm, PartSpec("rotary", dict(rotary_dim=16, theta=1e4))))
            return ModelSpec(self.architecture, self.hidden_size, self.vocab_size, layers, ModelSpec.sequential(2), norm)

    register_architecture("ToyWavesForCausalLM", WaveConfig,
                          lambda config, dtype, device: DecoderModel(config.to_model_spec(), dtype, device))

    def plain(weights, ids, with_wave=True):
        w = {k: v.double() for k, v in weights.items()}
        h = w["model.embed_tokens.weight"][torch.tensor(ids)]
        pos = torch.arange(len(ids))
        rotary = 1.0 / (1e4 ** (torch.arange(0, 16, 2, dtype=torch.float32) / 16))
        for layer in range(2):
            p = f"model.layers.{layer}."
            x = P.rms_norm(h, w[p + "input_layernorm.weight"], 1e-5)
            if layer == 0:
                h = h + plain_attention(x, w, p + "self_attn.", pos, None, added=waves(pos) if with_wave else None)
            else:
                h = h + plain_attention(x, w, p + "self_attn.", pos, rotary)
            x = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], 1e-5)
            h = h + P.mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"], "silu")
        return P.rms_norm(h, w["model.norm.weight"], 1e-5) @ w["lm_head.weight"].T

    try:
        config = WaveConfig(hidden_size=40, vocab_size=70)
        folder = write_random_model(config, 8, tmp_path / "waves", torch.float32)
        weights = load_file(str(folder / "model.safetensors"))
        requests = traces.make_requests(70, [33, 8, 47, 21], seed=14)
        ref = {rid: plain(weights, ids) for rid, ids in requests.items()}
        # the wave matters: without it the logits are somewhere else
        assert all((ref[rid] - plain(weights, ids, with_wave=False)).abs().max() > 1e-3 for rid, ids in requests.items())
        for builder, kwargs in ((traces.whole, {}), (traces.changing_portions, {"sizes": (5, 2, 11, 1)}), (traces.mixed, {"seed": 3, "max_live": 3})):
            steps, max_tokens = builder(requests, **kwargs)
            replayer = Replayer(folder, "float32", max_tokens)
            assert replayer.model.graph_safe  # nothing in it steps on the host
            got = traces.collect(requests, steps, traces.replay(replayer, steps))
            for rid in requests:
                assert torch.allclose(got[rid].double(), ref[rid], atol=3e-5), (builder.__name__, rid, (got[rid].double() - ref[rid]).abs().max())
        assert calls and set(calls) == {(3, 1, 16, True)}
    finally:
        unregister_architecture("ToyWavesForCausalLM")
        POSITIONS.unregister("toy_waves")


PLACE_PERIOD = 7
EMBED_SCALE = 1.5
HEAD_SCALE = 0.5


def test_toy_embedding_and_head_around_the_layers(tmp_path):
    """An embedding that scales the token's row and adds a row chosen by the position, and a head
    tied to the embedding's table that scales its logits and adds a bias of its own: both are
    registered here, declare their tensors (``model.embed_tokens.place.weight``, ``lm_head.bias``),
    and the model, the loader, the random-weights mode and replay use them as they are."""
    from dataclasses import dataclass

    from safetensors.torch import load_file

    from turboserve_b200.config import LayerSpec, ModelSpec, PartSpec, register_architecture, unregister_architecture
    from turboserve_b200.models import DecoderModel
    from turboserve_b200.ops import kernels
    from turboserve_b200.parts import EMBEDDINGS, HEADS, LogitHead, ParamSpec, TokenEmbedding, register_embedding, register_head
    from turboserve_b200.replay import Replayer
    from turboserve_b200.weights import load_weights, write_random_model

    class PlacedEmbedding(TokenEmbedding):
        def __init__(self, spec, hidden_size, vocab_size, dtype, device):
            self.hidden, self.vocab, self.period, self.scale = hidden_size, vocab_size, int(spec["period"]), float(spec["scale"])

        def param_specs(self):
            return [ParamSpec("weight", (self.vocab, self.hidden)), ParamSpec("place.weight", (self.period, self.hidden))]

        def bind(self, tensors):
            self.table, self.place = tensors["weight"].contiguous(), tensors["place.weight"]

        def forward(self, residual, ctx):
            n = ctx.batch.num_tokens
            kernels.embedding(ctx.batch.token_ids, self.table, residual, ctx.status)
            residual[:n].mul_(self.scale).add_(self.place.float()[ctx.batch.positions[:n].long() % self.period])

    class BiasedHead(LogitHead):
        def __init__(self, spec, hidden_size, vocab_size, dtype, device, tied=False):
            self.hidden, self.vocab, self.tied, self.scale = hidden_size, vocab_size, tied, float(spec["scale"])
            self.weight = None

        def param_specs(self):
            own = [] if self.tied else [ParamSpec("weight", (self.vocab, self.hidden))]
            return own + [ParamSpec("bias", (self.vocab,), role="bias", init="bias_normal")]

        def bind(self, tensors):
            self.bias = tensors["bias"]
            if not self.tied:
                self.weight = tensors["weight"]

        def tie(self, table):
            self.weight = table

        def forward(self, rows_in, logits, num_rows, ctx):
            logits[:num_rows] = (rows_in[:num_rows].float() @ self.weight.float().T) * self.scale + self.bias

    register_embedding("toy_placed", PlacedEmbedding)
    register_head("toy_biased", BiasedHead)

    @dataclass(frozen=True)
    class AroundConfig:
        hidden_size: int
        vocab_size: int
        tie_word_embeddings: bool
        architecture: str = "ToyAroundForCausalLM"

        @classmethod
        def from_dict(cls, data):
            return cls(data["hidden_size"], data["vocab_size"], data["tie_word_embeddings"])

        def to_dict(self):
            return dict(architectures=[self.architecture], hidden_size=self.hidden_size, vocab_size=self.vocab_size,
                        tie_word_embeddings=self.tie_word_embeddings)

        def to_model_spec(self):
            norm = PartSpec("rms_norm", {"eps": 1e-5})
            attn = PartSpec("attention", dict(num_heads=3, num_kv_heads=1, head_dim=16, qkv_bias=False, window=None))
            dense = PartSpec("gated_mlp", {"intermediate_size": 48})
            layers = (LayerSpec(attn, dense, norm, norm, PartSpec("rotary", dict(rotary_dim=16, theta=1e4))),)
            return ModelSpec(self.architecture, self.hidden_size, self.vocab_size, layers, ModelSpec.sequential(1), norm,
                             embedding=PartSpec("toy_placed", {"period": PLACE_PERIOD, "scale": EMBED_SCALE}),
                             head=PartSpec("toy_biased", {"scale": HEAD_SCALE}), tie_word_embeddings=self.tie_word_embeddings)

    register_architecture("ToyAroundForCausalLM", AroundConfig,
                          lambda config, dtype, device: DecoderModel(config.to_model_spec(), dtype, device))

    def plain(weights, ids, tied):
        w = {k: v.double() for k, v in weights.items()}
        pos = torch.arange(len(ids))
        h = w["model.embed_tokens.weight"][torch.tensor(ids)] * EMBED_SCALE + w["model.embed_tokens.place.weight"][pos % PLACE_PERIOD]
        rotary = 1.0 / (1e4 ** (torch.arange(0, 16, 2, dtype=torch.float32) / 16))
        p = "model.layers.0."
        x = P.rms_norm(h, w[p + "input_layernorm.weight"], 1e-5)
        h = h + plain_attention(x, w, p + "self_attn.", pos, rotary)
        x = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], 1e-5)
        h = h + P.mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"], "silu")
        matrix = w["model.embed_tokens.weight"] if tied else w["lm_head.weight"]
        return (P.rms_norm(h, w["model.norm.weight"], 1e-5) @ matrix.T) * HEAD_SCALE + w["lm_head.bias"]

    try:
        for tied in (True, False):
            config = AroundConfig(hidden_size=40, vocab_size=70, tie_word_embeddings=tied)
            folder = write_random_model(config, 21, tmp_path / f"around{int(tied)}", torch.float32)
            weights = load_file(str(folder / "model.safetensors"))
            assert weights["model.embed_tokens.place.weight"].shape == (PLACE_PERIOD, 40) and weights["lm_head.bias"].shape == (70,)
            assert ("lm_head.weight" in weights) == (not tied)
            assert weights["lm_head.bias"].abs().max() > 0
            requests = traces.make_requests(70, [33, 8, 47, 21], seed=24)
            ref = {rid: plain(weights, ids, tied) for rid, ids in requests.items()}
            for builder, kwargs in ((traces.whole, {}), (traces.changing_portions, {"sizes": (5, 2, 11, 1)}), (traces.mixed, {"seed": 3, "max_live": 3})):
                steps, max_tokens = builder(requests, **kwargs)
                replayer = Replayer(folder, "float32", max_tokens)
                assert (replayer.model.head.weight is replayer.model.embedding.table) == tied
                assert not replayer.model.graph_safe  # the toy parts did not say they were
                got = traces.collect(requests, steps, traces.replay(replayer, steps))
                for rid in requests:
                    assert torch.allclose(got[rid].double(), ref[rid], atol=3e-5), (tied, builder.__name__, rid, (got[rid].double() - ref[rid]).abs().max())
        # a tied checkpoint may still hold the head's copy of the table (not loaded), but never lacks the head's own bias
        model = DecoderModel(AroundConfig(40, 70, True).to_model_spec(), torch.float32, "cuda")
        assert model.optional_names() == {"lm_head.weight"}
        assert [p.name for p in model.named_params()][-1] == "lm_head.bias"
    finally:
        unregister_architecture("ToyAroundForCausalLM")
        EMBEDDINGS.unregister("toy_placed")
        HEADS.unregister("toy_biased")
