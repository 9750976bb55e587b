"""A toy architecture with a mixer that keeps state of its own, defined here and nowhere else.

The test registers a mixer kind, a configuration class and an architecture name, writes a
model folder with the random-weights mode, and steps it through the replay program's loop,
whole and cut, without a change to any file of the framework.
"""

import json

import pytest
import torch

import plain_qwen2 as P
import traces

pytestmark = pytest.mark.gpu


def register_toy():
    from dataclasses import dataclass

    from turboserve_b200.config import LayerSpec, ModelSpec, PartSpec, register_architecture
    from turboserve_b200.models import DecoderModel
    from turboserve_b200.parts import Mixer, ParamSpec, StateNeed, register_mixer

    class DecayMixer(Mixer):
        """state <- decay * state + (1 - decay) * x_t ;  out_t = W state.  One state per request."""

        def __init__(self, spec, hidden_size, dtype, device, position=None, shares_cache=False):
            self.hidden, self.decay, self.dtype = hidden_size, float(spec["decay"]), dtype

        def param_specs(self):
            return [ParamSpec("mix.weight", (self.hidden, self.hidden))]

        def bind(self, tensors):
            self.weight = tensors["mix.weight"]

        def cache_need(self):
            return StateNeed((self.hidden,), torch.float32)

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            start = 0
            for n, slot in zip(ctx.batch.query_lens_host, ctx.batch.state_slots_host):
                state = cache.state[slot]
                for t in range(start, start + n):
                    state = self.decay * state + (1 - self.decay) * x[t].float()
                    out[t] = (self.weight.float() @ state).to(x.dtype)
                cache.state[slot] = state
                start += n
            return out

    register_mixer("toy_decay", DecayMixer)

    @dataclass(frozen=True)
    class ToyConfig:
        hidden_size: int
        vocab_size: int
        decay: float
        intermediate_size: int
        architecture: str = "ToyStateForCausalLM"

        @classmethod
        def from_dict(cls, data):
            return cls(data["hidden_size"], data["vocab_size"], data["decay"], data["intermediate_size"])

        def to_dict(self):
            return dict(architectures=[self.architecture], hidden_size=self.hidden_size, vocab_size=self.vocab_size,
                        decay=self.decay, intermediate_size=self.intermediate_size)

        def to_model_spec(self):
            norm = PartSpec("rms_norm", {"eps": 1e-6})
            ff = PartSpec("gated_mlp", {"intermediate_size": self.intermediate_size})
            toy = LayerSpec(PartSpec("toy_decay", {"decay": self.decay}), ff, norm, norm, None)
            attn = LayerSpec(PartSpec("attention", dict(num_heads=2, num_kv_heads=1, head_dim=16, qkv_bias=True, window=12)), ff,
                             norm, norm, PartSpec("rotary", dict(rotary_dim=16, theta=1e4)))
            return ModelSpec(self.architecture, self.hidden_size, self.vocab_size, (toy, attn, toy), ModelSpec.sequential(3), norm)

    register_architecture("ToyStateForCausalLM", ToyConfig, lambda config, dtype, device: DecoderModel(config.to_model_spec(), dtype, device))
    return ToyConfig


def plain_toy(config, w, ids):
    w = {k: v.double() for k, v in w.items()}
    t = len(ids)
    h = w["model.embed_tokens.weight"][torch.tensor(ids)]
    pos = torch.arange(t)
    dims = dict(nh=2, nkv=1, d=16, eps=1e-6, theta=1e4, factor=1.0, act="silu")
    for layer in range(3):
        p = f"model.layers.{layer}."
        if layer == 1:
            h = P.decoder_layer(h, w, p, dims, pos, 12)
            continue
        x = P.rms_norm(h, w[p + "input_layernorm.weight"], 1e-6)
        state = torch.zeros(config.hidden_size, dtype=torch.float64)
        mixed = []
        for i in range(t):
            state = config.decay * state + (1 - config.decay) * x[i]
            mixed.append(w[p + "self_attn.mix.weight"] @ state)
        h = h + torch.stack(mixed)
        x = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], 1e-6)
        h = h + P.mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"], "silu")
    return P.rms_norm(h, w["model.norm.weight"], 1e-6) @ w["lm_head.weight"].T


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from safetensors.torch import load_file

    from turboserve_b200.config import config_from_dir, unregister_architecture
    from turboserve_b200.parts import MIXERS
    from turboserve_b200.replay import Replayer
    from turboserve_b200.weights import write_random_model

    ToyConfig = register_toy()
    try:
        config = ToyConfig(hidden_size=40, vocab_size=90, decay=0.8, intermediate_size=56)
        folder = write_random_model(config, 3, tmp_path / "toy", torch.float32)
        assert config_from_dir(folder) == config
        weights = load_file(str(folder / "model.safetensors"))
        assert "model.layers.0.self_attn.mix.weight" in weights and "model.layers.1.self_attn.q_proj.bias" in weights
        requests = traces.make_requests(90, [30, 9, 45, 17, 26], seed=1)
        ref = {rid: plain_toy(config, weights, ids) for rid, ids in requests.items()}
        for builder, kwargs in ((traces.whole, {}), (traces.changing_portions, {"sizes": (4, 2, 9, 1)}), (traces.mixed, {"seed": 2, "max_live": 3})):
            steps, max_tokens = builder(requests, **kwargs)
            replayer = Replayer(folder, "float32", max_tokens)
            plan = replayer.runner.plan
            assert [r.kind for r in plan.runs] == ["state", "paged", "state"] and plan.windows == [12]
            got = traces.collect(requests, steps, traces.replay(replayer, steps))
            for rid in requests:
                assert torch.allclose(got[rid].double(), ref[rid], atol=2e-5), (builder.__name__, rid)
            assert replayer.manager.slots.num_free == replayer.manager.slots.num_slots
    finally:
        unregister_architecture("ToyStateForCausalLM")
        MIXERS.unregister("toy_decay")


def test_toy_mixer_with_state_through_the_engine_with_preemption_and_a_small_budget(tmp_path):
    """The same toy model through ``LLMEngine``: a token budget that cuts its prompts, a pool so
    small that requests are preempted and computed again, steps launched ahead. The state must
    be carried across portions, reset at admission and again after a preemption: every token is
    the plain recurrence's argmax."""
    from safetensors.torch import load_file

    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig
    from turboserve_b200.config import unregister_architecture
    from turboserve_b200.parts import MIXERS
    from turboserve_b200.weights import write_random_model

    ToyConfig = register_toy()
    try:
        config = ToyConfig(hidden_size=40, vocab_size=90, decay=0.8, intermediate_size=56)
        folder = write_random_model(config, 3, tmp_path / "toy", torch.float32)
        weights = load_file(str(folder / "model.safetensors"))
        prompts = list(traces.make_requests(90, [30, 9, 45, 17, 26, 38], seed=6).values())
        engine = LLMEngine(EngineConfig(model=str(folder), dtype="float32", overlap_decode=True, scheduler=SchedulerConfig(
            max_num_seqs=4, max_num_batched_tokens=12, block_size=4, num_blocks=16)))
        with engine:
            assert not engine.model.graph_safe  # the toy mixer steps on the host: never captured
            outputs = engine.generate(prompts, SamplingParams(max_tokens=30, temperature=0.0, ignore_eos=True))
            stats = engine.stats()
            engine.scheduler.check_invariants()
            assert engine.cache.slots.num_free == engine.cache.slots.num_slots
        assert stats["num_preemptions"] > 0 and stats["num_overlapped_steps"] > 0, stats
        for prompt, out in zip(prompts, outputs):
            assert out.output_tokens == 30
            logits = plain_toy(config, weights, prompt + out.token_ids)
            for i, token in enumerate(out.token_ids):
                row = logits[len(prompt) + i - 1]
                best = int(row.argmax())
                assert token == best or row[best] - row[token] <= 1e-5, (i, token, best)
    finally:
        unregister_architecture("ToyStateForCausalLM")
        MIXERS.unregister("toy_decay")
