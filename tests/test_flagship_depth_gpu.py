"""Qwen2-7B's own widths at depth: eight layers (all 28 when ``TURBOSERVE_B200_DEPTH=28``)
against the plain implementation evaluated in float64 on the GPU.

float32 through replay, whole, with the tail one token at a time, and mixed, within a bound
fixed beforehand; bfloat16 through replay and, with captured graphs and steps launched ahead,
through ``LLMEngine.generate``. The one-layer tests next to this file check the kernels at
these widths; this one checks that nothing drifts over many layers of them.
"""

import os

import pytest
import torch

import plain_qwen2 as P
import traces
from tolerances import bf16_bounds, check_logits, fp32_atol_real_widths

pytestmark = pytest.mark.gpu

DEPTH = int(os.environ.get("TURBOSERVE_B200_DEPTH", "8"))
QWEN2_7B = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=DEPTH, hidden_size=3584,
    num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944, vocab_size=152064,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False,
    max_position_embeddings=4096,
)


@pytest.fixture(scope="module")
def deep(tmp_path_factory):
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.weights import write_random_model

    folder = write_random_model(config_from_dict(QWEN2_7B), 0, tmp_path_factory.mktemp("deep"), torch.bfloat16)
    config, weights = P.read_model_folder(folder)
    requests = traces.make_requests(config["vocab_size"], [70, 9, 33], seed=22)
    ref = {rid: P.forward_logits(config, weights, tokens, device="cuda") for rid, tokens in requests.items()}
    plain32 = max((P.forward_logits(config, weights, tokens, dtype=torch.float32, device="cuda").double() - ref[rid]).abs().max().item()
                  for rid, tokens in requests.items())
    # and in bfloat16 throughout (products, norms, softmax all rounded): what that precision costs at this depth
    plain16 = max((P.forward_logits(config, weights, tokens, dtype=torch.bfloat16, device="cuda").double() - ref[rid]).abs().max().item()
                  / max(1.0, ref[rid].abs().max().item()) for rid, tokens in requests.items())
    torch.cuda.empty_cache()
    return folder, config, weights, requests, ref, (plain32, plain16)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_widths_at_depth_through_replay(deep, dtype):
    from turboserve_b200.replay import Replayer

    folder, _, _, requests, ref, (plain32, plain16) = deep
    cuts = [(builder, builder(requests, **kwargs)) for builder, kwargs in
            ((traces.whole, {}), (traces.tail_one_by_one, {"tail": 32}), (traces.mixed, {"seed": 5, "max_live": 3}))]
    replayer = Replayer(folder, dtype, max(max_tokens for _, (_, max_tokens) in cuts))
    worst = worst_relative = 0.0
    for builder, (steps, _) in cuts:
        got = traces.collect(requests, steps, traces.replay(replayer, steps))
        assert replayer.manager.free_pages() == [g.num_pages for g in replayer.manager.groups]
        for rid in requests:
            difference = (got[rid].double() - ref[rid]).abs().max().item()
            worst = max(worst, difference)
            worst_relative = max(worst_relative, difference / max(1.0, ref[rid].abs().max().item()))
    print(f"{DEPTH} layers of the 7B widths, {dtype}: worst |engine - plain float64| {worst:.3e}, relative to the largest logit "
          f"{worst_relative:.3e} (plain float32 against float64: {plain32:.3e}; plain bfloat16, relative: {plain16:.3e}; "
          f"bounds: float32 {fp32_atol_real_widths(DEPTH):.1e}, bfloat16 {bf16_bounds(DEPTH)[0]:.3e}; "
          f"largest |logit| {max(r.abs().max().item() for r in ref.values()):.2f})")
    for builder, (steps, _) in cuts:
        got = traces.collect(requests, steps, traces.replay(replayer, steps))
        for rid in requests:
            check_logits(got[rid], ref[rid], dtype, f"{DEPTH} layers {dtype} {builder.__name__} {rid}",
                         fp32_atol=fp32_atol_real_widths(DEPTH), layers=DEPTH)
    if dtype == "bfloat16":
        assert worst_relative < plain16  # fp32 statistics and residual stream: nearer than bfloat16 throughout
    del replayer
    torch.cuda.empty_cache()


def test_real_widths_at_depth_generate_with_graphs(deep):
    """bfloat16 through the entry point, decode steps replayed from graphs and launched ahead: every
    token is the plain argmax given the tokens before it, or within the bfloat16 tolerance of it."""
    from turboserve_b200 import EngineConfig, LLMEngine, SamplingParams, SchedulerConfig

    folder, config, weights, requests, _, _ = deep
    slack_rel = bf16_bounds(DEPTH)[0]
    prompts = list(requests.values())
    engine = LLMEngine(EngineConfig(model=str(folder), dtype="bfloat16", scheduler=SchedulerConfig(
        max_num_seqs=4, max_num_batched_tokens=64, block_size=16, num_blocks=24)))
    with engine:
        outputs = engine.generate(prompts, SamplingParams(max_tokens=24, temperature=0.0, ignore_eos=True))
        assert engine.runner.num_graph_replays > 0 and engine.stats()["num_overlapped_steps"] > 0
    torch.cuda.empty_cache()
    for prompt, out in zip(prompts, outputs):
        assert out.output_tokens == 24
        logits = P.forward_logits(config, weights, prompt + out.token_ids, device="cuda")
        slack = slack_rel * max(1.0, logits.abs().max().item())
        for i, token in enumerate(out.token_ids):
            row = logits[len(prompt) + i - 1]
            best = int(row.argmax())
            assert token == best or row[best] - row[token] <= 2 * slack, (i, token, best, float(row[best] - row[token]))
