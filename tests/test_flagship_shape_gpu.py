"""One layer with the flagship's own sizes (Qwen2-7B: hidden 3584, 28 query heads on 4 kv heads of 128,
intermediate 18944, vocabulary 152064, untied head) against the plain implementation, in float32
and bfloat16: the kernels at the widths the benchmark runs them at, not only at tiny ones. And
the same with the widths of the benchmark's larger workloads (Qwen2.5-14B: hidden 5120, 40 query
heads on 8 kv heads, intermediate 13824), where the matrix products take other kernels."""

import pytest
import torch

import plain_qwen2 as P
import traces
from tolerances import FP32_ATOL, FP32_ATOL_REAL_WIDTHS, check_logits

pytestmark = pytest.mark.gpu

FLAGSHIP_LAYER = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=1, hidden_size=3584,
    num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944, vocab_size=152064,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False,
    max_position_embeddings=4096,
)


LARGER_LAYER = dict(FLAGSHIP_LAYER, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                    intermediate_size=13824, rms_norm_eps=1e-5)


@pytest.fixture(scope="module", params=[FLAGSHIP_LAYER, LARGER_LAYER], ids=["7b", "14b"])
def flagship(request, tmp_path_factory):
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.weights import write_random_model

    folder = write_random_model(config_from_dict(request.param), 0, tmp_path_factory.mktemp("flagship"), torch.bfloat16)
    config, weights = P.read_model_folder(folder)
    requests = traces.make_requests(config["vocab_size"], [70, 9, 33], seed=21)
    ref = {rid: P.forward_logits(config, weights, tokens) for rid, tokens in requests.items()}
    # what float32 arithmetic itself costs at these widths (inner sizes up to 18944 where the tiny
    # models have 256 at most): the plain implementation evaluated in float32 against itself in float64
    plain32 = max((P.forward_logits(config, weights, tokens, dtype=torch.float32).double() - ref[rid]).abs().max().item()
                  for rid, tokens in requests.items())
    return folder, requests, ref, plain32


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_layer_of_the_flagship_shape(flagship, dtype):
    from turboserve_b200.replay import Replayer

    folder, requests, ref, plain32 = flagship
    for builder, kwargs in ((traces.whole, {}), (traces.tail_one_by_one, {"tail": 12}), (traces.mixed, {"seed": 4, "max_live": 3})):
        steps, max_tokens = builder(requests, **kwargs)
        replayer = Replayer(folder, dtype, max_tokens)
        got = traces.collect(requests, steps, traces.replay(replayer, steps))
        for rid in requests:
            if dtype == "float32":
                # the bound of the tiny models, or four times what a plain float32 evaluation loses
                # at these widths, whichever is larger (the engine's sums run in another order),
                # and never more than the constant fixed beforehand for these widths
                worst = (got[rid].double() - ref[rid]).abs().max().item()
                bound = min(max(FP32_ATOL, 4.0 * plain32), FP32_ATOL_REAL_WIDTHS)
                print(f"one layer, {builder.__name__} {rid}: engine {worst:.3e}, plain float32 {plain32:.3e}, bound {bound:.3e}")
                assert torch.isfinite(got[rid]).all() and worst <= bound, (builder.__name__, rid, worst, bound, plain32)
            else:
                check_logits(got[rid], ref[rid], dtype, f"flagship layer {dtype} {builder.__name__} {rid}")
        del replayer
        torch.cuda.empty_cache()
