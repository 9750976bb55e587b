"""Run the reference's own model code once on the CPU and store what it computes.

    python tests/golden/make_reference_golden.py /path/to/reference/src

imports ``turboserve.engine.model.CausalLM`` from the given source tree (the reference needs
no build: it is pure Python), builds two tiny random Qwen2 models, copies this script's
random tensors into the reference's parameters by name, runs its paged forward over one whole
prompt with scrambled block ids, and writes ``reference_qwen2_<name>.npz`` beside this file:
the config, the weights, the token ids and the reference's float32 logits at every position.
``tests/test_plain.py`` compares ``tests/plain_qwen2.py`` with these files, so the
plain implementation is pinned to the reference's arithmetic without the reference being
present. The reference rejects a sliding window (``model/model_config.py:270-274``), so no case
has one. The third case has the sizes of the tests' second tiny configuration with its window
switched off, and a second, shorter prompt: 29 tokens, fewer than that configuration's window
of 32, where a window cannot bind, so the plain implementation with the window ON must give
the same logits there.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

CASES = {
    "gqa_tied": dict(
        architectures=["Qwen2ForCausalLM"], hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, intermediate_size=80, vocab_size=128, max_position_embeddings=128,
        rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True,
    ),
    "mqa_untied": dict(
        architectures=["Qwen2ForCausalLM"], hidden_size=48, num_hidden_layers=3, num_attention_heads=3,
        num_key_value_heads=1, head_dim=16, intermediate_size=72, vocab_size=200, max_position_embeddings=128,
        rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False,
        rope_scaling={"rope_type": "linear", "factor": 2.0},
    ),
    "windowless_b": dict(
        architectures=["Qwen2ForCausalLM"], hidden_size=96, num_hidden_layers=3, num_attention_heads=3,
        num_key_value_heads=1, head_dim=32, intermediate_size=256, vocab_size=1000, max_position_embeddings=512,
        rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False, use_sliding_window=False,
        sliding_window=32, max_window_layers=1,
    ),
}
SHORT_PROMPT = {"windowless_b": 29}
PROMPT_LEN = 37
BLOCK_SIZE = 8


def main(reference_src: str) -> None:
    sys.path.insert(0, reference_src)
    from turboserve.engine.core.kv_cache import KVCache
    from turboserve.engine.core.types import AttnMetadata, build_query_start_loc, pad_block_tables
    from turboserve.engine.model import CausalLM, ModelConfig

    for seed, (name, raw) in enumerate(CASES.items()):
        config = ModelConfig.from_dict(raw)
        model = CausalLM(config, dtype=torch.float32)
        generator = torch.Generator().manual_seed(100 + seed)
        weights: dict[str, torch.Tensor] = {}
        with torch.no_grad():
            for pname, param in model.named_parameters():
                if pname.endswith("layernorm.weight") or pname == "model.norm.weight":
                    value = 1.0 + 0.05 * torch.randn(param.shape, generator=generator)
                else:
                    value = 0.08 * torch.randn(param.shape, generator=generator)
                param.copy_(value)
                weights[pname] = value.clone()
        def run(length: int) -> tuple[torch.Tensor, torch.Tensor]:
            ids = torch.randint(0, raw["vocab_size"], (length,), generator=generator)
            num_blocks = -(-length // BLOCK_SIZE)
            order = torch.randperm(num_blocks + 3, generator=generator)[:num_blocks].tolist()
            cache = KVCache(config.num_hidden_layers, num_blocks + 3, BLOCK_SIZE, config.num_key_value_heads,
                            config.head_dim, dtype=torch.float32)
            slots = [order[p // BLOCK_SIZE] * BLOCK_SIZE + p % BLOCK_SIZE for p in range(length)]
            meta = AttnMetadata(
                slot_mapping=torch.tensor(slots), block_tables=pad_block_tables([order]),
                context_lens=torch.tensor([length]), query_start_loc=build_query_start_loc([length]),
                max_query_len=length, max_context_len=length, num_prefill_seqs=1,
            )
            with torch.no_grad():
                hidden = model(ids, torch.arange(length), cache, meta)
                return ids, model.compute_logits(hidden, list(range(length)))

        ids, logits = run(PROMPT_LEN)
        arrays = {f"w:{k}": v.numpy() for k, v in weights.items()}
        arrays["token_ids"] = ids.numpy()
        arrays["logits"] = logits.float().numpy()
        if name in SHORT_PROMPT:
            short_ids, short_logits = run(SHORT_PROMPT[name])
            arrays["short_token_ids"] = short_ids.numpy()
            arrays["short_logits"] = short_logits.float().numpy()
        arrays["config_json"] = np.frombuffer(json.dumps(raw).encode(), dtype=np.uint8)
        np.savez_compressed(HERE / f"reference_qwen2_{name}.npz", **arrays)
        print(name, "logits", tuple(logits.shape), "abs max", float(logits.abs().max()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_reference_golden.py <path to the reference's src folder>")
    main(sys.argv[1])
