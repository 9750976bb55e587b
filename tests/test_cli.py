"""The command line: names and meanings of its options, and what needs no GPU of its commands."""

import json

import pytest
import torch
from typer.testing import CliRunner

from conftest import TINY_A
from turboserve_b200.cli import app

runner = CliRunner()


def test_version_and_hwinfo_run_without_a_gpu():
    import turboserve_b200

    result = runner.invoke(app, ["version"])
    assert result.exit_code == 0 and turboserve_b200.__version__ in result.stdout
    result = runner.invoke(app, ["hwinfo"])
    assert result.exit_code == 0
    info = json.loads(result.stdout)
    assert info["torch"] == torch.__version__ and "cuda_available" in info


def test_generate_has_the_options_of_the_reference():
    import typer

    command = typer.main.get_command(app).commands["engine"].commands["generate"]
    options = {opt for param in command.params for opt in param.opts}
    for option in ("--model", "-m", "--max-tokens", "--temperature", "--top-p", "--top-k", "--seed", "--dtype", "--num-blocks",
                   "--max-num-seqs", "--max-num-batched-tokens", "--block-size", "--ignore-eos", "--stats", "--prompt-ids"):
        assert option in options, option
    defaults = {param.name: param.default for param in command.params}
    assert defaults["temperature"] == 0.0 and defaults["top_p"] == 1.0 and defaults["top_k"] == 0 and defaults["block_size"] == 16


def test_random_weights_writes_a_model_folder(tmp_path):
    from safetensors import safe_open

    config = tmp_path / "config.json"
    config.write_text(json.dumps(TINY_A))
    out = tmp_path / "model"
    result = runner.invoke(app, ["engine", "random-weights", "--config", str(config), "--out", str(out), "--seed", "7"])
    assert result.exit_code == 0, result.stdout
    written = json.loads((out / "config.json").read_text())
    assert written["hidden_size"] == TINY_A["hidden_size"] and written["architectures"] == ["Qwen2ForCausalLM"]
    with safe_open(str(out / "model.safetensors"), "pt") as f:
        names = set(f.keys())
        assert "model.embed_tokens.weight" in names and "model.layers.1.self_attn.q_proj.bias" in names
        assert "lm_head.weight" not in names  # tied to the embedding in this configuration
        assert f.get_tensor("model.norm.weight").dtype == torch.bfloat16
    again = tmp_path / "again"
    runner.invoke(app, ["engine", "random-weights", "--config", str(out), "--out", str(again), "--seed", "7"])
    from safetensors.torch import load_file

    first, second = load_file(str(out / "model.safetensors")), load_file(str(again / "model.safetensors"))
    assert first.keys() == second.keys() and all(torch.equal(first[k], second[k]) for k in first)  # the seed decides every value


def test_kv_size_plans_without_a_gpu(tmp_path):
    config = tmp_path / "config.json"
    config.write_text(json.dumps(TINY_A))
    result = runner.invoke(app, ["engine", "kv-size", "-m", str(tmp_path), "--total-memory-gib", "1", "--block-size", "16",
                                 "--max-num-seqs", "4", "--max-model-len", "256", "--dtype", "bfloat16"])
    assert result.exit_code == 0, result.stdout
    report = json.loads(result.stdout)
    assert report["num_blocks"] == 4 * (256 // 16) and report["source"] == "max_model_len"


@pytest.mark.gpu
def test_generate_prints_tokens(model_folders):
    result = runner.invoke(app, ["engine", "generate", "-m", str(model_folders["A"]), "--prompt-ids", "5,17,3", "--prompt-ids", "9",
                                 "--max-tokens", "6", "--ignore-eos", "--num-blocks", "32", "--dtype", "float32", "--stats"])
    assert result.exit_code == 0, result.stdout
    outputs = [line for line in result.stdout.splitlines() if line.startswith("output ")]
    assert len(outputs) == 2 and all(len(json.loads(line.split(": ", 1)[1])) == 6 for line in outputs)
    assert result.stdout.count("6 tokens, finish_reason=length") == 2
    assert '"num_finished": 2' in result.stdout  # --stats


@pytest.mark.gpu
def test_generate_with_a_penalty_and_log_probabilities(model_folders):
    result = runner.invoke(app, ["engine", "generate", "-m", str(model_folders["D"]), "--prompt-ids", "5,17,3,5,17,3", "--max-tokens", "8",
                                 "--ignore-eos", "--num-blocks", "32", "--repetition-penalty", "1.5", "--logprobs"])
    assert result.exit_code == 0, result.stdout
    line = next(line for line in result.stdout.splitlines() if line.strip().startswith("logprobs:"))
    values = [float(v) for v in line.split(":", 1)[1].split()]
    assert len(values) == 8 and all(v <= 0.0 for v in values)
