"""Weights: the random-weights folder, loading by name, and the one error that lists everything (no GPU)."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from conftest import TINY_A, TINY_B
from turboserve_b200.config import config_from_dict, lookup
from turboserve_b200.weights import WeightLoadError, load_weights, write_random_model


def build(raw, dtype=torch.float32):
    config = config_from_dict(raw)
    return config, lookup(config.architecture).build_model(config, dtype, "cpu")


def test_random_folder_is_deterministic_and_complete(tmp_path):
    config, model = build(TINY_A)
    one = write_random_model(config, 0, tmp_path / "one")
    two = write_random_model(config, 0, tmp_path / "two")
    other = write_random_model(config, 1, tmp_path / "other")
    a, b, c = (load_file(str(p / "model.safetensors")) for p in (one, two, other))
    assert set(a) == {p.name for p in model.named_params()}
    assert "lm_head.weight" not in a  # tied
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert any(not torch.equal(a[k], c[k]) for k in a)
    assert all(t.dtype == torch.bfloat16 for t in a.values())
    assert json.loads((one / "config.json").read_text())["architectures"] == ["Qwen2ForCausalLM"]
    # the init rules: matrices N(0, 0.02), biases not zero, gains around one
    assert 0.015 < a["model.layers.0.mlp.gate_proj.weight"].float().std() < 0.025
    assert a["model.layers.0.self_attn.q_proj.bias"].float().abs().max() > 0
    gain = a["model.norm.weight"].float()
    assert abs(gain.mean() - 1) < 0.01 and 0.005 < gain.std() < 0.02


def test_load_keeps_dtypes_by_role(tmp_path):
    config, model = build(TINY_B, torch.bfloat16)
    folder = write_random_model(config, 1, tmp_path / "m", torch.float32)
    stored = load_weights(model, folder)
    assert set(stored.values()) == {"F32"}
    assert model.embedding.table.dtype == torch.bfloat16 and model.head.weight.dtype == torch.bfloat16
    assert model.blocks[0].mixer.qkv.dtype == torch.bfloat16
    assert model.blocks[0].mixer.qkv_b.dtype == torch.float32  # a bias stored in 32-bit stays so
    assert model.final_norm.gain.dtype == torch.float32
    raw = load_file(str(folder / "model.safetensors"))
    assert torch.equal(model.final_norm.gain, raw["model.norm.weight"])
    q = raw["model.layers.1.self_attn.q_proj.weight"].to(torch.bfloat16)
    assert torch.equal(model.blocks[1].mixer.qkv[: q.shape[0]], q)
    assert model.head.weight is not model.embedding.table


def test_tied_head_shares_storage_and_tolerates_a_copy(tmp_path):
    config, model = build(TINY_A)
    folder = write_random_model(config, 0, tmp_path / "m")
    tensors = load_file(str(folder / "model.safetensors"))
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    save_file(tensors, str(folder / "model.safetensors"))
    load_weights(model, folder)
    assert model.head.weight is model.embedding.table


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config, model = build(TINY_B)
    folder = write_random_model(config, 1, tmp_path / "m")
    tensors = load_file(str(folder / "model.safetensors"))
    del tensors["model.layers.2.mlp.up_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.extra.weight"] = torch.zeros(3)
    tensors["model.norm.weight"] = torch.zeros(95, dtype=torch.bfloat16)
    tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(32, 95, dtype=torch.bfloat16)
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightLoadError) as info:
        load_weights(model, folder)
    text = str(info.value)
    assert "missing tensors (2)" in text and "model.layers.2.mlp.up_proj.weight" in text and "lm_head.weight" in text
    assert "unexpected tensors (1)" in text and "model.layers.0.extra.weight" in text
    assert "wrong shapes (2)" in text and "model.norm.weight: checkpoint has [95], model needs [96]" in text
    assert not model.loaded


def test_folder_errors(tmp_path):
    config, model = build(TINY_A)
    with pytest.raises(WeightLoadError, match="does not exist"):
        load_weights(model, tmp_path / "nothing")
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(WeightLoadError, match="no safetensors"):
        load_weights(model, empty)
    (empty / "pytorch_model.bin").write_bytes(b"x")
    with pytest.raises(WeightLoadError, match="pickled"):
        load_weights(model, empty)
    (empty / "model.safetensors").write_bytes(b"short")
    with pytest.raises(WeightLoadError, match="not a safetensors"):
        load_weights(model, empty)
    a_file = tmp_path / "file"
    a_file.write_text("x")
    with pytest.raises(WeightLoadError, match="is a file"):
        load_weights(model, a_file)


def test_sharded_checkpoint_and_missing_shard(tmp_path):
    config, model = build(TINY_A)
    folder = write_random_model(config, 0, tmp_path / "m")
    tensors = load_file(str(folder / "model.safetensors"))
    names = sorted(tensors)
    half = len(names) // 2
    save_file({n: tensors[n] for n in names[:half]}, str(folder / "model-00001-of-00002.safetensors"))
    save_file({n: tensors[n] for n in names[half:]}, str(folder / "model-00002-of-00002.safetensors"))
    (folder / "model.safetensors").unlink()
    weight_map = {n: "model-00001-of-00002.safetensors" for n in names[:half]}
    weight_map.update({n: "model-00002-of-00002.safetensors" for n in names[half:]})
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    load_weights(model, folder)
    assert model.loaded
    (folder / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(WeightLoadError, match="lists shard"):
        load_weights(model, folder)
    (folder / "model.safetensors.index.json").write_text(json.dumps({"nothing": 1}))
    with pytest.raises(WeightLoadError, match="weight_map"):
        load_weights(model, folder)


def test_exporter_prefixes_are_rewritten_before_names_are_compared(tmp_path):
    """``transformer.`` / ``language_model.model.`` / ``language_model.lm_head.`` / ``model.decoder.`` in
    front of the decoder stack load as ``model.`` / ``lm_head.``
    (``src/turboserve/engine/model/weights.py:56-61,181-196``); a name left over is still reported."""
    config, model = build(TINY_B)
    folder = write_random_model(config, 1, tmp_path / "m", torch.float32)
    plain = {name: tensor.clone() for name, tensor in load_file(str(folder / "model.safetensors")).items()}  # the file is rewritten below
    for old_model, old_head in (("transformer.", "lm_head."), ("language_model.model.", "language_model.lm_head."),
                                ("model.decoder.", "lm_head.")):
        renamed = {}
        for name, tensor in plain.items():
            if name.startswith("model."):
                renamed[old_model + name[len("model."):]] = tensor
            else:
                renamed[old_head + name[len("lm_head."):]] = tensor
        assert "model.embed_tokens.weight" not in renamed
        save_file(renamed, str(folder / "model.safetensors"))
        _, fresh = build(TINY_B)
        load_weights(fresh, folder)
        assert torch.equal(fresh.head.weight, plain["lm_head.weight"]) and torch.equal(fresh.embedding.table, plain["model.embed_tokens.weight"])
        assert torch.equal(fresh.blocks[2].feed_forward.down, plain["model.layers.2.mlp.down_proj.weight"])
    renamed["transformer.extra.weight"] = torch.zeros(2)
    save_file(renamed, str(folder / "model.safetensors"))
    with pytest.raises(WeightLoadError, match=r"unexpected tensors \(1\): model.extra.weight"):
        load_weights(build(TINY_B)[1], folder)


def test_parts_are_bound_one_at_a_time(tmp_path):
    """Loading fetches a part's tensors, binds them and lets them go before the next part's are
    read: at no time are the unfused tensors of more than one part alive."""
    import gc
    import weakref

    config, model = build(TINY_B)
    folder = write_random_model(config, 1, tmp_path / "m", torch.float32)
    alive, most = [], [0]
    bind_stream = model.bind_stream

    def watching(fetch):
        def watched(param):
            gc.collect()
            matrices = [ref for ref in alive if ref() is not None]
            most[0] = max(most[0], len(matrices))
            value = fetch(param)
            if any(f".{n}_proj.weight" in param.name for n in "qkv") or "gate_proj" in param.name or "up_proj" in param.name:
                alive.append(weakref.ref(value))  # tensors that bind() fuses into new ones
            return value

        bind_stream(watched)

    model.bind_stream = watching
    load_weights(model, folder)
    # q, k and v of one attention part, or gate and up of one feed-forward; never two parts' worth
    assert 0 < most[0] <= 3
