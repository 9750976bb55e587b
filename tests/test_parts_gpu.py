"""Each part of a layer alone, built through its registry with sizes of its own."""

import math

import pytest
import torch

import plain_qwen2 as P

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def close(got, ref, dtype):
    """Largest difference relative to the size of the values: 2e-6 in float32, 2e-2 in bfloat16."""
    bound = (2e-6 if dtype == torch.float32 else 2e-2) * max(1.0, ref.abs().max().item())
    return (got.double().cpu() - ref).abs().max().item() <= bound


def make_ctx(slices, num_groups, dtype):
    from turboserve_b200.engine.batch import StepContext, Workspace, build_step_batch

    batch = build_step_batch(slices, num_groups, DEV)
    return StepContext(batch=batch, workspace=Workspace(DEV), dtype=dtype, device=torch.device(DEV),
                       status=torch.zeros(1, dtype=torch.int32, device=DEV))


def bind_random(part, dtype, seed=0, scale=0.2):
    g = torch.Generator().manual_seed(seed)
    host = {}
    for spec in part.param_specs():
        value = torch.randn(spec.shape, generator=g) * scale
        if spec.role == "gain":
            value = 1 + value
        value = value.to(dtype).float()  # what the device holds is exactly this
        host[spec.name] = value
    part.bind({name: v.to(DEV).to(next(s for s in part.param_specs() if s.name == name).device_dtype(dtype)) for name, v in host.items()})
    return {k: v.double() for k, v in host.items()}


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    from turboserve_b200.config import PartSpec
    from turboserve_b200.engine.batch import RequestSlice
    from turboserve_b200.parts import NORMS

    norm = NORMS.get("rms_norm")(PartSpec("rms_norm", {"eps": 2e-5}), 72, dtype, DEV)
    w = bind_random(norm, dtype)
    ctx = make_ctx([RequestSlice([1] * 6, 0, [[0]])], 1, dtype)
    residual = torch.randn(6, 72, device=DEV)
    delta = torch.randn(6, 72, device=DEV).to(dtype)
    expect = residual.double().cpu() + delta.double().cpu()
    out = torch.empty(6, 72, dtype=dtype, device=DEV)
    norm.forward(residual, delta, out, ctx)
    assert close(out, P.rms_norm(expect, w["weight"], 2e-5), dtype)
    assert torch.allclose(residual.double().cpu(), expect, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    """The two parts around the layers, alone: rows of the table into the float32 residual stream (an
    id beyond the table is flagged, not read), and float32 logits from the head's own matrix or,
    tied, from the embedding's; a vocabulary and a width that are no power of two."""
    from turboserve_b200.config import PartSpec
    from turboserve_b200.engine.batch import RequestSlice
    from turboserve_b200.parts import EMBEDDINGS, HEADS

    hidden, vocab = 72, 101
    embedding = EMBEDDINGS.get("table")(PartSpec("table"), hidden, vocab, dtype, DEV)
    table = bind_random(embedding, dtype, seed=3)["weight"]
    ids = [5, 100, 0, 17, 17, 64]
    ctx = make_ctx([RequestSlice(ids, 0, [[0]])], 1, dtype)
    residual = torch.full((6, hidden), float("nan"), device=DEV)
    embedding.forward(residual, ctx)
    assert torch.equal(residual.double().cpu(), table[torch.tensor(ids)]) and int(ctx.status.item()) == 0
    assert embedding.table.dtype == dtype and embedding.scratch_per_token() == 0 and embedding.graph_safe
    ctx.batch.token_ids[1] = vocab  # beyond the table
    embedding.forward(residual, ctx)
    assert int(ctx.status.item()) & 1

    rows = torch.randn(4, hidden).to(dtype)
    for tied in (False, True):
        head = HEADS.get("linear")(PartSpec("linear"), hidden, vocab, dtype, DEV, tied=tied)
        assert [p.name for p in head.param_specs()] == ([] if tied else ["weight"])
        if tied:
            head.bind({})
            head.tie(embedding.table)
            matrix = table
            with pytest.raises(ValueError):
                head.tie(embedding.table[:, :8])
        else:
            matrix = bind_random(head, dtype, seed=4)["weight"]
        logits = torch.full((4, vocab), float("nan"), device=DEV)
        head.forward(rows.to(DEV), logits, 3, ctx)
        assert logits.dtype == torch.float32 and torch.isnan(logits[3]).all()  # only the rows that were asked for
        ref = rows.double()[:3] @ matrix.T
        bound = (2e-5 if dtype == torch.float32 else 2e-2) * max(1.0, ref.abs().max().item())
        assert (logits[:3].double().cpu() - ref).abs().max().item() <= bound


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["silu", "gelu_pytorch_tanh"])
def test_feed_forward_part(dtype, act):
    from turboserve_b200.config import PartSpec
    from turboserve_b200.engine.batch import RequestSlice
    from turboserve_b200.parts import FEED_FORWARDS

    # 136: gate rows then up rows; 192: runs of 64 (in bfloat16 few rows take the product with the fused activation)
    for inter in (136, 192):
        mlp = FEED_FORWARDS.get("gated_mlp")(PartSpec("gated_mlp", {"intermediate_size": inter, "activation": act, "bias": inter == 192}), 72, dtype, DEV)
        w = bind_random(mlp, dtype)
        assert mlp.gate_block == (64 if inter == 192 else 0)
        for rows in (3, 70):  # the few-rows product and the many-rows product
            ctx = make_ctx([RequestSlice([1] * rows, 0, [[0] * 8])], 1, dtype)
            x = torch.randn(rows, 72).to(dtype)
            out = mlp.forward(x.to(DEV), ctx)
            if inter == 192:
                gate = x.double() @ w["gate_proj.weight"].T + w["gate_proj.bias"]
                up = x.double() @ w["up_proj.weight"].T + w["up_proj.bias"]
                act_fn = torch.nn.functional.silu if act == "silu" else (lambda t: torch.nn.functional.gelu(t, approximate="tanh"))
                ref = (act_fn(gate) * up) @ w["down_proj.weight"].T + w["down_proj.bias"]
            else:
                ref = P.mlp(x.double(), w["gate_proj.weight"], w["up_proj.weight"], w["down_proj.weight"], act)
            assert close(out, ref, dtype), (inter, rows)


def test_position_part():
    from turboserve_b200.config import PartSpec
    from turboserve_b200.parts import POSITIONS

    rope = POSITIONS.get("rotary")(PartSpec("rotary", {"rotary_dim": 48, "theta": 777.0, "factor": 2.0}), DEV)
    expect = 1.0 / (777.0 ** (torch.arange(0, 48, 2, dtype=torch.float32) / 48))
    assert torch.equal(rope.inv_freq.cpu(), expect) and rope.factor == 2.0
    with pytest.raises(ValueError):
        POSITIONS.get("rotary")(PartSpec("rotary", {"rotary_dim": 7, "theta": 1.0}), DEV)


def plain_attention_layer(x, w, nh, nkv, d, theta, factor, window, scale, qkv_bias=True):
    t = x.shape[0]
    def proj(name, heads):
        y = x @ w[f"{name}.weight"].T
        if qkv_bias:
            y = y + w[f"{name}.bias"]
        return y.view(t, heads, d)
    q, k, v = proj("q_proj", nh), proj("k_proj", nkv), proj("v_proj", nkv)
    cos, sin = P.rope_cos_sin(torch.arange(t), d, theta, factor, torch.float64)
    q, k = P.apply_rope(q, cos, sin), P.apply_rope(k, cos, sin)
    attended = P.attention(q * (scale / d ** -0.5), k, v, window).reshape(t, nh * d)
    return attended @ w["o_proj.weight"].T + w["o_proj.bias"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 9])
def test_attention_mixer_part_whole_and_cut(dtype, window):
    from turboserve_b200.cache import CacheStorage, GroupSpec, plan_cache
    from turboserve_b200.config import PartSpec
    from turboserve_b200.engine.batch import RequestSlice
    from turboserve_b200.parts import MIXERS

    hidden, nh, nkv, d, scale = 88, 5, 1, 16, 0.3
    spec = PartSpec("attention", dict(num_heads=nh, num_kv_heads=nkv, head_dim=d, scale=scale, qkv_bias=True, out_bias=True, window=window))
    position = PartSpec("rotary", dict(rotary_dim=d, theta=300.0, factor=1.0))
    mixer = MIXERS.get("attention")(spec, hidden, dtype, DEV, position=position)
    w = bind_random(mixer, dtype)
    plan = plan_cache([mixer.cache_need()], [None])
    storage = CacheStorage(plan, [GroupSpec("g", window, 16, 4)], 2, dtype, DEV)
    t = 23
    x = torch.randn(t, hidden).to(dtype)
    ref = plain_attention_layer(x.double(), w, nh, nkv, d, 300.0, 1.0, window, scale)
    table = [7, 2, 9, 0, 5, 11]
    ctx = make_ctx([RequestSlice([0] * t, 0, [table])], 1, dtype)
    whole = mixer.forward(x.to(DEV), ctx, storage.run_caches[0]).double().cpu()
    assert close(whole, ref, dtype)
    # the same through another set of pages, in three portions
    storage2 = CacheStorage(plan, [GroupSpec("g", window, 16, 4)], 2, dtype, DEV)
    table2 = [1, 15, 3, 8, 4, 6]
    parts, start = [], 0
    for n in (10, 2, 11):
        ctx = make_ctx([RequestSlice([0] * n, start, [table2])], 1, dtype)
        parts.append(mixer.forward(x[start:start + n].to(DEV), ctx, storage2.run_caches[0]).double().cpu())
        start += n
    cut = torch.cat(parts)
    assert close(cut, ref, dtype)
    if dtype == torch.float32:
        assert torch.equal(cut, whole)


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part(dtype):
    from turboserve_b200.cache import CacheStorage, GroupSpec, plan_cache
    from turboserve_b200.config import PartSpec
    from turboserve_b200.engine.batch import RequestSlice
    from turboserve_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS

    hidden, nh, nkv, d, inter, eps = 64, 2, 2, 32, 72, 1e-4
    mixer = MIXERS.get("attention")(PartSpec("attention", dict(num_heads=nh, num_kv_heads=nkv, head_dim=d, qkv_bias=True)), hidden, dtype, DEV,
                                    position=PartSpec("rotary", dict(rotary_dim=d, theta=1e4)))
    ff = FEED_FORWARDS.get("gated_mlp")(PartSpec("gated_mlp", dict(intermediate_size=inter)), hidden, dtype, DEV)
    n1 = NORMS.get("rms_norm")(PartSpec("rms_norm", dict(eps=eps)), hidden, dtype, DEV)
    n2 = NORMS.get("rms_norm")(PartSpec("rms_norm", dict(eps=eps)), hidden, dtype, DEV)
    wm, wf, w1, w2 = bind_random(mixer, dtype, 1), bind_random(ff, dtype, 2), bind_random(n1, dtype, 3), bind_random(n2, dtype, 4)
    block = BLOCKS.get("pre_norm")(mixer, ff, n1, n2)
    weights = {"p.input_layernorm.weight": w1["weight"], "p.post_attention_layernorm.weight": w2["weight"]}
    weights.update({f"p.self_attn.{k}": v for k, v in wm.items()})
    weights.update({f"p.mlp.{k}": v for k, v in wf.items()})
    t = 13
    h0 = torch.randn(t, hidden)
    dims = dict(nh=nh, nkv=nkv, d=d, eps=eps, theta=1e4, factor=1.0, act="silu")
    ref = P.decoder_layer(h0.double(), weights, "p.", dims, torch.arange(t), None)
    storage = CacheStorage(plan_cache([mixer.cache_need()], [None]), [GroupSpec("g", None, 8, 4)], 1, dtype, DEV)
    ctx = make_ctx([RequestSlice([0] * t, 0, [[3, 1, 6, 2]])], 1, dtype)
    residual = h0.to(DEV).clone()
    pending = block.forward(residual, None, ctx, storage.run_caches[0])
    got = residual.double().cpu() + pending.double().cpu()
    assert close(got, ref, dtype)


def test_run_order_may_name_a_layer_twice_and_share_a_cache():
    """A model whose order is data: layer 0, layer 1, layer 0 again, then a layer reading run 1's cache."""
    from turboserve_b200.cache import CacheManager
    from turboserve_b200.config import LayerRun, LayerSpec, ModelSpec, PartSpec
    from turboserve_b200.engine.batch import RequestSlice
    from turboserve_b200.engine.runner import ModelRunner, make_groups
    from turboserve_b200.models import DecoderModel

    hidden, nh, nkv, d, inter, vocab, eps = 48, 3, 1, 16, 40, 50, 1e-6
    norm = PartSpec("rms_norm", dict(eps=eps))
    attn = PartSpec("attention", dict(num_heads=nh, num_kv_heads=nkv, head_dim=d, qkv_bias=True))
    rope = PartSpec("rotary", dict(rotary_dim=d, theta=1e4))
    ff = PartSpec("gated_mlp", dict(intermediate_size=inter))
    layer = LayerSpec(attn, ff, norm, norm, rope)
    spec = ModelSpec("Toy", hidden, vocab, (layer, layer, layer), (LayerRun(0), LayerRun(1), LayerRun(0), LayerRun(2, cache_from=1)),
                     norm, tie_word_embeddings=True)
    model = DecoderModel(spec, torch.float32, DEV)
    names = [p.name for p in model.named_params()]
    assert "model.layers.2.self_attn.k_proj.weight" not in names and "model.layers.2.self_attn.q_proj.weight" in names
    plan = model.cache_plan()
    assert [r.owner for r in plan.runs] == [0, 1, 2, 1] and len(plan.windows) == 1
    g = torch.Generator().manual_seed(0)
    w = {}
    for p in model.named_params():
        v = torch.randn(p.spec.shape, generator=g) * 0.1
        w[p.name] = 1 + v if p.spec.role == "gain" else v
    model.bind({k: v.to(DEV) for k, v in w.items()})
    wd = {k: v.double() for k, v in w.items()}
    t = 21
    ids = torch.randint(0, vocab, (t,), generator=g)
    dims = dict(nh=nh, nkv=nkv, d=d, eps=eps, theta=1e4, factor=1.0, act="silu")
    pos = torch.arange(t)
    h = P.embed(wd["model.embed_tokens.weight"], ids)
    h = P.decoder_layer(h, wd, "model.layers.0.", dims, pos, None)
    # run 1, keeping its keys and values for the last run
    x1 = P.rms_norm(h, wd["model.layers.1.input_layernorm.weight"], eps)
    cos, sin = P.rope_cos_sin(pos, d, 1e4, 1.0, torch.float64)
    k1 = P.apply_rope((x1 @ wd["model.layers.1.self_attn.k_proj.weight"].T + wd["model.layers.1.self_attn.k_proj.bias"]).view(t, nkv, d), cos, sin)
    v1 = (x1 @ wd["model.layers.1.self_attn.v_proj.weight"].T + wd["model.layers.1.self_attn.v_proj.bias"]).view(t, nkv, d)
    h = P.decoder_layer(h, wd, "model.layers.1.", dims, pos, None)
    h = P.decoder_layer(h, wd, "model.layers.0.", dims, pos, None)
    x = P.rms_norm(h, wd["model.layers.2.input_layernorm.weight"], eps)
    q = P.apply_rope((x @ wd["model.layers.2.self_attn.q_proj.weight"].T + wd["model.layers.2.self_attn.q_proj.bias"]).view(t, nh, d), cos, sin)
    h = h + P.attention(q, k1, v1, None).reshape(t, nh * d) @ wd["model.layers.2.self_attn.o_proj.weight"].T
    x = P.rms_norm(h, wd["model.layers.2.post_attention_layernorm.weight"], eps)
    h = h + P.mlp(x, wd["model.layers.2.mlp.gate_proj.weight"], wd["model.layers.2.mlp.up_proj.weight"], wd["model.layers.2.mlp.down_proj.weight"], "silu")
    ref = P.rms_norm(h, wd["model.norm.weight"], eps) @ wd["model.embed_tokens.weight"].T

    groups = make_groups(plan, 8, 6)
    runner = ModelRunner(model, groups, 2)
    manager = CacheManager(groups, 2)
    manager.admit("a")
    got, start = [], 0
    for n in (9, 1, 11):
        manager.grow("a", n)
        out = runner.step([RequestSlice(ids[start:start + n].tolist(), start, [list(x) for x in manager.tables("a")], 0, list(range(n)))])
        got.append(out.double().cpu())
        start += n
    runner.check_status()
    assert torch.allclose(torch.cat(got), ref, atol=5e-6)
