"""The plain implementation itself: pinned to the reference's arithmetic, and its own parts (no GPU)."""

import json
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen2 as P
from conftest import TINY_B

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["gqa_tied", "mqa_untied", "windowless_b"])
def test_plain_equals_the_reference_model_code(name):
    """Logits stored by tests/golden/make_reference_golden.py from the reference's own CausalLM."""
    data = np.load(GOLDEN / f"reference_qwen2_{name}.npz")
    config = json.loads(bytes(data["config_json"]).decode())
    weights = {key[2:]: torch.from_numpy(data[key]) for key in data.files if key.startswith("w:")}
    ours = P.forward_logits(config, weights, data["token_ids"].tolist())
    theirs = torch.from_numpy(data["logits"]).double()
    assert ours.shape == theirs.shape
    # the reference computed in float32: its own rounding is what is left
    assert (ours - theirs).abs().max().item() < 5e-6


def test_a_window_that_cannot_bind_changes_nothing_the_reference_computes():
    """The second tiny configuration's sizes, run by the reference with the window off (it rejects
    one): the plain implementation with the window ON equals it on a prompt shorter than the
    window, and differs from it (so the window is really on) on the longer prompt."""
    data = np.load(GOLDEN / "reference_qwen2_windowless_b.npz")
    config = json.loads(bytes(data["config_json"]).decode())
    for key in ("hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim", "intermediate_size", "vocab_size",
                "num_hidden_layers", "rope_theta", "rms_norm_eps", "sliding_window", "max_window_layers"):
        assert config[key] == TINY_B[key], key
    weights = {key[2:]: torch.from_numpy(data[key]) for key in data.files if key.startswith("w:")}
    windowed = dict(config, use_sliding_window=True)
    assert [P.layer_window(windowed, i) for i in range(3)] == [None, 32, 32]
    short = P.forward_logits(windowed, weights, data["short_token_ids"].tolist())
    assert len(data["short_token_ids"]) == 29
    assert (short - torch.from_numpy(data["short_logits"]).double()).abs().max().item() < 5e-6
    long_on = P.forward_logits(windowed, weights, data["token_ids"].tolist())
    theirs = torch.from_numpy(data["logits"]).double()
    assert (long_on[:32] - theirs[:32]).abs().max().item() < 5e-6  # the first 32 positions see everything either way
    assert (long_on[32:] - theirs[32:]).abs().max().item() > 1e-3  # from position 32 on the window hides keys


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    t, nh, nkv, d = 9, 4, 2, 8
    q, k, v = torch.randn(t, nh, d, dtype=torch.float64), torch.randn(t, nkv, d, dtype=torch.float64), torch.randn(t, nkv, d, dtype=torch.float64)
    full = P.attention(q, k, v, None)
    # by hand, one query head at a time
    for head in range(nh):
        kv = head // 2
        for i in range(t):
            scores = (k[: i + 1, kv] @ q[i, head]) * d ** -0.5
            expect = torch.softmax(scores, 0) @ v[: i + 1, kv]
            assert torch.allclose(full[i, head], expect, atol=1e-12)
    win = P.attention(q, k, v, 3)
    for i in range(t):
        lo = max(0, i - 2)
        scores = (k[lo: i + 1, 0] @ q[i, 0]) * d ** -0.5
        assert torch.allclose(win[i, 0], torch.softmax(scores, 0) @ v[lo: i + 1, 0], atol=1e-12)
    assert torch.allclose(win[:3], full[:3])  # the window does not bind before it is full
    # a change to a future key or to a key behind the window changes nothing
    k2 = k.clone(); k2[5] += 10
    assert torch.equal(P.attention(q, k2, v, None)[:5], full[:5])
    assert torch.equal(P.attention(q, k2, v, 3)[8], win[8])


def test_rope_is_a_rotation_that_depends_on_distance_only():
    d = 16
    x = torch.randn(5, 1, d, dtype=torch.float64)
    pos = torch.arange(5)
    cos, sin = P.rope_cos_sin(pos, d, 10000.0, 1.0, torch.float64)
    y = P.apply_rope(x, cos, sin)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    assert torch.equal(y[0], x[0])  # position 0 is the identity
    a, b = torch.randn(1, 1, d, dtype=torch.float64), torch.randn(1, 1, d, dtype=torch.float64)
    def dot(pa, pb):
        ca, sa = P.rope_cos_sin(torch.tensor([pa]), d, 10000.0, 1.0, torch.float64)
        cb, sb = P.rope_cos_sin(torch.tensor([pb]), d, 10000.0, 1.0, torch.float64)
        return (P.apply_rope(a, ca, sa) * P.apply_rope(b, cb, sb)).sum()
    assert abs(dot(3, 1) - dot(10, 8)) < 1e-6
    c2, s2 = P.rope_cos_sin(torch.tensor([8]), d, 10000.0, 2.0, torch.float64)
    c1, s1 = P.rope_cos_sin(torch.tensor([4]), d, 10000.0, 1.0, torch.float64)
    assert torch.equal(c2, c1) and torch.equal(s2, s1)  # linear scaling divides the position


def test_norm_and_mlp():
    x = torch.randn(3, 10, dtype=torch.float64)
    w = torch.rand(10, dtype=torch.float64) + 0.5
    y = P.rms_norm(x, w, 1e-6)
    assert torch.allclose((y / w).pow(2).mean(-1), torch.ones(3, dtype=torch.float64), atol=1e-5)
    g, u, dn = torch.randn(7, 10, dtype=torch.float64), torch.randn(7, 10, dtype=torch.float64), torch.randn(10, 7, dtype=torch.float64)
    out = P.mlp(x, g, u, dn, "silu")
    hand = ((x @ g.T) / (1 + torch.exp(-(x @ g.T))) * (x @ u.T)) @ dn.T
    assert torch.allclose(out, hand)


def test_layer_window_rule():
    assert [P.layer_window(TINY_B, i) for i in range(3)] == [None, 32, 32]
    assert P.layer_window({**TINY_B, "use_sliding_window": False}, 2) is None


def test_sampling_stages():
    logits = torch.tensor([2.0, 1.0, 0.5, -1.0, 3.0, 0.0])
    assert P.sample_token(logits, temperature=0.0)[0] == 4
    # a penalty on the top token moves the argmax
    tok, lp = P.sample_token(logits, temperature=0.0, repetition_penalty=4.0, history=[4, 4, 3])
    assert tok == 0 and lp == pytest.approx(float(torch.log_softmax(torch.tensor([2.0, 1.0, 0.5, -4.0, 0.75, 0.0]), 0)[0]))
    # top-k = 1 and a tiny top-p are greedy whatever the noise
    for counter in range(20):
        assert P.sample_token(logits, temperature=1.5, top_k=1, seed=3, counter=counter)[0] == 4
        assert P.sample_token(logits, temperature=1.5, top_p=0.01, seed=3, counter=counter)[0] == 4
        assert P.sample_token(logits, temperature=1.0, top_k=2, seed=9, counter=counter)[0] in (0, 4)
    # draws follow the softmax
    counts = torch.zeros(6)
    for counter in range(4000):
        counts[P.sample_token(logits, temperature=1.0, seed=1, counter=counter)[0]] += 1
    assert (counts / 4000 - torch.softmax(logits, 0)).abs().max() < 0.03
    u = P.sample_uniforms(5, 7, 1000)
    assert 0 < u.min() and u.max() < 1 and abs(u.mean() - 0.5) < 0.05
