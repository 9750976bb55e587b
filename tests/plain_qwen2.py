"""A plain, slow Qwen2: whole sequences, no cache, one function per part, torch on the CPU.

This is what the engine is compared with. It shares no code with ``turboserve_b200``: it reads
``config.json`` with ``json`` and ``model.safetensors`` with ``safetensors`` itself, and every
function is written from the reference's formulas (file:line under
``src/turboserve/engine/``). Everything is computed in float64 unless ``dtype`` says
otherwise, from the stored weights upcast exactly.

``tests/golden/make_reference_golden.py`` compares this file once with the reference's own
``CausalLM`` on a tiny random model; the sliding window is not in the reference
(``model/model_config.py:270-274`` rejects it) and rests on the formula alone: a query at
position p sees keys j with ``p - window < j <= p``.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def read_model_folder(folder: str | Path) -> tuple[dict, dict[str, torch.Tensor]]:
    from safetensors.torch import load_file

    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    weights = load_file(str(folder / "model.safetensors"))
    return config, weights


def derived(config: dict) -> dict:
    """Sizes and constants by the reference's parsing rules (model/model_config.py:254-314)."""
    nh = config["num_attention_heads"]
    out = {
        "L": config["num_hidden_layers"],
        "H": config["hidden_size"],
        "nh": nh,
        "nkv": config.get("num_key_value_heads", nh),                      # :277-278
        "d": config.get("head_dim") or config["hidden_size"] // nh,        # :279-282
        "eps": float(config.get("rms_norm_eps", 1e-6)),                    # :301
        "theta": float(config.get("rope_theta", 10000.0)),                 # :112
        "factor": 1.0,
        "tie": bool(config.get("tie_word_embeddings", False)),            # :305
        "act": config.get("hidden_act", "silu"),
    }
    scaling = config.get("rope_scaling")
    if isinstance(scaling, dict) and (scaling.get("rope_type") or scaling.get("type")) == "linear":
        out["factor"] = float(scaling.get("factor", 1.0))                  # :120
    return out


def layer_window(config: dict, layer: int) -> int | None:
    """Keys a layer sees: layers >= max_window_layers are windowed when use_sliding_window."""
    if config.get("use_sliding_window") and config.get("sliding_window"):
        if layer >= config.get("max_window_layers", config["num_hidden_layers"]):
            return int(config["sliding_window"])
    return None


def embed(table: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
    """h0[t] = E[ids[t]]  (model/model.py:105)."""
    return table[token_ids]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """w * x * rsqrt(mean(x^2) + eps)  (model/layers.py:202-208)."""
    variance = x.pow(2).mean(dim=-1, keepdim=True)
    return weight * (x * torch.rsqrt(variance + eps))


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, factor: float, dtype) -> tuple[torch.Tensor, torch.Tensor]:  # noqa: E501
    """inv_freq = 1/theta^(2i/d); angles = (pos / factor) x inv_freq; emb = cat(f, f)  (model/layers.py:258-288)."""
    # The angles are float32 products, as in the reference's float32 tables; cos and sin of
    # those angles are then taken in the working precision.
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    inv_freq = (1.0 / (theta ** exponent)).to(positions.device)
    freqs = torch.outer(positions.to(torch.float32) / factor, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1).to(dtype)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """[x1, x2] -> [-x2, x1] over halves  (model/layers.py:214-222)."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x * cos + rotate_half(x) * sin, x: [T, heads, d]  (model/layers.py:298-302)."""
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None) -> torch.Tensor:
    """Causal (optionally windowed) grouped-query attention over a whole sequence.

    q: [T, nh, d], k, v: [T, nkv, d]. kv head j serves query heads j*g .. j*g+g-1
    (``repeat_interleave``, model/attention.py:198-199); scale = d^-0.5
    (model/model_config.py:224-227); key j visible to query i iff j <= i
    (model/attention.py:139-148) and, with a window, i - window < j.
    """
    t, nh, d = q.shape
    group = nh // k.shape[1]
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * (d ** -0.5)
    i = torch.arange(t, device=q.device)[:, None]
    j = torch.arange(t, device=q.device)[None, :]
    visible = j <= i
    if window is not None:
        visible = visible & (j > i - window)
    scores = scores.masked_fill(~visible[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hij,jhd->ihd", probs, v)


def activation(x: torch.Tensor, name: str) -> torch.Tensor:
    """model/layers.py:61-67."""
    if name == "silu":
        return x * torch.sigmoid(x)
    if name == "gelu":
        return torch.nn.functional.gelu(x)
    if name == "gelu_pytorch_tanh":
        return torch.nn.functional.gelu(x, approximate="tanh")
    raise ValueError(name)


def mlp(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, act: str) -> torch.Tensor:
    """down(act(gate x) * up x)  (model/layers.py:439-440)."""
    return (activation(x @ gate.T, act) * (x @ up.T)) @ down.T


def decoder_layer(h: torch.Tensor, w: dict[str, torch.Tensor], prefix: str, dims: dict, positions: torch.Tensor,
                  window: int | None) -> torch.Tensor:
    """Pre-norm block  (model/layers.py:469-487; projections :386-391)."""
    t = h.shape[0]
    nh, nkv, d = dims["nh"], dims["nkv"], dims["d"]
    x = rms_norm(h, w[prefix + "input_layernorm.weight"], dims["eps"])
    q = (x @ w[prefix + "self_attn.q_proj.weight"].T + w[prefix + "self_attn.q_proj.bias"]).view(t, nh, d)
    k = (x @ w[prefix + "self_attn.k_proj.weight"].T + w[prefix + "self_attn.k_proj.bias"]).view(t, nkv, d)
    v = (x @ w[prefix + "self_attn.v_proj.weight"].T + w[prefix + "self_attn.v_proj.bias"]).view(t, nkv, d)
    cos, sin = rope_cos_sin(positions, d, dims["theta"], dims["factor"], h.dtype)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    attended = attention(q, k, v, window).reshape(t, nh * d)
    h = h + attended @ w[prefix + "self_attn.o_proj.weight"].T
    x = rms_norm(h, w[prefix + "post_attention_layernorm.weight"], dims["eps"])
    return h + mlp(x, w[prefix + "mlp.gate_proj.weight"], w[prefix + "mlp.up_proj.weight"],
                   w[prefix + "mlp.down_proj.weight"], dims["act"])


class _Upcast:
    """Weights by name, upcast (and moved) one at a time when they are asked for."""

    def __init__(self, weights, dtype, device) -> None:
        self.weights, self.dtype, self.device = weights, dtype, device

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.weights[name].to(device=self.device, dtype=self.dtype)


def forward_logits(config: dict, weights: dict[str, torch.Tensor], token_ids, dtype=torch.float64, device="cpu") -> torch.Tensor:
    """Logits at every position of one whole sequence: [T, vocab]  (model/model.py:105-108,237-244).

    ``device`` only says where the same torch calls run (a model of real widths and depth takes
    minutes in float64 on a CPU); the result comes back on the CPU.
    """
    dims = derived(config)
    w = _Upcast(weights, dtype, device)
    ids = torch.as_tensor(token_ids, dtype=torch.long, device=device)
    positions = torch.arange(ids.numel(), device=device)
    h = embed(w["model.embed_tokens.weight"], ids)
    for layer in range(dims["L"]):
        h = decoder_layer(h, w, f"model.layers.{layer}.", dims, positions, layer_window(config, layer))
    h = rms_norm(h, w["model.norm.weight"], dims["eps"])
    head = w["model.embed_tokens.weight"] if dims["tie"] else w["lm_head.weight"]
    return (h @ head.T).cpu()


def greedy_generate(config: dict, weights: dict[str, torch.Tensor], prompt, num_tokens: int, dtype=torch.float64) -> list[int]:
    """Argmax continuation by recomputing the whole sequence for every token."""
    ids = list(prompt)
    out = []
    for _ in range(num_tokens):
        logits = forward_logits(config, weights, ids, dtype)
        nxt = int(torch.argmax(logits[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out


# -- sampling, plain ---------------------------------------------------------------------------------


def sample_uniforms(seed: int, counter: int, vocab: int) -> torch.Tensor:
    """The counter-based uniforms of the engine's sampler, restated with Python integers."""
    mask = (1 << 64) - 1
    out = []
    for index in range(vocab):
        x = ((seed * 0x9E3779B97F4A7C15) & mask) ^ ((counter << 32) | index)
        x ^= x >> 30
        x = (x * 0xBF58476D1CE4E5B9) & mask
        x ^= x >> 27
        x = (x * 0x94D049BB133111EB) & mask
        x ^= x >> 31
        out.append(((x >> 41) + 0.5) / 8388608.0)
    return torch.tensor(out, dtype=torch.float64)


def sample_token(logits: torch.Tensor, *, temperature: float, top_k: int = 0, top_p: float = 1.0,
                 repetition_penalty: float = 1.0, history=(), seed: int = 0, counter: int = 0) -> tuple[int, float]:
    """One row through the reference's stages (core/sampler.py:190-238), drawn by Gumbel-max.

    penalty (:83-122) -> logprobs of the penalised row (:222-223) -> temperature (:125-135) ->
    top-k keeps values >= the k-th largest (:138-148) -> top-p keeps a token iff the mass
    strictly ahead of it is <= p (:151-168) -> greedy argmax or a draw from the softmax.
    """
    row = logits.to(torch.float64).clone()
    if repetition_penalty != 1.0 and len(history):
        ids = torch.tensor(sorted(set(int(h) for h in history)), dtype=torch.long)
        picked = logits.to(torch.float64)[ids]
        row[ids] = torch.where(picked < 0, picked * repetition_penalty, picked / repetition_penalty)
    logprobs = torch.log_softmax(row, dim=-1)
    if temperature == 0.0:
        token = int(torch.argmax(row))
        return token, float(logprobs[token])
    row = row / temperature
    if 0 < top_k < row.numel():
        threshold = torch.topk(row, top_k).values[-1]
        row = row.masked_fill(row < threshold, float("-inf"))
    if top_p < 1.0:
        order = torch.argsort(row, descending=True, stable=True)
        probs = torch.softmax(row[order], dim=-1)
        before = probs.cumsum(-1) - probs
        remove = torch.zeros_like(row, dtype=torch.bool)
        remove[order] = before > top_p
        row = row.masked_fill(remove, float("-inf"))
    u = sample_uniforms(seed, counter, row.numel())
    gumbel = -torch.log(-torch.log(u))
    token = int(torch.argmax(row + gumbel))
    return token, float(logprobs[token])
