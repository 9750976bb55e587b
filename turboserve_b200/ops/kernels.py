"""Python faces of the CUDA entry points: argument checks, pointers, the current stream.

Each function takes CUDA tensors, checks what the kernel assumes (device, dtype, contiguity of
the innermost dimension), passes raw pointers to the ``extern "C"`` symbol and raises
:class:`KernelError` when the entry point refuses or the launch fails. There is no fallback
to torch ops here: a missing extension is an error.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import load_library

TS_F32, TS_BF16 = 0, 1
_ERRORS = {
    -1: "dtype not supported by this kernel",
    -2: "a size this kernel does not take",
    -3: "a pointer or stride is not aligned as the kernel needs",
    -4: "an argument was refused",
}

ACTIVATION_CODES = {"silu": 0, "gelu": 1, "gelu_pytorch_tanh": 2}


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or its launch failed."""


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return TS_F32
    if dtype == torch.bfloat16:
        return TS_BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


_launches = 0


def launch_count() -> int:
    """How many kernels of this package have been launched so far in this process."""
    return _launches


def _check(code: int, name: str, launches: int = 1) -> None:
    """Raise for a refused call; else count the ``launches`` kernels the entry point started."""
    global _launches
    if code == 0:
        _launches += launches
        return
    if code in _ERRORS:
        raise KernelError(f"{name}: {_ERRORS[code]}")
    raise KernelError(f"{name}: CUDA error {code} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream of the current device as a raw handle (asked of torch's C layer directly where
    it offers that: ``torch.cuda.current_stream()`` costs several microseconds of Python per launch)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, dtype: torch.dtype | None, name: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if t.dim() and t.stride(-1) != 1:
        raise KernelError(f"{name} must be contiguous in its last dimension")


_functions: dict[str, ctypes._CFuncPtr] = {}


def _fn(lib: str, symbol: str, argtypes: list, restype=c_int):
    fn = _functions.get(symbol)
    if fn is None:
        fn = getattr(load_library(lib), symbol)
        fn.argtypes = argtypes
        fn.restype = restype
        _functions[symbol] = fn
    return fn


# ---------------------------------------------------------------------------------------
# layer_ops.cu
# ---------------------------------------------------------------------------------------


def embedding(ids: torch.Tensor, table: torch.Tensor, residual: torch.Tensor, status: torch.Tensor | None = None) -> None:
    """``residual[t] = float(table[ids[t]])``; ids int32 [T], residual fp32 [T, H]."""
    _need(ids, torch.int32, "ids"); _need(table, None, "table"); _need(residual, torch.float32, "residual")
    num_tokens, hidden = ids.numel(), table.shape[1]
    if residual.shape[-1] != hidden or residual.shape[0] < num_tokens or not residual.is_contiguous() or not table.is_contiguous():
        raise KernelError("embedding: residual must be contiguous [tokens, hidden]")
    fn = _fn("layer_ops", "ts_embedding", [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(dtype_code(table.dtype), _ptr(ids), _ptr(table), _ptr(residual), num_tokens, hidden, table.shape[0], _ptr(status), _stream()), "embedding")


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, gain: torch.Tensor, eps: float,
                out: torch.Tensor, rows: torch.Tensor | None = None, num_rows: int | None = None) -> None:
    """Fused ``residual += delta`` and RMSNorm into ``out`` (see ``layer_ops.cu``)."""
    _need(residual, torch.float32, "residual"); _need(gain, torch.float32, "gain"); _need(out, None, "out")
    hidden = residual.shape[-1]
    if delta is not None:
        _need(delta, out.dtype, "delta")
        if not delta.is_contiguous() or delta.shape[-1] != hidden:
            raise KernelError("add_rmsnorm: delta must be contiguous [rows, hidden]")
    if not residual.is_contiguous() or not out.is_contiguous() or out.shape[-1] != hidden or gain.numel() != hidden:
        raise KernelError("add_rmsnorm: shapes do not agree")
    if rows is not None:
        _need(rows, torch.int32, "rows")
        n = rows.numel() if num_rows is None else num_rows
    else:
        n = residual.shape[0] if num_rows is None else num_rows
    if out.shape[0] < n:
        raise KernelError("add_rmsnorm: out has too few rows")
    fn = _fn("layer_ops", "ts_add_rmsnorm", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p])
    _check(fn(dtype_code(out.dtype), _ptr(residual), _ptr(delta), _ptr(gain), _ptr(out), _ptr(rows), n, hidden, float(eps), _stream()), "add_rmsnorm")


def act_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str, num_tokens: int | None = None,
            block: int = 0) -> None:
    """``out[t, i] = act(gate[t, i]) * up[t, i]`` in fp32, rounded once.

    ``block == 0``: a row of ``gate_up`` is ``[gate | up]``. ``block > 0``: gate and up alternate
    in runs of ``block`` features (``[g 0..b-1 | u 0..b-1 | g b..2b-1 | ...]``).
    """
    _need(gate_up, None, "gate_up"); _need(out, gate_up.dtype, "out")
    inter = out.shape[-1]
    if gate_up.shape[-1] != 2 * inter or not gate_up.is_contiguous() or not out.is_contiguous():
        raise KernelError("act_mul: gate_up must be contiguous [tokens, 2 * intermediate]")
    if activation not in ACTIVATION_CODES:
        raise KernelError(f"act_mul: unknown activation {activation!r}")
    n = gate_up.shape[0] if num_tokens is None else num_tokens
    fn = _fn("layer_ops", "ts_act_mul", [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(out.dtype), _ptr(gate_up), _ptr(out), n, inter, ACTIVATION_CODES[activation], int(block),
              _stream()), "act_mul")


def rope_cache_write(qkv: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor, seq_of_token: torch.Tensor,
                     block_table: torch.Tensor, k_pages: torch.Tensor | None, v_pages: torch.Tensor | None,
                     num_tokens: int, num_heads: int, num_kv_heads: int, head_dim: int,
                     inv_freq: torch.Tensor | None, rotary_dim: int, factor: float, write_kv: bool,
                     status: torch.Tensor | None = None) -> None:
    """Bias, rotary encoding of q and k in fp32, and append of k, v to the paged cache."""
    _need(qkv, None, "qkv"); _need(positions, torch.int32, "positions"); _need(seq_of_token, torch.int32, "seq_of_token")
    _need(block_table, torch.int32, "block_table")
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.dim() != 2 or qkv.shape[1] < width:
        raise KernelError("rope_cache_write: qkv is narrower than its heads")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != width:
            raise KernelError("rope_cache_write: bias length does not match the projected heads")
    page_size = 1
    if write_kv:
        if k_pages is None or v_pages is None:
            raise KernelError("rope_cache_write: pages are needed to write keys and values")
        _need(k_pages, qkv.dtype, "k_pages"); _need(v_pages, qkv.dtype, "v_pages")
        if not k_pages.is_contiguous() or not v_pages.is_contiguous() or tuple(k_pages.shape[2:]) != (num_kv_heads, head_dim):
            raise KernelError("rope_cache_write: pages must be contiguous [pages, page_size, kv_heads, head_dim]")
        page_size = k_pages.shape[1]
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq")
        if inv_freq.numel() * 2 != rotary_dim:
            raise KernelError("rope_cache_write: inv_freq must hold rotary_dim / 2 values")
    fn = _fn("layer_ops", "ts_rope_cache_write",
             [c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
              c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(fn(dtype_code(qkv.dtype), _ptr(qkv), qkv.stride(0), _ptr(bias), _ptr(positions), _ptr(seq_of_token),
              _ptr(block_table), block_table.stride(0), _ptr(k_pages), _ptr(v_pages), page_size, num_tokens,
              num_heads, num_kv_heads, head_dim, _ptr(inv_freq), rotary_dim, float(factor), int(write_kv),
              _ptr(status), _stream()), "rope_cache_write")


# ---------------------------------------------------------------------------------------
# attention_generic.cu
# ---------------------------------------------------------------------------------------


def paged_attention_generic(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                            block_table: torch.Tensor, seq_of_token: torch.Tensor, positions: torch.Tensor,
                            num_tokens: int, num_heads: int, num_kv_heads: int, head_dim: int,
                            window: int | None, scale: float, status: torch.Tensor | None = None) -> None:
    """Attention of every token over its sequence's pages; any dtype and head size <= 256.

    ``q`` is ``[tokens, >= num_heads * head_dim]`` (it may be the fused qkv buffer), ``out``
    ``[tokens, num_heads * head_dim]``.
    """
    _need(q, None, "q"); _need(out, q.dtype, "out"); _need(k_pages, q.dtype, "k_pages"); _need(v_pages, q.dtype, "v_pages")
    _need(block_table, torch.int32, "block_table"); _need(seq_of_token, torch.int32, "seq_of_token"); _need(positions, torch.int32, "positions")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or tuple(k_pages.shape[2:]) != (num_kv_heads, head_dim):
        raise KernelError("paged_attention: pages must be contiguous [pages, page_size, kv_heads, head_dim]")
    if q.shape[1] < num_heads * head_dim or out.shape[1] < num_heads * head_dim:
        raise KernelError("paged_attention: q or out is narrower than its heads")
    fn = _fn("attention_generic", "ts_paged_attention_generic",
             [c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(fn(dtype_code(q.dtype), _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages),
              _ptr(block_table), block_table.stride(0), _ptr(seq_of_token), _ptr(positions), num_tokens,
              k_pages.shape[1], num_heads, num_kv_heads, head_dim, int(window or 0), float(scale), _ptr(status),
              _stream()), "paged_attention_generic")


# ---------------------------------------------------------------------------------------
# gemm_simt.cu
# ---------------------------------------------------------------------------------------


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None, m: int | None = None) -> None:
    """``out[:m] = a[:m] @ w.T (+ bias)`` with fp32 FFMA accumulation; any sizes."""
    _need(a, None, "a"); _need(w, a.dtype, "w"); _need(out, None, "out")
    if a.dim() != 2 or w.dim() != 2 or out.dim() != 2 or a.shape[1] != w.shape[1] or out.shape[1] != w.shape[0]:
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    rows = a.shape[0] if m is None else m
    if out.shape[0] < rows or a.shape[0] < rows:
        raise KernelError("gemm: fewer rows than asked for")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != w.shape[0]:
            raise KernelError("gemm: bias length does not match the output width")
    fn = _fn("gemm_simt", "ts_gemm_simt",
             [c_int, c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(a.dtype), dtype_code(out.dtype), _ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out),
              out.stride(0), rows, w.shape[0], a.shape[1], _stream()), "gemm_simt")


# ---------------------------------------------------------------------------------------
# sampling.cu
# ---------------------------------------------------------------------------------------


def argmax(logits: torch.Tensor, tokens: torch.Tensor, num_rows: int | None = None) -> None:
    _need(logits, torch.float32, "logits"); _need(tokens, torch.int32, "tokens")
    n = logits.shape[0] if num_rows is None else num_rows
    fn = _fn("sampling", "ts_argmax", [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), n, logits.shape[1], _ptr(tokens), _stream()), "argmax")


def sample(logits: torch.Tensor, work: torch.Tensor, tokens: torch.Tensor, *, num_rows: int | None = None,
           temperature: torch.Tensor | None = None, top_k: torch.Tensor | None = None, top_p: torch.Tensor | None = None,
           penalty: torch.Tensor | None = None, seed: torch.Tensor | None = None, counter: torch.Tensor | None = None,
           history: torch.Tensor | None = None, history_start: torch.Tensor | None = None,
           logprobs: torch.Tensor | None = None) -> None:
    """One token per row of fp32 ``logits``; per-row option arrays, ``None`` switches a stage off.

    ``work`` is fp32 scratch of at least ``[rows, vocab]``; ``seed`` is int64 (read as
    unsigned), ``counter`` int32 (the index of the token being generated).
    """
    _need(logits, torch.float32, "logits"); _need(work, torch.float32, "work"); _need(tokens, torch.int32, "tokens")
    n = logits.shape[0] if num_rows is None else num_rows
    vocab = logits.shape[1]
    if work.numel() < n * vocab or not work.is_contiguous():
        raise KernelError("sample: work must hold rows * vocab floats")
    for name, tensor, dtype in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                                ("top_p", top_p, torch.float32), ("penalty", penalty, torch.float32),
                                ("seed", seed, torch.int64), ("counter", counter, torch.int32),
                                ("history", history, torch.int32), ("history_start", history_start, torch.int32),
                                ("logprobs", logprobs, torch.float32)):
        if tensor is not None:
            _need(tensor, dtype, name)
    fn = _fn("sampling", "ts_sample", [c_void_p, c_longlong, c_void_p, c_int, c_int] + [c_void_p] * 11)
    _check(fn(_ptr(logits), logits.stride(0), _ptr(work), n, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p),
              _ptr(penalty), _ptr(seed), _ptr(counter), _ptr(history), _ptr(history_start), _ptr(tokens),
              _ptr(logprobs), _stream()), "sample")


def sample_slots(logits: torch.Tensor, work: torch.Tensor, tokens: torch.Tensor, num_rows: int, *, temperature: torch.Tensor,
                 top_k: torch.Tensor, top_p: torch.Tensor, seed: torch.Tensor, prompt_len: torch.Tensor,
                 seq_slot: torch.Tensor, seq_context: torch.Tensor, partial: torch.Tensor, chunks: int,
                 row_token: torch.Tensor | None = None, seq_of_token: torch.Tensor | None = None,
                 step_tokens: torch.Tensor | None = None, penalty: torch.Tensor | None = None,
                 seen: torch.Tensor | None = None, want_logprob: torch.Tensor | None = None,
                 logprobs: torch.Tensor | None = None) -> None:
    """One token per row with the options looked up by state slot (arrays over the slots).

    A row finds its request through a step's own index arrays: ``row_token`` (per row: the step's
    token whose logits the row holds; without it the row itself), ``seq_of_token`` (per token: its
    request in the step, negative for padding, whose row is skipped; without it the token itself),
    ``seq_slot`` and ``seq_context`` (per request: its state slot and its length after the step).
    The index of the token being generated is ``seq_context - prompt_len[slot]``. ``partial`` is
    zeroed int32 scratch of ``rows * (4 * chunks + 1)`` words; a row that needs one pass only
    (greedy, or a draw without top-k and top-p) is cut into ``chunks`` blocks.

    ``penalty`` (per slot) goes with ``seen`` (int32 ``[slots, ceil(vocab / 32)]``: the bitmap of the
    tokens each slot's request holds); ``step_tokens`` (per token of the step: its id) lets a row
    add the token its logits come from to that bitmap first. ``want_logprob`` (per slot, int32)
    goes with ``logprobs`` (float32 per row): the log-probability of the chosen token under the
    penalised row."""
    _need(logits, torch.float32, "logits"); _need(work, torch.float32, "work"); _need(tokens, torch.int32, "tokens")
    vocab = logits.shape[1]
    if work.numel() < num_rows * vocab or not work.is_contiguous():
        raise KernelError("sample_slots: work must hold rows * vocab floats")
    for name, tensor, dtype in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                                ("top_p", top_p, torch.float32), ("seed", seed, torch.int64), ("prompt_len", prompt_len, torch.int32),
                                ("seq_slot", seq_slot, torch.int32), ("seq_context", seq_context, torch.int32),
                                ("partial", partial, torch.int32)):
        _need(tensor, dtype, name)
    for name, tensor, dtype in (("row_token", row_token, torch.int32), ("seq_of_token", seq_of_token, torch.int32),
                                ("penalty", penalty, torch.float32), ("seen", seen, torch.int32),
                                ("step_tokens", step_tokens, torch.int32), ("want_logprob", want_logprob, torch.int32),
                                ("logprobs", logprobs, torch.float32)):
        if tensor is not None:
            _need(tensor, dtype, name)
    if partial.numel() < num_rows * (4 * chunks + 1):
        raise KernelError("sample_slots: partial is too small")
    if row_token is not None and row_token.numel() < num_rows:
        raise KernelError("sample_slots: row_token has fewer entries than rows")
    seen_words = 0
    if penalty is not None:
        if seen is None or seen.dim() != 2 or not seen.is_contiguous() or seen.shape[1] * 32 < vocab or seen.shape[0] < penalty.numel():
            raise KernelError("sample_slots: a penalty needs seen [slots, ceil(vocab / 32)]")
        seen_words = seen.shape[1]
    if (want_logprob is None) != (logprobs is None) or (logprobs is not None and logprobs.numel() < num_rows):
        raise KernelError("sample_slots: want_logprob and logprobs (one per row) go together")
    fn = _fn("sampling", "ts_sample_slots", [c_void_p, c_longlong, c_void_p, c_int, c_int] + [c_void_p] * 12 + [c_int] +
             [c_void_p] * 3 + [c_int] + [c_void_p] * 2)
    _check(fn(_ptr(logits), logits.stride(0), _ptr(work), num_rows, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p),
              _ptr(seed), _ptr(prompt_len), _ptr(row_token), _ptr(seq_of_token), _ptr(seq_slot), _ptr(seq_context),
              _ptr(step_tokens), _ptr(tokens), _ptr(partial), int(chunks), _ptr(penalty), _ptr(want_logprob),
              _ptr(seen if penalty is not None else None), seen_words, _ptr(logprobs), _stream()),
           "sample_slots", launches=2)  # the one-pass kernel, then the cluster kernel for rows with filters


def mark_seen(token_ids: torch.Tensor, seq_of_token: torch.Tensor, state_slots: torch.Tensor, penalty: torch.Tensor,
              seen: torch.Tensor, num_tokens: int, vocab: int) -> None:
    """Set, in ``seen`` (int32 ``[slots, ceil(vocab / 32)]``), the bit of every token of the step whose
    request's slot has a penalty other than 1 (``penalty`` per slot)."""
    for name, tensor, dtype in (("token_ids", token_ids, torch.int32), ("seq_of_token", seq_of_token, torch.int32),
                                ("state_slots", state_slots, torch.int32), ("penalty", penalty, torch.float32),
                                ("seen", seen, torch.int32)):
        _need(tensor, dtype, name)
    if token_ids.numel() < num_tokens or seq_of_token.numel() < num_tokens:
        raise KernelError("mark_seen: fewer tokens than asked for")
    if seen.dim() != 2 or not seen.is_contiguous() or seen.shape[1] * 32 < vocab or seen.shape[0] < penalty.numel():
        raise KernelError("mark_seen: seen must be [slots, ceil(vocab / 32)]")
    fn = _fn("sampling", "ts_mark_seen", [c_void_p] * 5 + [c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(token_ids), _ptr(seq_of_token), _ptr(state_slots), _ptr(penalty), _ptr(seen), seen.shape[1], num_tokens,
              vocab, _stream()), "mark_seen")


def sample_uniform_host(seed: int, counter: int, index: int) -> float:
    fn = _fn("sampling", "ts_sample_uniform_host", [ctypes.c_ulonglong, ctypes.c_uint, ctypes.c_uint], restype=c_float)
    return float(fn(seed & 0xFFFFFFFFFFFFFFFF, counter, index))
