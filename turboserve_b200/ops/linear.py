"""The matrix product ``out = x @ weight.T``: which kernel runs for which dtype and shape.

The rule is explicit, measured on B200 (graph-timed, every weight read from HBM) and has no
fallback chain:

* float32: the FFMA kernel (``gemm_simt.cu``), always. No TF32, no tensor cores.
* bfloat16 with an inner size that is not a multiple of 8: the FFMA kernel (rows of such a
  matrix are not 16-byte aligned, which every tensor-core path needs).
* bfloat16, at most :data:`TC_MAX_ROWS` rows and at least :data:`TC_MIN_FEATURES` output
  features (the gate/up projection, the output head): the TMA + tcgen05 kernel
  (``gemm_tc.cu``): 6.0 to 6.8 TB/s, ahead of cuBLAS and of the register-streaming kernel.
* bfloat16, at most :data:`SKINNY_MAX_ROWS` rows, fewer output features, and few enough of them
  that all blocks of the register-streaming kernel (``gemm_skinny.cu``) are on the device at
  once (one block of eight warps per 16 features, two blocks a multiprocessor: up to 4,736
  features on 148): 7 to 8 µs on the 26 to 33 MB projections of a 3,584-wide model where a
  library call takes 9 to 11, 27 µs on its down projection where it takes 28. With more
  features its last blocks run nearly alone and the library wins (5,120 features: 16.1 against
  11.8 µs for 5,120 inputs, 37.9 against 26.6 µs for 13,824), so those go to the library.
* every other bfloat16 shape: cuBLAS through ``torch.mm``, as the reference does for every
  product (``src/turboserve/engine/model/layers.py:142``). Where the output is float32 (the
  output head) or a bias is to be added, the library writes its float32 accumulators and the
  bias is added to them, as in every other path here, so a row of logits does not depend on how
  many rows were asked for (the reference casts a bfloat16 result,
  ``src/turboserve/engine/model/model.py:243-244``).

:func:`gated_linear` is the gate/up projection with its activation: for at most
:data:`TC_MAX_ROWS` bfloat16 rows the tcgen05 kernel applies ``act(gate) * up`` in its epilogue,
else :func:`linear` is followed by the activation kernel.
"""

from __future__ import annotations

import torch

from . import kernels

SKINNY_MAX_ROWS = 8
TC_MAX_ROWS = 64
TC_MIN_FEATURES = 16384


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
           rows: int | None = None, ctx=None, early_trigger: bool = True) -> torch.Tensor:
    """``out[:rows] = x[:rows] @ weight.T (+ bias)``; ``bias`` is float32.

    ``ctx`` (a step context) lends scratch and the status word to kernels that want them.
    ``early_trigger=False`` asks a kernel of this package not to let the next kernel of the stream
    start ahead of its own end (for a next kernel that is slow to launch that way).
    """
    m = x.shape[0] if rows is None else rows
    if m == 0:
        return out
    n, k = weight.shape
    if x.dtype == torch.float32 or k % 8 != 0:
        kernels.gemm_simt(x, weight, out, bias, m)
        return out
    if m <= TC_MAX_ROWS and n >= TC_MIN_FEATURES:
        from . import tc

        tc.gemm_tc(x, weight, out, bias, m, slices=1, status=ctx.status if ctx is not None else None)
        return out
    if m <= SKINNY_MAX_ROWS:
        from . import skinny

        if -(-n // 16) <= 2 * skinny.num_sms(x.device):
            skinny.gemm_skinny(x, weight, out, bias, m, early_trigger=early_trigger)
            return out
    xs, os_ = x[:m], out[:m]
    if out.dtype == torch.bfloat16 and bias is None:
        torch.mm(xs, weight.t(), out=os_)
        return out
    wide = torch.mm(xs, weight.t(), out_dtype=torch.float32)
    if bias is not None:
        wide.add_(bias)
    os_.copy_(wide)
    return out


GATE_BLOCK = 64
"""Run length of the gate/up interleaving that :func:`interleave_gate_up` makes and :func:`gated_linear` reads."""


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> tuple[torch.Tensor, int]:
    """One ``[2 * I, ...]`` tensor for both projections (weights or biases) and its block length.

    When ``I`` is a multiple of :data:`GATE_BLOCK` the rows alternate in runs of that many (64
    gate features, then the 64 up features that go with them), so that one 128-row tile of the
    tcgen05 product holds what its fused activation needs; else gate rows come first, then up
    rows, and the block length is 0.
    """
    inter = gate.shape[0]
    if inter % GATE_BLOCK:
        return torch.cat([gate, up], dim=0).contiguous(), 0
    shape = (inter // GATE_BLOCK, GATE_BLOCK) + tuple(gate.shape[1:])
    both = torch.stack([gate.reshape(shape), up.reshape(shape)], dim=1)
    return both.reshape((2 * inter,) + tuple(gate.shape[1:])).contiguous(), GATE_BLOCK


def gated_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None, activation: str,
                 block: int, rows: int | None = None, ctx=None) -> torch.Tensor:
    """``out[:rows] = act(x gate^T) * (x up^T)`` for a ``weight`` made by :func:`interleave_gate_up`.

    bfloat16, at most :data:`TC_MAX_ROWS` rows and an interleaved weight: one tcgen05 kernel whose
    epilogue applies the activation (3.6 µs and a launch less per layer of a decode step; the
    result equals the two-kernel path bit for bit, since gate and up are rounded to bfloat16
    before the activation in both). Everything else: :func:`linear`, then the activation kernel.
    """
    m = x.shape[0] if rows is None else rows
    if m == 0:
        return out
    n, k = weight.shape
    if x.dtype == torch.bfloat16 and block == GATE_BLOCK and k % 8 == 0 and m <= TC_MAX_ROWS:
        from . import tc

        tc.gemm_tc_gated(x, weight, out, bias, activation, m, status=ctx.status if ctx is not None else None)
        return out
    both = ctx.buffer("mlp.gate_up", (x.shape[0], n)) if ctx is not None else torch.empty(x.shape[0], n, dtype=x.dtype, device=x.device)
    linear(x, weight, both, bias, m, ctx)
    kernels.act_mul(both, out, activation, m, block=block)
    return out
