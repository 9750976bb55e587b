"""The tolerances of the engine-against-plain comparisons, fixed before the first run.

float32: every product and sum is fp32 where the plain implementation is float64; with
logits of order 1 the observed difference is below 1e-6, the bound is 5e-6 (absolute, on
logits whose largest magnitude is about 1 to 3).

bfloat16: weights are identical (stored in bfloat16), activations are rounded to bfloat16
between kernels (8 bits of mantissa, relative step 2^-8 = 0.0039) while statistics, softmax,
rotation and the residual stream are fp32. The bound on a logit is 0.02 x max(1, largest
|logit| of the request), and 0.004 on the mean absolute difference.

bfloat16 at depth: the bound above was fixed for models of two and three layers. Every layer
rounds its activations anew and independent roundings add in quadrature, so for a model of
more than three layers the bounds grow with the square root of the depth: x sqrt(layers / 3)
(``bf16_bounds``), 1.63 times at eight layers, 3.06 times at 28. The deep tests also evaluate
the plain implementation itself in bfloat16 (every product, norm and softmax rounded) and
print its distance from float64 beside the engine's; the engine, which keeps statistics and
the residual stream in fp32, has to be nearer than that.

float32 at the widths of the named models (inner sizes of 3,584 to 18,944 where the tiny models
have 64 to 576, eight and more layers): rounding grows with the square root of the inner size,
about eight times here, and with depth; the bound is 1e-4 on logits of the same magnitude,
twenty times the tiny models' bound, up to eight layers, and x sqrt(layers / 8) beyond
(``fp32_atol_real_widths``: 1.9e-4 at 28 layers). The tests print what they see beside it, and
what a float32 evaluation of the plain implementation itself loses.
"""

FP32_ATOL = 5e-6
FP32_ATOL_REAL_WIDTHS = 1e-4
BF16_REL_MAX = 0.02
BF16_MEAN = 0.004


def fp32_atol_real_widths(layers: int = 1) -> float:
    return FP32_ATOL_REAL_WIDTHS * max(1.0, (layers / 8.0) ** 0.5)


def bf16_bounds(layers: int = 1) -> tuple[float, float]:
    """(bound on the largest difference, bound on the mean difference), both relative to the scale."""
    growth = max(1.0, (layers / 3.0) ** 0.5)
    return BF16_REL_MAX * growth, BF16_MEAN * growth


def check_logits(ours, ref, dtype: str, what: str = "", fp32_atol: float = FP32_ATOL, layers: int = 1) -> None:
    import torch

    assert ours.shape == ref.shape, f"{what}: shape {tuple(ours.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(ours).all(), f"{what}: non-finite logits"
    diff = (ours.double() - ref.double()).abs()
    if dtype == "float32":
        worst = diff.max().item()
        where = divmod(int(diff.argmax()), diff.shape[1])
        assert worst <= fp32_atol, f"{what}: max |diff| {worst:.3e} at position {where[0]}, token {where[1]}"
    else:
        scale = max(1.0, ref.abs().max().item())
        worst = diff.max().item() / scale
        where = divmod(int(diff.argmax()), diff.shape[1])
        rel_max, rel_mean = bf16_bounds(layers)
        assert worst <= rel_max, f"{what}: max |diff| / scale {worst:.3e} at position {where[0]}, token {where[1]}"
        assert diff.mean().item() / scale <= rel_mean, f"{what}: mean |diff| / scale {diff.mean().item() / scale:.3e}"
