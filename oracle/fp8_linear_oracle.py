"""TEST INFRASTRUCTURE ONLY: what the FP8 linear layer behind the fused operator must compute, on the CPU.

The reference project has no FP8 linear layer (its column-parallel projection is ``F.linear`` on bf16,
``model/tensor_parallel.py:66``); what consumes the fused operator's FP8 output is defined by the quantisation the
operator applies (``gpuk/__init__.py:165-171``: ``norm_out = (n / scale).to(fp8)``), i.e. the dequantised product

    y[m, n] = sum_k x_fp8[m, k] * w_fp8[n, k] * x_scale[m] * w_scale[n].

Every e4m3 value and every product of two of them is exact in float64, so this restatement has no rounding of its own
before the final scaling; the kernel (fp32 accumulation, one rounding to bf16) must land within one bf16 step of it.
Only ``tests/`` may import this module.
"""
from __future__ import annotations

import torch


def fp8_linear_reference(x_fp8: torch.Tensor, x_scale: torch.Tensor, w_fp8: torch.Tensor, w_scale: torch.Tensor) -> torch.Tensor:
    """float64 [tokens, n]; ``x_scale`` holds one scale per token, ``w_scale`` one per output channel (any shapes)."""
    m, n = x_fp8.shape[0], w_fp8.shape[0]
    return (x_fp8.double() @ w_fp8.double().t()) * x_scale.double().reshape(m, 1) * w_scale.double().reshape(1, n)


def within_one_bf16_step(got: torch.Tensor, want: torch.Tensor) -> bool:
    """|got - want| <= 2^-7 |want| (one bf16 step at the value, with margin for the fp32 accumulation) plus a floor
    for values that cancel to almost nothing."""
    err = (got.double() - want).abs()
    tol = want.abs() * 2.0 ** -7 + want.abs().max() * 1e-6
    return bool(torch.isfinite(got.float()).all()) and bool((err <= tol).all())
