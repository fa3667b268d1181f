"""CPU restatement of the reference's tensor-parallel epilogue (test oracle).

TEST INFRASTRUCTURE ONLY.  The product path (``gpuk_b200``) never imports this module.

What is restated, with the reference lines each function follows:

* ``allreduce_t1``       fp32 sum over ranks in rank order, one rounding to the input dtype.
                         This is what the reference's fused kernels compute for the sum
                         (``src/impl/all_reduce_fusion_impl.h:70-83, 242-255, 311-324``) and
                         what its C++ tests use as the CPU answer
                         (``test/cpp/test_all_reduce.cpp:565-587``).
* ``add_rms_quant``      everything after the collective in
                         ``GPUKDistEnv.allreduce_add_rms_native`` (``gpuk/__init__.py:147-173``):
                         residual add in the input dtype, RMSNorm with the same dtype
                         rounding points (``rms_norm_forward``, ``:150-155``; identical to
                         ``model/transformer_model.py:464-475``), per-token amax/max scale,
                         division, clamp, cast to FP8 (``:159-164``).
* ``epilogue_t1``        ``allreduce_t1`` followed by ``add_rms_quant``.
* quantisation policies  ``quant_type`` 0/1/2 carry the reference's meaning
                         (``src/impl/all_reduce_fusion_impl.h:13-17``; saturation values
                         ``src/common/float8.h:216-218, 249-251`` = 240 and 120).  3 and 4
                         are additive: e4m3fn with the OCP maximum 448, dynamic per token (3)
                         or with one caller-supplied static scale for the whole tensor (4).

One deliberate deviation from the native Python path, taken from the reference's fused
kernel instead: a row whose amax is zero gets scale 1 (``all_reduce_fusion_impl.h:217,221``)
rather than 0 (which would turn the row into NaNs).

Parity status: pinned.  ``tests/test_oracle.py`` checks this module bit-for-bit against
golden vectors produced by the reference's own ``allreduce_add_rms_native`` run over gloo
(``tests/golden/make_golden.py``) and checks the FP8 cast against the reference's software
conversion compiled from ``src/common/float8.h``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch

QUANT_NONE = 0
QUANT_FP8_E4M3FN_240 = 1      # reference policy 1: dynamic per token, saturates at 240
QUANT_FP8_E4M3FNUZ_120 = 2    # reference policy 2: dynamic per token, fnuz flavour, 120
QUANT_FP8_E4M3FN_448 = 3      # additive: dynamic per token, OCP e4m3fn maximum
QUANT_FP8_E4M3FN_448_STATIC = 4  # additive: one static scale for the whole tensor


@dataclass(frozen=True)
class QuantPolicy:
    quant_type: int
    fp8_dtype: Optional[torch.dtype]
    fp8_max: float
    static: bool


POLICIES = {
    QUANT_NONE: QuantPolicy(0, None, 0.0, False),
    QUANT_FP8_E4M3FN_240: QuantPolicy(1, torch.float8_e4m3fn, 240.0, False),
    QUANT_FP8_E4M3FNUZ_120: QuantPolicy(2, torch.float8_e4m3fnuz, 120.0, False),
    QUANT_FP8_E4M3FN_448: QuantPolicy(3, torch.float8_e4m3fn, 448.0, False),
    QUANT_FP8_E4M3FN_448_STATIC: QuantPolicy(4, torch.float8_e4m3fn, 448.0, True),
}


def allreduce_t1(parts: Sequence[torch.Tensor]) -> torch.Tensor:
    """Sum of the per-rank partials: fp32 accumulate in rank order, one rounding.

    Follows ``test/cpp/test_all_reduce.cpp:565-587`` (``allreduce_ref``).
    """
    acc = parts[0].float().clone()
    for p in parts[1:]:
        acc += p.float()
    return acc.to(parts[0].dtype)


def rms_norm_forward(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``gpuk/__init__.py:150-155``: fp32 variance, one rounding after ``* rstd``, one after ``* w``."""
    input_dtype = x.dtype
    variance = x.float().pow(2).mean(-1, keepdim=True)
    x = x * torch.rsqrt(variance + eps)
    x = x.to(input_dtype)
    return weight * x


def add_rms_quant(
    allreduce_out: torch.Tensor,
    residual_in: torch.Tensor,
    rms_weight: torch.Tensor,
    eps: float,
    quant_type: int = QUANT_NONE,
    static_scale: Optional[float] = None,
) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Everything after the collective in ``gpuk/__init__.py:157-173``.

    Returns ``(residual_out, norm_out, scale)``; ``scale`` is ``[M, 1]`` fp32 for the dynamic
    policies, a one-element fp32 tensor for the static policy and ``None`` without
    quantisation.
    """
    pol = POLICIES[quant_type]
    residual_out = allreduce_out + residual_in
    norm_out = rms_norm_forward(residual_out, rms_weight, eps)
    if pol.fp8_dtype is None:
        return residual_out, norm_out, None
    if pol.static:
        if static_scale is None:
            raise ValueError("static policy needs static_scale")
        scale = torch.tensor([static_scale], dtype=torch.float32)
        q = norm_out.float() / scale
    else:
        scale, _ = norm_out.float().abs().max(dim=-1, keepdim=True)
        scale = scale / pol.fp8_max
        # all_reduce_fusion_impl.h:217 -- an all-zero row keeps scale 1
        scale = torch.where(scale == 0, torch.ones_like(scale), scale)
        q = norm_out / scale          # bf16 / fp32 -> fp32, as in gpuk/__init__.py:161
    q = q.float().clamp_(min=-pol.fp8_max, max=pol.fp8_max)
    return residual_out, q.to(pol.fp8_dtype), scale


def epilogue_t1(
    parts: Sequence[torch.Tensor],
    residual_in: torch.Tensor,
    rms_weight: torch.Tensor,
    eps: float,
    quant_type: int = QUANT_NONE,
    static_scale: Optional[float] = None,
):
    """T1 oracle: fp32-accumulated all-reduce, then the PyTorch operator sequence."""
    return add_rms_quant(allreduce_t1(parts), residual_in, rms_weight, eps, quant_type, static_scale)


# ----------------------------------------------------------------------------------------
# comparison helpers
# ----------------------------------------------------------------------------------------

def fp8_code_index(codes_u8: torch.Tensor, fnuz: bool = False) -> torch.Tensor:
    """Map FP8 bit patterns to a signed integer that is monotone in the encoded value.

    Neighbouring representable values differ by exactly 1, so the absolute difference of
    two indices is the distance in units in the last place.  ``+0`` and ``-0`` both map
    to 0.  NaN codes map to a large sentinel.
    """
    c = codes_u8.to(torch.int32)
    mag = c & 0x7F
    idx = torch.where(c >= 0x80, -mag, mag)
    if fnuz:
        nan = c == 0x80
    else:
        nan = mag == 0x7F
    return torch.where(nan, torch.full_like(idx, 1 << 20), idx)


def fp8_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Element-wise distance in e4m3 ulps between two FP8 tensors of the same flavour."""
    fnuz = a.dtype == torch.float8_e4m3fnuz
    ia = fp8_code_index(a.view(torch.uint8), fnuz)
    ib = fp8_code_index(b.view(torch.uint8), fnuz)
    return (ia - ib).abs()


@dataclass
class ParityReport:
    residual_mismatch_frac: float
    residual_max_abs: float
    norm_max_abs: float
    fp8_exact_frac: float
    fp8_within_1ulp_frac: float
    scale_max_rel: float
    scale_rows: int = 0
    scale_rows_beyond_1e3: int = 0

    def check(self, *, fp8_frac=0.999, scale_rel=1e-3, scale_step=2.0 ** -7) -> None:
        """FP8 codes within one step on >= fp8_frac of the elements; scales within scale_rel.

        The row maximum is a 16-bit value: when the two sides' fp32 row statistics differ in the
        last bit, that value can round to the neighbouring 16-bit number on one side, which moves
        the scale by one 16-bit step (2^-8 .. 2^-7 relative); the multiplication by the weight
        rounds once more and can carry that to a second step.  Such a row is tolerated only as an
        outlier: at most one row, or 0.1 % of the rows, and never by more than two steps.
        """
        assert self.fp8_within_1ulp_frac >= fp8_frac, self
        assert self.scale_max_rel <= 2 * scale_step, self
        assert self.scale_rows_beyond_1e3 <= max(1, self.scale_rows // 1000), self
        if self.scale_rows_beyond_1e3 == 0:
            assert self.scale_max_rel <= scale_rel, self


def compare(got, want, *, atol=2e-2, rtol=2e-2) -> ParityReport:
    """Compare ``(residual_out, norm_out, scale)`` triples; raises on a bf16 allclose miss."""
    g_res, g_norm, g_scale = got
    w_res, w_norm, w_scale = want
    torch.testing.assert_close(g_res.float(), w_res.float(), atol=atol, rtol=rtol)
    res_mis = (g_res.float() != w_res.float()).float().mean().item()
    res_abs = (g_res.float() - w_res.float()).abs().max().item() if g_res.numel() else 0.0
    if w_scale is None:
        torch.testing.assert_close(g_norm.float(), w_norm.float(), atol=atol, rtol=rtol)
        nabs = (g_norm.float() - w_norm.float()).abs().max().item() if g_norm.numel() else 0.0
        return ParityReport(res_mis, res_abs, nabs, 1.0, 1.0, 0.0)
    d = fp8_ulp_distance(g_norm, w_norm)
    n = max(d.numel(), 1)
    exact = (d == 0).sum().item() / n if d.numel() else 1.0
    near = (d <= 1).sum().item() / n if d.numel() else 1.0
    srel = ((g_scale.float().reshape(-1) - w_scale.float().reshape(-1)).abs()
            / w_scale.float().reshape(-1).abs().clamp_min(1e-30))
    beyond = int((srel > 1e-3).sum().item()) if srel.numel() else 0
    rows = srel.numel()
    srel = srel.max().item() if srel.numel() else 0.0
    return ParityReport(res_mis, res_abs, 0.0, exact, near, srel, rows, beyond)
