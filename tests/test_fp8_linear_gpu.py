"""The FP8 linear layer that consumes the fused operator's output (gpuk_fp8_linear_skinny, through the C ABI)
against a float64 product of the dequantised operands, and against torch._scaled_mm on the same inputs."""
import ctypes

import pytest
import torch

from gpuk_b200 import cabi
from oracle import fp8_linear_oracle as fo

E4M3 = torch.float8_e4m3fn


def _case(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(m, k, generator=g) * 100).clamp_(-448, 448).to(E4M3)
    w = (torch.randn(n, k, generator=g) * 100).clamp_(-448, 448).to(E4M3)
    xs = torch.rand(m, 1, generator=g) * 0.02 + 1e-3
    ws = torch.rand(1, n, generator=g) * 0.02 + 1e-3
    return x, xs, w, ws


def _want(x, xs, w, ws):
    return fo.fp8_linear_reference(x, xs, w, ws)


def _run(x, xs, w, ws, k_split=0, packed=False, frags=0):
    cabi.check(cabi.lib.gpuk_set_tuning(b"fp8_frags_per_warp", frags))
    try:
        return _run_with_current_tuning(x, xs, w, ws, k_split, packed)
    finally:
        cabi.check(cabi.lib.gpuk_set_tuning(b"fp8_frags_per_warp", 0))


def _run_with_current_tuning(x, xs, w, ws, k_split, packed):
    m, k = x.shape
    n = w.shape[0]
    dx, dxs, dw, dws = x.cuda(), xs.cuda().contiguous(), w.cuda(), ws.cuda().contiguous()
    if packed:
        blocked = torch.empty_like(dw)
        cabi.check(cabi.lib.gpuk_fp8_pack_weight(ctypes.c_void_p(dw.data_ptr()), ctypes.c_void_p(blocked.data_ptr()), n, k,
                                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        want = dw.view(torch.uint8).view(n // 16, 16, k // 64, 64).permute(0, 2, 1, 3).contiguous().view(n, k)
        assert torch.equal(blocked.view(torch.uint8), want)
        dw = blocked
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    rc = cabi.lib.gpuk_fp8_linear_skinny(ctypes.c_void_p(dx.data_ptr()), ctypes.c_void_p(dxs.data_ptr()), ctypes.c_void_p(dw.data_ptr()),
                                         ctypes.c_void_p(dws.data_ptr()), ctypes.c_void_p(out.data_ptr()), m, n, k, 1 if packed else 0, k_split,
                                         ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    cabi.check(rc)
    torch.cuda.synchronize()
    cabi.check(cabi.lib.gpuk_fp8_linear_status())
    return out.cpu()


def _close(got, want):
    """fp32 accumulation of exact FP8 products, one rounding to bf16: within one bf16 step (2^-8 relative) of the
    float64 result, plus the accumulation error of k terms (far below that)."""
    assert fo.within_one_bf16_step(got, want), (float((got.double() - want).abs().max()), float(want.abs().max()))


def test_oracle_on_known_answers():
    """The float64 restatement on values small enough to check by hand, and its tolerance helper."""
    x = torch.tensor([[1.0, 2.0, -0.5, 0.0] * 16]).to(E4M3)              # one token, k = 64
    w = torch.tensor([[2.0, 1.0, 4.0, 448.0] * 16, [0.5] * 64]).to(E4M3)
    y = fo.fp8_linear_reference(x, torch.tensor([[0.5]]), w, torch.tensor([[2.0, 4.0]]))
    assert y.tolist() == [[16 * (2.0 + 2.0 - 2.0) * 0.5 * 2.0, 16 * (0.5 + 1.0 - 0.25) * 0.5 * 4.0]]
    assert fo.within_one_bf16_step(y.to(torch.bfloat16), y)
    assert not fo.within_one_bf16_step((y * 1.02).to(torch.bfloat16), y)


@pytest.mark.gpu
@pytest.mark.parametrize("frags", [1, 2])
@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("k_split", [0, 1, 2, 4, 8])
@pytest.mark.parametrize("m,n,k", [(32, 128, 64), (1, 256, 8192), (8, 1280, 8192), (17, 7168, 1024), (32, 1024, 3584), (31, 384, 4160)])
def test_matches_float64_product(m, n, k, k_split, packed, frags):
    """Token counts that leave groups of 8 partly or wholly empty, k that does not divide over the cluster
    (3584 / 64 = 56 steps over 8 parts, 4160 / 64 = 65), one k step only, every cluster size, both weight layouts
    (the blocked one is also compared with the same rearrangement done by PyTorch), one and two fragments per warp."""
    x, xs, w, ws = _case(m, n, k, seed=m * 7 + n + k)
    _close(_run(x, xs, w, ws, k_split, packed, frags), _want(x, xs, w, ws))


@pytest.mark.gpu
def test_reproducible_and_close_to_the_library_gemm():
    m, n, k = 32, 7168, 8192       # w1|w3 of the decoder benchmark on one of eight ranks
    x, xs, w, ws = _case(m, n, k, seed=3)
    a = _run(x, xs, w, ws)
    b = _run(x, xs, w, ws)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))      # fixed summation order
    assert torch.equal(a.view(torch.int16), _run(x, xs, w, ws, packed=True).view(torch.int16))      # ... whatever the weight layout
    assert torch.equal(a.view(torch.int16), _run(x, xs, w, ws, frags=1).view(torch.int16))          # ... and the warps' share
    lib = torch._scaled_mm(x.cuda(), w.cuda().t(), scale_a=xs.cuda(), scale_b=ws.cuda(), out_dtype=torch.bfloat16).cpu()
    _close(lib, _want(x, xs, w, ws))
    # both are within a bf16 step of the float64 product (the library accumulates less exactly): mostly the same bits
    assert float((a.view(torch.int16) == lib.view(torch.int16)).float().mean()) > 0.9


@pytest.mark.gpu
def test_consumes_the_fused_operators_output():
    """norm_out and scale_out of the one-GPU fused operator go straight into the linear layer."""
    from tests import util
    tokens, hidden, n = 24, 4096, 512
    parts, res, wnorm = util.random_case(1, tokens, hidden, torch.bfloat16, seed=5)
    _, q, s = util.k1(parts[0].cuda(), res.cuda(), wnorm.cuda(), 1e-6, 3)
    g = torch.Generator().manual_seed(6)
    w = torch.randn(n, hidden, generator=g).clamp_(-3, 3)
    wsc = w.abs().amax(dim=1, keepdim=True) / 448.0
    wq = (w / wsc).to(E4M3)
    got = _run(q, s, wq, wsc.t().contiguous())
    _close(got, _want(q, s, wq, wsc.t()))


def test_shapes_outside_the_kernels_range_are_refused_before_any_cuda_call():
    null = ctypes.c_void_p(16)
    f = cabi.lib.gpuk_fp8_linear_skinny
    assert f(null, null, null, null, null, 33, 128, 64, 0, 0, None) == cabi.ERR_UNSUPPORTED and "32" in cabi.last_error()
    assert f(null, null, null, null, null, 8, 100, 64, 0, 0, None) == cabi.ERR_UNSUPPORTED
    assert f(null, null, null, null, null, 8, 128, 96, 0, 0, None) == cabi.ERR_UNSUPPORTED
    assert f(null, null, null, null, null, 8, 128, 64, 0, 3, None) == cabi.ERR_INVALID_ARGUMENT
    assert f(null, null, null, null, null, 8, 128, 64, 2, 0, None) == cabi.ERR_INVALID_ARGUMENT
    assert f(None, null, null, null, null, 8, 128, 64, 0, 0, None) == cabi.ERR_INVALID_ARGUMENT
    assert f(null, null, null, null, null, 0, 128, 64, 0, 0, None) == cabi.OK          # no tokens: nothing to do
    assert cabi.lib.gpuk_fp8_pack_weight(null, ctypes.c_void_p(32), 24, 64, None) == cabi.ERR_UNSUPPORTED
    assert cabi.lib.gpuk_fp8_pack_weight(null, null, 16, 64, None) == cabi.ERR_INVALID_ARGUMENT      # in place


def test_python_wrapper_refuses_what_the_kernel_cannot_take():
    """gpuk_b200.fp8_linear on the host side: shapes it is built for, and operands it must refuse before any launch."""
    import gpuk_b200 as gpuk
    assert gpuk.fp8_linear_supported(32, 7168, 8192) and gpuk.fp8_linear_supported(1, 128, 64)
    assert not gpuk.fp8_linear_supported(33, 7168, 8192) and not gpuk.fp8_linear_supported(0, 128, 64)
    assert not gpuk.fp8_linear_supported(8, 100, 64) and not gpuk.fp8_linear_supported(8, 128, 96)
    x = torch.zeros(8, 64).to(E4M3)
    w = torch.zeros(128, 64).to(E4M3)
    with pytest.raises(RuntimeError, match="CUDA"):
        gpuk.fp8_linear(x, torch.ones(8, 1), w, torch.ones(1, 128))            # host tensors
    with pytest.raises(RuntimeError, match="float8_e4m3fn"):
        gpuk.fp8_linear(x.float(), torch.ones(8, 1), w, torch.ones(1, 128))
    with pytest.raises(RuntimeError, match="CUDA"):
        gpuk.fp8_pack_weight(w)
