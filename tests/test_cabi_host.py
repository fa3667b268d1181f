"""CPU-side checks of the boundary: the C-ABI library loads and exports what the header
declares, argument validation happens before any CUDA call, and the launch policy is sane."""
import ctypes
import os
import re

import pytest

from gpuk_b200 import cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "gpuk_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gpuk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared()
    assert len(names) >= 25
    for n in names:
        assert hasattr(cabi.lib, n), n
    assert set(names) == set(cabi._SIGNATURES), set(names) ^ set(cabi._SIGNATURES)


def test_header_cites_the_reference_for_each_entry_point():
    text = open(os.path.join(ROOT, "include", "gpuk_b200.h")).read()
    for needle in ("src/register.cpp", "all_reduce_fusion.cpp", "communicator.h", "all_reduce_fusion_impl.h"):
        assert needle in text


def test_argument_validation_precedes_cuda():
    """Same failures as init_ar_fusion (src/ops/all_reduce_fusion.cpp:256-266), as status codes."""
    h = ctypes.c_void_p()
    for world in (0, 1, 3, 5, 16):
        assert cabi.lib.gpuk_ws_create(0, 0, world, 1 << 20, 0, ctypes.byref(h)) == cabi.ERR_INVALID_ARGUMENT
        assert "world size is not supported" in cabi.last_error()
    assert cabi.lib.gpuk_ws_create(0, 2, 2, 1 << 20, 0, ctypes.byref(h)) == cabi.ERR_INVALID_ARGUMENT
    assert "invalid rank" in cabi.last_error()
    assert cabi.lib.gpuk_ws_create(0, -1, 2, 1 << 20, 0, ctypes.byref(h)) == cabi.ERR_INVALID_ARGUMENT
    assert cabi.lib.gpuk_ws_create(0, 0, 2, 0, 0, ctypes.byref(h)) == cabi.ERR_INVALID_ARGUMENT
    assert cabi.lib.gpuk_ws_destroy(None) == cabi.OK
    assert cabi.lib.gpuk_ws_status(None, None) == cabi.ERR_INVALID_ARGUMENT
    assert cabi.lib.gpuk_allreduce_inplace(None, None, 16, 0, None) == cabi.ERR_INVALID_ARGUMENT
    assert cabi.lib.gpuk_status_string(cabi.ERR_PEER_TIMEOUT).decode().startswith("timed out")


def test_plan_benchmark_configs():
    sms = 148
    c2 = cabi.plan(8, 8 * 8192, 8192, sm_count=sms)
    # eight rows are spread over the GPU: each row is held by a cluster of eight CTAs
    assert c2.one_shot == 1 and c2.rows == 8 and c2.row_vecs == 1024 and c2.cluster == 8 and c2.grid == 64
    assert c2.vpt * c2.threads * c2.cluster >= c2.row_vecs and c2.threads == 128
    c3 = cabi.plan(8, 1024 * 8192, 8192, sm_count=sms)
    assert c3.one_shot == 0 and c3.message_bytes == 16 << 20
    assert c3.grid * c3.rows_per_chunk <= 1024 and c3.grid <= 2048 and c3.cluster == 1
    assert c3.lead_push >= 1 and c3.lead_reduce >= 1
    c4 = cabi.plan(8, 16384 * 7168, 7168, sm_count=sms)
    assert c4.one_shot == 0 and c4.row_vecs == 896 and c4.vpt * c4.threads >= 896 and c4.threads % 32 == 0
    c5 = cabi.plan(8, 32 * 8192, 8192, sm_count=sms)
    assert c5.message_bytes == 512 << 10
    one_gpu = cabi.plan(1, 16384 * 7168, 7168, sm_count=sms)
    assert one_gpu.one_shot == 0 and one_gpu.grid <= sms * 8


@pytest.mark.parametrize("world", [2, 4, 8])
def test_plan_crossover_moves_with_the_threshold(world):
    numel = 64 * 4096
    lo = cabi.plan(world, numel, 4096, oneshot_max_bytes=1024)
    hi = cabi.plan(world, numel, 4096, oneshot_max_bytes=1 << 21)
    assert lo.one_shot == 0 and hi.one_shot == 1


def test_plan_rejects_bad_shapes():
    p = cabi.Plan()
    f = cabi.lib.gpuk_plan_allreduce_rms
    assert f(8, 4 * 1020, 1020, cabi.DTYPE_BF16, 148, 0, 0, ctypes.byref(p)) == cabi.ERR_UNSUPPORTED
    assert f(8, 4 * 1024 + 8, 1024, cabi.DTYPE_BF16, 148, 0, 0, ctypes.byref(p)) == cabi.ERR_INVALID_ARGUMENT
    assert f(3, 4 * 1024, 1024, cabi.DTYPE_BF16, 148, 0, 0, ctypes.byref(p)) == cabi.ERR_INVALID_ARGUMENT
    assert f(8, 4 * 1024, 1024, 7, 148, 0, 0, ctypes.byref(p)) == cabi.ERR_UNSUPPORTED
    assert f(8, 2 * 65536, 65536, cabi.DTYPE_BF16, 148, 0, 0, ctypes.byref(p)) == cabi.ERR_UNSUPPORTED
    assert f(8, 1027, 0, cabi.DTYPE_BF16, 148, 0, 0, ctypes.byref(p)) == cabi.ERR_UNSUPPORTED


def test_plan_tiles_cover_every_legal_row():
    for hidden in range(8, 32768 + 1, 8 * 37):
        p = cabi.plan(8, 4 * hidden, hidden)
        assert p.vpt in (1, 2, 4, 8) and p.threads % 32 == 0 and p.threads <= (512 if p.vpt >= 4 else 1024)
        assert p.cluster in (1, 2, 4, 8) and p.grid % p.cluster == 0
        assert p.vpt * p.threads * p.cluster >= p.row_vecs == hidden // 8


@pytest.mark.parametrize("world", [2, 4, 8])
def test_plan_tiles_respect_the_kernels_launch_bounds(world):
    """The kernels are compiled for at most 256 threads per CTA in the two-shot exchange (512 for the
    8-vector tile) and 1024 / 256 / 512 in the one-shot exchange (kernels.cuh: ar_max_threads); a plan
    beyond that would fail at launch.  Also: the grid is whole clusters, a cluster covers its row."""
    for hidden in list(range(8, 4096, 8 * 7)) + list(range(4096, 32768 + 1, 8 * 61)) + [1024, 2048, 4096, 7168, 8192, 16384, 32768]:
        for tokens in (1, 7, 8, 32, 64, 148, 149, 300, 1024, 5000):
            for crossover in (1, 1 << 40):
                p = cabi.plan(world, tokens * hidden, hidden, oneshot_max_bytes=crossover)
                limit = (512 if p.vpt == 8 else 256) if not p.one_shot else {1: 1024, 2: 1024, 4: 256, 8: 512}[p.vpt]
                assert 32 <= p.threads <= limit and p.threads % 32 == 0, (hidden, tokens, crossover, p.threads, p.vpt)
                assert p.cluster in (1, 2, 4, 8) and p.grid % p.cluster == 0 and p.grid >= p.cluster
                seg = -(-p.row_vecs // p.cluster)
                assert p.vpt * p.threads >= seg and seg * p.cluster >= p.row_vecs
                assert p.grid // p.cluster <= -(-p.rows // p.rows_per_chunk)
                assert p.lead_push >= 1 and p.lead_reduce >= 1


def test_attach_symmetric_validates_before_touching_cuda():
    assert cabi.lib.gpuk_ws_attach_symmetric(None, None, 2, None, 1 << 20) == cabi.ERR_INVALID_ARGUMENT


def test_tuning_names_and_ranges():
    """gpuk_set_tuning: process-wide knobs of the entry points that have no workspace; pure host state."""
    assert cabi.lib.gpuk_set_tuning(b"fp8_frags_per_warp", 2) == cabi.OK
    assert cabi.lib.gpuk_set_tuning(b"fp8_frags_per_warp", 3) == cabi.ERR_INVALID_ARGUMENT
    assert cabi.lib.gpuk_set_tuning(b"fp8_frags_per_warp", 0) == cabi.OK
    assert cabi.lib.gpuk_set_tuning(b"k1_stages", 9) == cabi.ERR_INVALID_ARGUMENT
    assert cabi.lib.gpuk_set_tuning(b"no_such_knob", 1) == cabi.ERR_INVALID_ARGUMENT and "no_such_knob" in cabi.last_error()
    assert cabi.lib.gpuk_set_tuning(None, 1) == cabi.ERR_INVALID_ARGUMENT
