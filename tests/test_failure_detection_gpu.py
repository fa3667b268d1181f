"""Failure detection without a GPU fault: a device-side wait for a peer that never answers
runs out after its budget, records where, and returns; the context stays usable."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

from gpuk_b200 import cabi   # noqa: E402
from tests import util       # noqa: E402


def test_wait_runs_out_and_reports():
    with util.EmulatedGroup(2) as g:
        ws = g.ws[1]
        cabi.check(cabi.lib.gpuk_ws_set_timeout_ns(ws, 50_000_000))      # 50 ms
        t0 = time.time()
        cabi.check(cabi.lib.gpuk_ws_selftest_wait(ws, util.stream_ptr()))
        rc, st = g.status(1)
        elapsed = time.time() - t0
        assert rc == cabi.ERR_PEER_TIMEOUT
        assert st[0] == 1 and st[1] == 1 and st[3] == 3, st               # timed out, on rank 1, in the self-test stage
        assert "gave up waiting" in cabi.last_error()
        assert 0.04 < elapsed < 5.0
        # the context is alive: clear the latch and run a real exchange on the same workspaces
        for h in g.ws:
            cabi.check(cabi.lib.gpuk_ws_clear_status(h))
        parts, res, w = util.random_case(2, 4, 1024, torch.bfloat16, seed=2)
        outs = g.fused([p.cuda() for p in parts], res.cuda(), w.cuda(), 1e-6, 3)
        assert outs[0][1].shape == (4, 1024)


def test_call_before_peers_are_opened_is_refused():
    h = ctypes.c_void_p()
    cabi.check(cabi.lib.gpuk_ws_create(0, 0, 2, 1 << 20, 0, ctypes.byref(h)))
    x = torch.zeros(4, 1024, dtype=torch.bfloat16, device="cuda")
    rc = cabi.lib.gpuk_allreduce_inplace(h, util.ptr(x), x.numel(), 0, util.stream_ptr())
    assert rc == cabi.ERR_NOT_READY
    cabi.lib.gpuk_ws_destroy(h)


def test_corrupt_ipc_handle_is_an_error_not_a_crash():
    h = ctypes.c_void_p()
    cabi.check(cabi.lib.gpuk_ws_create(0, 0, 2, 1 << 20, 0, ctypes.byref(h)))
    junk = (ctypes.c_uint8 * 128)(*([0xAB] * 128))
    rc = cabi.lib.gpuk_ws_open_data_handles(h, junk, 2)
    assert rc == cabi.ERR_CUDA
    rc = cabi.lib.gpuk_ws_open_data_handles(h, junk, 3)
    assert rc == cabi.ERR_INVALID_ARGUMENT
    cabi.lib.gpuk_ws_destroy(h)
    torch.zeros(1, device="cuda").sum().item()      # context still answers
