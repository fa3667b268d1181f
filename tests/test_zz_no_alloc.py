"""The no-allocation self-check entry point against the workspace-based emulation.

gpuk_selfcheck_allreduce_rms runs the N-rank fused exchange on one GPU with staging memory
that is compiled into the library, for callers that must not allocate device memory (a health
probe inside a server whose arena owns the GPU).  Its results must be the bits that
gpuk_emulated_allreduce_rms produces with allocated workspaces, call after call -- the built-in
array is shared by all calls and carries the protocol's call counter from one to the next.

Collected last on purpose: a failure here cannot hide another test's result in a run that
stops at the first failure.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from gpuk_b200 import cabi                # noqa: E402
from oracle import epilogue_oracle as eo  # noqa: E402
from tests import util                    # noqa: E402


def _selfcheck(parts, residual, weight, eps, quant, static_scale, mode, check_free=True):
    world = len(parts)
    outs = [util.alloc_outputs(p, quant, static_scale) for p in parts]
    arr = lambda ts: (ctypes.c_void_p * world)(*[t.data_ptr() for t in ts])
    torch.cuda.synchronize()
    # free bytes as the driver counts them: a cudaMalloc inside the library cannot hide from this
    # (torch.cuda.memory_allocated() only sees PyTorch's own caching allocator)
    free_before = torch.cuda.mem_get_info()[0]
    before = torch.cuda.memory_allocated()
    cabi.check(cabi.lib.gpuk_selfcheck_allreduce_rms(
        world, arr(parts), util.ptr(residual), util.ptr(weight), arr([o[0] for o in outs]), arr([o[1] for o in outs]),
        arr([o[2] for o in outs]), parts[0].numel(), parts[0].shape[-1], cabi.dtype_code(parts[0].dtype), eps, quant,
        mode, util.stream_ptr()))
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    if check_free:
        assert torch.cuda.mem_get_info()[0] == free_before
    st = (ctypes.c_uint32 * 8)()
    assert cabi.lib.gpuk_selfcheck_status(st, util.stream_ptr()) == cabi.OK, (list(st), cabi.last_error())
    return [(o[0].cpu(), o[1].cpu(), o[2].cpu() if quant else None) for o in outs]


@pytest.mark.parametrize("world,tokens,hidden,quant,mode", [
    (2, 4, 4096, 3, 1), (2, 4, 4096, 3, 2), (8, 2, 8192, 4, 1), (8, 2, 8192, 3, 2), (4, 16, 1024, 1, 2), (4, 13, 1024, 0, 1),
])
def test_matches_workspace_based_entry_point_twice_in_a_row(world, tokens, hidden, quant, mode):
    static = 0.05 if quant == 4 else None
    with util.EmulatedGroup(world, max_bytes=1 << 20) as g:
        for call in range(2):
            parts, res, w = util.random_case(world, tokens, hidden, torch.bfloat16, seed=world * 13 + tokens + call)
            d_parts, d_res, d_w = [p.cuda() for p in parts], res.cuda(), w.cuda()
            want = g.fused(d_parts, d_res, d_w, 1e-6, quant, static, force_mode=mode)
            # the first launch of a kernel loads its code onto the device (lazy module loading), which
            # the driver's free-byte count shows: the count is compared from the second call on
            got = _selfcheck(d_parts, d_res, d_w, 1e-6, quant, static, mode, check_free=call > 0)
            oracle = eo.epilogue_t1(parts, res, w, 1e-6, quant, static)
            for r in range(world):
                # same kernels, same summation order: identical bits, well inside the parity bars
                assert torch.equal(got[r][0].view(torch.uint8), want[r][0].view(torch.uint8)), (call, r)
                assert torch.equal(got[r][1].view(torch.uint8), want[r][1].view(torch.uint8)), (call, r)
                if quant:
                    assert torch.equal(got[r][2], want[r][2]), (call, r)
                util.check_against_oracle(got[r], oracle, quant)


def test_world_size_changes_between_calls():
    """All emulated ranks share ONE call counter (its low bit selects the staging buffer): after a
    two-rank call, ranks 2..7 must not be one call behind ranks 0 and 1.  World 2, then 4, then 8,
    and back, in both exchange modes, each against the workspace-based entry point."""
    seq = [(2, 1), (4, 1), (8, 1), (2, 2), (8, 2), (4, 2), (8, 1), (2, 1), (4, 2)]
    for i, (world, mode) in enumerate(seq):
        parts, res, w = util.random_case(world, 3, 2048, torch.bfloat16, seed=500 + i)
        d_parts, d_res, d_w = [p.cuda() for p in parts], res.cuda(), w.cuda()
        with util.EmulatedGroup(world, max_bytes=1 << 20) as g:
            want = g.fused(d_parts, d_res, d_w, 1e-6, 3, force_mode=mode)
        got = _selfcheck(d_parts, d_res, d_w, 1e-6, 3, None, mode, check_free=False)
        for r in range(world):
            assert torch.equal(got[r][0].view(torch.uint8), want[r][0].view(torch.uint8)), (i, r)
            assert torch.equal(got[r][1].view(torch.uint8), want[r][1].view(torch.uint8)), (i, r)
            assert torch.equal(got[r][2], want[r][2]), (i, r)


def test_status_reads_ok_when_no_call_gave_up():
    st = (ctypes.c_uint32 * 8)()
    assert cabi.lib.gpuk_selfcheck_status(st, util.stream_ptr()) == cabi.OK
    assert list(st) == [0] * 8


def test_refuses_messages_beyond_the_built_in_scratch():
    parts, res, w = util.random_case(2, 8, 4096, torch.bfloat16, seed=1)       # 64 KiB per rank > 32 KiB
    d_parts, d_res, d_w = [p.cuda() for p in parts], res.cuda(), w.cuda()
    with pytest.raises(cabi.GpukError) as e:
        _selfcheck(d_parts, d_res, d_w, 1e-6, 3, None, 0)
    assert e.value.status == cabi.ERR_TOO_LARGE and "32768" in str(e.value)
