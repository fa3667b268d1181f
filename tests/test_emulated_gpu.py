"""The N-rank kernels on ONE GPU: all ranks of a group run inside one cooperative launch
(gpuk_emulated_allreduce_rms), so the exchange logic, the self-announcing staging protocol and the fused
epilogue are checked against the T1 oracle without needing N GPUs."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import epilogue_oracle as eo   # noqa: E402
from gpuk_b200 import workloads as oin           # noqa: E402
from tests import util                     # noqa: E402

ONE_SHOT, TWO_SHOT, SYMMETRIC = 1, 2, 3


def _check_all_ranks(outs, want, quant):
    for r, got in enumerate(outs):
        util.check_against_oracle(got, want, quant)
        # every rank must hold the same bits (same summation order everywhere)
        assert torch.equal(got[0].view(torch.uint8), outs[0][0].view(torch.uint8)), r
        assert torch.equal(got[1].view(torch.uint8), outs[0][1].view(torch.uint8)), r


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mode", [ONE_SHOT, TWO_SHOT])
@pytest.mark.parametrize("tokens,hidden,quant", [
    (1, 4096, 3), (8, 8192, 4), (129, 1024, 1), (128, 1024, 2), (37, 7168, 3), (16, 2048, 0), (5, 2056, 3),
])
def test_fused_bf16(world, mode, tokens, hidden, quant):
    parts, res, w = util.random_case(world, tokens, hidden, torch.bfloat16, seed=world * 1000 + tokens + hidden)
    static = 0.05 if quant == 4 else None
    with util.EmulatedGroup(world) as g:
        outs = g.fused([p.cuda() for p in parts], res.cuda(), w.cuda(), 1e-6, quant, static, force_mode=mode)
    want = eo.epilogue_t1(parts, res, w, 1e-6, quant, static)
    _check_all_ranks(outs, want, quant)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("mode", [ONE_SHOT, TWO_SHOT])
def test_fused_other_dtypes(dtype, mode):
    """fp32 and fp16 at 129 x 1024, as in test/test_all_reduce_fusion.py:177-204."""
    for world in (2, 8):
        parts, res, w = util.random_case(world, 129, 1024, dtype, seed=world + 77)
        with util.EmulatedGroup(world) as g:
            outs = g.fused([p.cuda() for p in parts], res.cuda(), w.cuda(), 1e-6, 3, force_mode=mode)
        want = eo.epilogue_t1(parts, res, w, 1e-6, 3)
        for got in outs:
            # fp32 has no rounding points to pin the sum, so the residual is compared by tolerance
            util.check_against_oracle(got, want, 3, exact_residual=dtype != torch.float32)


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("lead_push,lead_reduce", [(0, 0), (2, 3), (100000, 100000)])
def test_two_shot_many_chunks_per_cta(world, lead_push, lead_reduce):
    """More rows than resident CTAs: every CTA pipelines several chunks (scatter s, reduce
    s - lead_push, epilogue s - lead_push - lead_reduce), the regime of the prefill benchmark;
    0 keeps the default depths, the huge value runs the three stages strictly one after another."""
    parts, res, w = util.random_case(world, 1500, 1024, torch.bfloat16, seed=5 + world)
    with util.EmulatedGroup(world, max_bytes=4 << 20) as g:
        g.set_option("two_shot_ws", 0)      # the pipeline depths belong to the kernel without specialised warps
        g.set_option("lead_push", lead_push)
        g.set_option("lead_reduce", lead_reduce)
        outs = g.fused([p.cuda() for p in parts], res.cuda(), w.cuda(), 1e-6, 3, force_mode=TWO_SHOT)
    want = eo.epilogue_t1(parts, res, w, 1e-6, 3)
    _check_all_ranks(outs, want, 3)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("rows_per_chunk", [1, 3, 0])
@pytest.mark.parametrize("tokens,hidden,quant", [(1, 4096, 3), (129, 1024, 1), (700, 2048, 3), (37, 7168, 4), (1500, 1024, 0)])
def test_two_shot_rows_per_chunk_and_repeated_calls(world, rows_per_chunk, tokens, hidden, quant):
    """The two-shot kernel whose CTAs walk scatter / reduce / finish in lock step, with chunks of one
    and of three rows (the last chunk ragged), and (rows_per_chunk 0) whatever kernel the policy
    picks -- the warp-specialised one where no cluster shares a row; twice on the same workspace."""
    parts, res, w = util.random_case(world, tokens, hidden, torch.bfloat16, seed=world * 7 + tokens)
    static = 0.05 if quant == 4 else None
    with util.EmulatedGroup(world, max_bytes=4 << 20) as g:
        g.set_option("two_shot_ws", 0 if rows_per_chunk else 1)
        g.set_option("rows_per_chunk", rows_per_chunk)
        for _ in range(2):      # twice: the call counter and the staging parity must advance consistently
            outs = g.fused([p.cuda() for p in parts], res.cuda(), w.cuda(), 1e-6, quant, static, force_mode=TWO_SHOT)
    want = eo.epilogue_t1(parts, res, w, 1e-6, quant, static)
    _check_all_ranks(outs, want, quant)


def test_plain_allreduce_with_three_rows_per_chunk():
    g0 = torch.Generator().manual_seed(11)
    parts = [torch.randn(300 * 1024 + 64, generator=g0).to(torch.bfloat16) for _ in range(4)]
    want = eo.allreduce_t1(parts)
    with util.EmulatedGroup(4) as g:
        g.set_option("two_shot_ws", 0)
        g.set_option("rows_per_chunk", 3)
        outs = g.plain([p.cuda() for p in parts], force_mode=TWO_SHOT)
    for got in outs:
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_back_to_back_calls_mixed_shapes_and_modes():
    """One workspace, a sequence of calls that changes shape and exchange mode: exercises the
    call counter, the double-buffered staging and its reuse."""
    world = 4
    seq = [(8, 2048, ONE_SHOT), (8, 2048, ONE_SHOT), (8, 2048, ONE_SHOT), (300, 1024, TWO_SHOT), (8, 2048, ONE_SHOT),
           (64, 4096, TWO_SHOT), (64, 4096, TWO_SHOT), (3, 1024, ONE_SHOT), (700, 1024, TWO_SHOT), (1, 8192, ONE_SHOT)]
    with util.EmulatedGroup(world, max_bytes=4 << 20) as g:
        for i, (tokens, hidden, mode) in enumerate(seq):
            parts, res, w = util.random_case(world, tokens, hidden, torch.bfloat16, seed=100 + i)
            outs = g.fused([p.cuda() for p in parts], res.cuda(), w.cuda(), 1e-6, 3, force_mode=mode)
            want = eo.epilogue_t1(parts, res, w, 1e-6, 3)
            _check_all_ranks(outs, want, 3)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mode", [ONE_SHOT, TWO_SHOT])
@pytest.mark.parametrize("numel", [8, 4096, 8 * 1024 + 8, 300 * 1024 + 64])
def test_plain_allreduce(world, mode, numel):
    """allreduce_inplace: fp32 accumulation in rank order, one rounding
    (test/cpp/test_all_reduce.cpp:565-587), including a ragged last row."""
    g0 = torch.Generator().manual_seed(numel + world)
    parts = [torch.randn(numel, generator=g0).to(torch.bfloat16) for _ in range(world)]
    want = eo.allreduce_t1(parts)
    with util.EmulatedGroup(world) as g:
        outs = g.plain([p.cuda() for p in parts], force_mode=mode)
    for got in outs:
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_plain_allreduce_f32():
    g0 = torch.Generator().manual_seed(1)
    parts = [torch.randn(5000, generator=g0) for _ in range(4)]
    want = eo.allreduce_t1(parts)
    with util.EmulatedGroup(4) as g:
        outs = g.plain([p.cuda() for p in parts], force_mode=TWO_SHOT)
    for got in outs:
        torch.testing.assert_close(got, want, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("tokens,hidden,quant", [(1, 8192, 3), (3, 2056, 3), (20, 4096, 4), (40, 8192, 1), (70, 7168, 0)])
def test_one_shot_rows_split_over_a_cluster(world, tokens, hidden, quant):
    """Few rows: each row is exchanged and normalised by a thread-block cluster (the two row-wide
    reductions cross CTAs); called twice so that the staging double buffer and the call counter
    advance, and with a ragged split (2056 / 8 = 257 vectors over two CTAs)."""
    from gpuk_b200 import cabi
    plan = cabi.plan(world, tokens * hidden, hidden, oneshot_max_bytes=2 << 20)
    assert plan.one_shot == 1 and plan.cluster > 1
    static = 0.05 if quant == 4 else None
    with util.EmulatedGroup(world) as g:
        for call in range(2):
            parts, res, w = util.random_case(world, tokens, hidden, torch.bfloat16, seed=world * 31 + tokens + call)
            outs = g.fused([p.cuda() for p in parts], res.cuda(), w.cuda(), 1e-6, quant, static, force_mode=ONE_SHOT)
            want = eo.epilogue_t1(parts, res, w, 1e-6, quant, static)
            _check_all_ranks(outs, want, quant)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("tokens,hidden,quant,rows_per_chunk", [
    (1, 4096, 3, 0), (129, 1024, 1, 0), (700, 2048, 3, 3), (37, 7168, 4, 0), (1500, 1024, 0, 2), (5, 2056, 3, 0)])
def test_exchange_through_symmetric_memory(world, tokens, hidden, quant, rows_per_chunk):
    """Copy-in, flag, slice reduction from every rank's buffer, broadcast, flag, epilogue -- here
    with peer loads standing in for the switch reduction; three calls in a row on the same buffers
    (no double buffering: the flags alone keep consecutive calls apart)."""
    static = 0.05 if quant == 4 else None
    with util.EmulatedGroup(world, max_bytes=4 << 20) as g:
        g.attach_symmetric(tokens * hidden * 2)
        if rows_per_chunk:
            g.set_option("rows_per_chunk", rows_per_chunk)
        for call in range(3):
            parts, res, w = util.random_case(world, tokens, hidden, torch.bfloat16, seed=world * 17 + tokens + call)
            outs = g.fused([p.cuda() for p in parts], res.cuda(), w.cuda(), 1e-6, quant, static, force_mode=SYMMETRIC)
            want = eo.epilogue_t1(parts, res, w, 1e-6, quant, static)
            _check_all_ranks(outs, want, quant)


def test_symmetric_exchange_interleaved_with_the_push_exchange_and_refused_without_a_buffer():
    from gpuk_b200 import cabi
    world = 4
    parts, res, w = util.random_case(world, 300, 2048, torch.bfloat16, seed=77)
    d = [p.cuda() for p in parts], res.cuda(), w.cuda()
    want = eo.epilogue_t1(parts, res, w, 1e-6, 3)
    with util.EmulatedGroup(world, max_bytes=4 << 20) as g:
        with pytest.raises(cabi.GpukError) as e:
            g.fused(*d, 1e-6, 3, force_mode=SYMMETRIC)
        assert e.value.status == cabi.ERR_NOT_READY
        g.attach_symmetric(300 * 2048 * 2)
        for mode in (SYMMETRIC, TWO_SHOT, SYMMETRIC, ONE_SHOT, SYMMETRIC):
            _check_all_ranks(g.fused(*d, 1e-6, 3, force_mode=mode), want, 3)
        # automatic choice by message size
        g.set_option("sym_min_bytes", 1 << 20)
        _check_all_ranks(g.fused(*d, 1e-6, 3), want, 3)
        big, res2, w2 = util.random_case(world, 301, 2048, torch.bfloat16, seed=78)
        with pytest.raises(cabi.GpukError) as e:
            g.fused([p.cuda() for p in big], res2.cuda(), w2.cuda(), 1e-6, 3, force_mode=SYMMETRIC)
        assert e.value.status == cabi.ERR_TOO_LARGE


@pytest.mark.parametrize("mode,tokens,hidden", [(ONE_SHOT, 16, 4096), (TWO_SHOT, 16, 4096), (ONE_SHOT, 8, 8192)])
def test_launch_without_the_planned_cluster_is_reported_and_writes_nothing(mode, tokens, hidden):
    """A row is split over a thread-block cluster; if the launch runs without its cluster
    attribute, every CTA would see itself as CTA 0 of a cluster of one and finish only the first
    segment of each row.  The kernels compare the cluster they run in with the planned one and
    report status 3 before they store anything: outputs keep their fill, the workspace says so,
    and after gpuk_ws_clear_status the same workspaces exchange correctly."""
    from gpuk_b200 import cabi
    world = 2
    plan = cabi.plan(world, tokens * hidden, hidden, oneshot_max_bytes=(2 << 20) if mode == ONE_SHOT else 1)
    assert plan.cluster > 1
    parts, res, w = util.random_case(world, tokens, hidden, torch.bfloat16, seed=tokens + hidden)
    d_parts, d_res, d_w = [p.cuda() for p in parts], res.cuda(), w.cuda()
    with util.EmulatedGroup(world) as g:
        outs = [util.alloc_outputs(p, 3) for p in d_parts]
        for o in outs:
            o[0].fill_(7.0)
            o[1].view(torch.uint8).fill_(0x55)
        g.set_option("test_withhold_cluster", 1)
        g.fused(d_parts, d_res, d_w, 1e-6, 3, force_mode=mode, outs=outs, check_status=False)
        for r in range(world):
            rc, st = g.status(r)
            assert rc == cabi.ERR_BAD_LAUNCH, (rc, st)
            assert st[0] == 3 and st[1] == r and st[6] == 1, st          # code, rank, cluster size seen
            assert "cluster" in cabi.last_error()
            assert torch.all(outs[r][0] == 7.0) and torch.all(outs[r][1].view(torch.uint8) == 0x55)
            assert torch.all(outs[r][2] == -1.0)
        g.set_option("test_withhold_cluster", 0)
        g.clear_status()
        got = g.fused(d_parts, d_res, d_w, 1e-6, 3, force_mode=mode)
    _check_all_ranks(got, eo.epilogue_t1(parts, res, w, 1e-6, 3), 3)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("tokens,hidden,quant,dtype", [
    (300, 8192, 3, torch.bfloat16), (301, 7168, 3, torch.bfloat16), (160, 16384, 1, torch.bfloat16), (150, 32768, 3, torch.bfloat16),
    (999, 136, 4, torch.bfloat16), (333, 2056, 0, torch.bfloat16), (200, 4096, 2, torch.float16), (180, 1000, 3, torch.float32)])
def test_two_shot_with_specialised_warps(world, tokens, hidden, quant, dtype):
    """The kernel of the bandwidth regime: one CTA per SM whose warps scatter, reduce and finish rows
    independently.  Tiles of 1, 2, 4 and 8 vectors per finishing thread, rows that fill their tile and
    rows that do not, slices that do not divide the row (2056 / 8 = 257 vectors over 2, 4, 8 ranks), all
    element types and policies; three calls in a row so both staging buffers are reused."""
    from gpuk_b200 import cabi
    plan = cabi.plan(world, tokens * hidden, hidden, dtype=cabi.dtype_code(dtype), oneshot_max_bytes=1)
    assert plan.ws == 1 and plan.ws_tf + plan.ws_tr + plan.ws_ts <= 768 and plan.ws_vpt * plan.ws_tf >= plan.row_vecs
    static = 0.05 if quant == 4 else None
    with util.EmulatedGroup(world, max_bytes=16 << 20) as g:
        for call in range(3):
            parts, res, w = util.random_case(world, tokens, hidden, dtype, seed=world * 11 + tokens + call)
            outs = g.fused([p.cuda() for p in parts], res.cuda(), w.cuda(), 1e-6, quant, static, force_mode=TWO_SHOT)
            want = eo.epilogue_t1(parts, res, w, 1e-6, quant, static)
            for got in outs:
                util.check_against_oracle(got, want, quant, exact_residual=dtype != torch.float32)
                assert torch.equal(got[1].view(torch.uint8), outs[0][1].view(torch.uint8))


@pytest.mark.parametrize("tokens,hidden,quant,dtype", [
    (300, 8192, 3, torch.bfloat16), (1500, 1024, 1, torch.bfloat16), (301, 7168, 4, torch.bfloat16), (333, 2056, 0, torch.bfloat16),
    (160, 16384, 3, torch.bfloat16), (200, 4096, 2, torch.float16), (180, 1000, 3, torch.float32)])
def test_two_ranks_one_hop_and_two_hops_agree(tokens, hidden, quant, dtype):
    """At two ranks the kernel with specialised warps sends whole rows to the peer and every rank adds its own row
    while finishing (one hop); the option two_rank_one_hop = 0 keeps reduce-scatter + all-gather (two hops).  Both
    must give the oracle's result and each other's bits, call after call on one workspace, in either order."""
    static = 0.05 if quant == 4 else None
    with util.EmulatedGroup(2, max_bytes=16 << 20) as g:
        for call, one_hop in enumerate([1, 0, 0, 1, 1]):
            g.set_option("two_rank_one_hop", one_hop)
            parts, res, w = util.random_case(2, tokens, hidden, dtype, seed=tokens + call // 2)
            outs = g.fused([p.cuda() for p in parts], res.cuda(), w.cuda(), 1e-6, quant, static, force_mode=TWO_SHOT)
            want = eo.epilogue_t1(parts, res, w, 1e-6, quant, static)
            for got in outs:
                util.check_against_oracle(got, want, quant, exact_residual=dtype != torch.float32)
                assert torch.equal(got[1].view(torch.uint8), outs[0][1].view(torch.uint8))
            if call % 2 == 1:      # same inputs as the call before, the other exchange
                for a, b in zip(outs, prev):
                    assert torch.equal(a[0].view(torch.uint8), b[0].view(torch.uint8))
                    assert torch.equal(a[1].view(torch.uint8), b[1].view(torch.uint8))
            prev = outs


def test_two_ranks_output_over_the_input_takes_two_hops():
    """residual_out may be the input buffer itself.  The one-hop exchange reads the input while it finishes rows, so
    the call must notice the overlap and take the two-hop exchange, which never reads a row after finishing it."""
    tokens, hidden = 400, 4096
    parts, res, w = util.random_case(2, tokens, hidden, torch.bfloat16, seed=21)
    want = eo.epilogue_t1(parts, res, w, 1e-6, 3)
    with util.EmulatedGroup(2, max_bytes=8 << 20) as g:
        d_parts = [p.cuda() for p in parts]
        outs = [util.alloc_outputs(p, 3) for p in d_parts]
        outs = [(d_parts[r], o[1], o[2]) for r, o in enumerate(outs)]      # residual_out over the input
        got = g.fused(d_parts, res.cuda(), w.cuda(), 1e-6, 3, force_mode=TWO_SHOT, outs=outs)
    _check_all_ranks(got, want, 3)


def _emulated_call_async(g, parts, res, w, quant, outs):
    import ctypes
    from gpuk_b200 import cabi
    ws = (ctypes.c_void_p * g.world)(*[h.value for h in g.ws])
    cabi.check(cabi.lib.gpuk_emulated_allreduce_rms(
        ws, g.world, g._arr(parts), util.ptr(res), util.ptr(w), g._arr([o[0] for o in outs]), g._arr([o[1] for o in outs]),
        g._arr([o[2] for o in outs]), parts[0].numel(), parts[0].shape[-1], cabi.dtype_code(parts[0].dtype), 1e-6, quant,
        TWO_SHOT, util.stream_ptr()))


@pytest.mark.parametrize("world", [2, 8])
def test_input_produced_in_scrambled_row_blocks_while_the_exchange_runs(world):
    """The step before the path (model/tensor_parallel.py:117): the exchange is launched while its input does
    not exist yet.  Row blocks of every rank's partial arrive one by one, in a different scrambled order on
    every rank, each followed by its ready word -- written by the copy engine from pinned memory, which needs
    no SM (the waiting kernel holds them).  A kernel that read a row before its word would pick up the NaN
    fill; results must be those of the oracle."""
    import ctypes
    from cuda.bindings import runtime as cudart  # noqa: F401  (imported before any kernel waits)
    from gpuk_b200 import cabi
    tokens, hidden, rows_per_word = 600, 2048, 64
    nwords = -(-tokens // rows_per_word)
    assert cabi.plan(world, tokens * hidden, hidden, oneshot_max_bytes=1).ws == 1
    parts, res, w = util.random_case(world, tokens, hidden, torch.bfloat16, seed=world + 4000)
    want = eo.epilogue_t1(parts, res, w, 1e-6, 3)
    pinned = [p.pin_memory() for p in parts]
    with util.EmulatedGroup(world, max_bytes=4 << 20) as g:
        g.set_option("ws_max_ctas", 16)        # the kernels of all emulated ranks leave some SMs of the one GPU free
        for call in range(2):
            value = call + 1                   # words count calls up, nothing is reset in between
            d_parts = [torch.full((tokens, hidden), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
            if call == 0:
                words = [torch.zeros(nwords, dtype=torch.int32, device="cuda") for _ in range(world)]
            flag = torch.tensor([value], dtype=torch.int32).pin_memory()
            d_res, d_w = res.cuda(), w.cuda()
            outs = [util.alloc_outputs(p, 3) for p in d_parts]
            # everything that allocates or creates (streams included: creating one can wait for the device to go
            # idle) happens before the launch; after it only copies are enqueued
            feeder = torch.cuda.Stream()
            gen = torch.Generator().manual_seed(call)
            orders = [torch.randperm(nwords, generator=gen).tolist() for _ in range(world)]
            torch.cuda.synchronize()
            for r in range(world):
                cabi.check(cabi.lib.gpuk_ws_set_ready_words(g.ws[r], ctypes.c_void_p(words[r].data_ptr()), rows_per_word, value))
            _emulated_call_async(g, d_parts, d_res, d_w, 3, outs)
            for step in range(nwords):
                for r in range(world):
                    i = orders[r][step]
                    lo, hi = i * rows_per_word, min((i + 1) * rows_per_word, tokens)
                    util.h2d_async(d_parts[r][lo:hi], pinned[r][lo:hi], feeder)
                    util.h2d_async(words[r][i:i + 1], flag, feeder)
            torch.cuda.synchronize()
            for r in range(world):
                rc, st = g.status(r)
                assert rc == 0, (r, st, cabi.last_error())
            got = [(o[0].cpu(), o[1].cpu(), o[2].cpu()) for o in outs]
            _check_all_ranks(got, want, 3)


def test_ready_word_that_never_arrives_is_reported_and_ready_words_are_refused_where_they_cannot_work():
    import ctypes
    from gpuk_b200 import cabi
    world, tokens, hidden = 2, 300, 2048
    parts, res, w = util.random_case(world, tokens, hidden, torch.bfloat16, seed=9)
    d_parts, d_res, d_w = [p.cuda() for p in parts], res.cuda(), w.cuda()
    with util.EmulatedGroup(world, max_bytes=4 << 20) as g:
        words = [torch.ones(5, dtype=torch.int32, device="cuda") for _ in range(world)]
        words[1][3] = 0                                         # rows 192..255 of rank 1 never become ready
        for r in range(world):
            cabi.check(cabi.lib.gpuk_ws_set_timeout_ns(g.ws[r], 50_000_000))
            cabi.check(cabi.lib.gpuk_ws_set_ready_words(g.ws[r], ctypes.c_void_p(words[r].data_ptr()), 64, 1))
        outs = [util.alloc_outputs(p, 3) for p in d_parts]
        _emulated_call_async(g, d_parts, d_res, d_w, 3, outs)
        torch.cuda.synchronize()
        rc, st = g.status(1)
        assert rc == cabi.ERR_PEER_TIMEOUT and st[0] == 1 and st[1] == 1 and st[3] == 6, (rc, st)      # stage 6: a ready word
        g.clear_status()
        # ready words apply to one call: the next one runs without them and is correct
        _check_all_ranks(g.fused(d_parts, d_res, d_w, 1e-6, 3, force_mode=TWO_SHOT), eo.epilogue_t1(parts, res, w, 1e-6, 3), 3)
        # a call that takes the one-shot exchange cannot wait for ready words: refused, not ignored
        small = util.random_case(world, 4, 2048, torch.bfloat16, seed=10)
        for r in range(world):
            cabi.check(cabi.lib.gpuk_ws_set_ready_words(g.ws[r], ctypes.c_void_p(words[r].data_ptr()), 64, 1))
        with pytest.raises(cabi.GpukError) as e:
            g.fused([p.cuda() for p in small[0]], small[1].cuda(), small[2].cuda(), 1e-6, 3)
        assert e.value.status == cabi.ERR_UNSUPPORTED


def test_prefill_distribution_with_outliers_eight_ranks():
    """Config 4's inputs (0.1 % of the partials multiplied by 20, seeds of the benchmark) at
    2048 of its 16384 rows, eight ranks, two-shot: more chunks than resident CTAs."""
    cfg = oin.CONFIGS["c4"]
    parts, res, w = oin.make_case(cfg, 8, tokens=2048)
    with util.EmulatedGroup(8, max_bytes=32 << 20) as g:
        outs = g.fused([p.cuda() for p in parts], res.cuda(), w.cuda(), cfg.eps, cfg.quant_type, force_mode=TWO_SHOT)
    want = eo.epilogue_t1(parts, res, w, cfg.eps, cfg.quant_type)
    _check_all_ranks(outs, want, cfg.quant_type)


def test_mid_batch_config_two_and_eight_ranks():
    """Config 3 (1024 x 8192, the benchmark's seeds) as the policy runs it."""
    cfg = oin.CONFIGS["c3"]
    for world in (2, 8):
        parts, res, w = oin.make_case(cfg, world)
        with util.EmulatedGroup(world, max_bytes=16 << 20) as g:
            outs = g.fused([p.cuda() for p in parts], res.cuda(), w.cuda(), cfg.eps, cfg.quant_type)
        want = eo.epilogue_t1(parts, res, w, cfg.eps, cfg.quant_type)
        _check_all_ranks(outs, want, cfg.quant_type)


def test_benchmark_decode_config_eight_ranks():
    """Config 2 (8 x 8192, partials ~N(0,1)/sqrt(8), static scale 0.05) and config 5's message."""
    for name in ("c2", "c5"):
        cfg = oin.CONFIGS[name]
        parts, res, w = oin.make_case(cfg, 8)
        with util.EmulatedGroup(8) as g:
            outs = g.fused([p.cuda() for p in parts], res.cuda(), w.cuda(), cfg.eps, cfg.quant_type, cfg.static_scale)
        want = eo.epilogue_t1(parts, res, w, cfg.eps, cfg.quant_type, cfg.static_scale)
        _check_all_ranks(outs, want, cfg.quant_type)


def test_message_larger_than_workspace_is_an_error():
    from gpuk_b200 import cabi
    parts, res, w = util.random_case(2, 64, 4096, torch.bfloat16, seed=1)
    with util.EmulatedGroup(2, max_bytes=64 * 1024) as g:
        with pytest.raises(cabi.GpukError) as e:
            g.fused([p.cuda() for p in parts], res.cuda(), w.cuda(), 1e-6, 3)
        assert e.value.status == cabi.ERR_TOO_LARGE
