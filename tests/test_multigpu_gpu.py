"""Real multi-GPU runs (skipped when fewer than two GPUs are visible).

* one process owning all GPUs with peer access enabled, like the reference's C++ harness
  (test/cpp/test_all_reduce.cpp:337-356,652-653);
* one process per GPU with NCCL bootstrap and CUDA-IPC handle exchange through GPUKDistEnv,
  like test/test_all_reduce_fusion.py:30-98, compared with the oracle (T1) and with the live
  NCCL path (T2).
"""
import ctypes
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import epilogue_oracle as eo   # noqa: E402
from tests import util                     # noqa: E402

NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0
needs2 = pytest.mark.skipif(NGPU < 2, reason="needs at least two GPUs")


def _worlds():
    return [w for w in (2, 4, 8) if w <= NGPU] or [2]


class PeerGroup:
    """One workspace per device, wired by raw peer pointers inside one process."""

    def __init__(self, world, max_bytes=64 << 20):
        from gpuk_b200 import cabi
        self.cabi = cabi
        self.world = world
        cabi.check(cabi.lib.gpuk_enable_peer_access(world))
        self.ws = []
        for r in range(world):
            h = ctypes.c_void_p()
            cabi.check(cabi.lib.gpuk_ws_create(r, r, world, max_bytes, 0, ctypes.byref(h)))
            self.ws.append(h)
        flags = (ctypes.c_void_p * world)()
        data = (ctypes.c_void_p * world)()
        for r in range(world):
            f, d = ctypes.c_void_p(), ctypes.c_void_p()
            cabi.check(cabi.lib.gpuk_ws_local_pointers(self.ws[r], ctypes.byref(f), ctypes.byref(d)))
            flags[r], data[r] = f, d
        for r in range(world):
            cabi.check(cabi.lib.gpuk_ws_set_peer_pointers(self.ws[r], flags, data, world))

    def close(self):
        for h in self.ws:
            self.cabi.lib.gpuk_ws_destroy(h)

    def attach_symmetric(self, message_bytes, min_bytes):
        """Plain device buffers with peer access stand in for symmetric memory (no multicast mapping)."""
        cabi = self.cabi
        nbytes = (2 * ((message_bytes + 255) // 256 * 256) + cabi.SYM_FLAG_BYTES + 1023) // 256 * 256
        self.sym = [torch.zeros(nbytes, dtype=torch.uint8, device=f"cuda:{r}") for r in range(self.world)]
        for r in range(self.world):
            torch.cuda.synchronize(r)
        bases = (ctypes.c_void_p * self.world)(*[t.data_ptr() for t in self.sym])
        for h in self.ws:
            cabi.check(cabi.lib.gpuk_ws_attach_symmetric(h, bases, self.world, None, nbytes))
            cabi.check(cabi.lib.gpuk_ws_set_option(h, b"sym_min_bytes", min_bytes))

    def fused(self, parts, residual, weight, eps, quant, static_scale=None):
        cabi = self.cabi
        dev = [(parts[r].cuda(r), residual.cuda(r), weight.cuda(r)) for r in range(self.world)]
        outs = [util.alloc_outputs(dev[r][0], quant, static_scale) for r in range(self.world)]
        hidden = parts[0].shape[-1]
        for r in range(self.world):      # launches are asynchronous: all ranks are in flight together
            with torch.cuda.device(r):
                x, res, w = dev[r]
                cabi.check(cabi.lib.gpuk_allreduce_rms(
                    self.ws[r], util.ptr(x), util.ptr(res), util.ptr(w), util.ptr(outs[r][0]), util.ptr(outs[r][1]),
                    util.ptr(outs[r][2]), x.numel(), hidden, cabi.dtype_code(x.dtype), eps, quant,
                    ctypes.c_void_p(torch.cuda.current_stream(r).cuda_stream)))
        for r in range(self.world):
            torch.cuda.synchronize(r)
        for r in range(self.world):
            out = (ctypes.c_uint32 * 8)()
            assert cabi.lib.gpuk_ws_status(self.ws[r], out) == 0, list(out)
        return [(o[0].cpu(), o[1].cpu(), o[2].cpu() if quant else None) for o in outs]


@needs2
@pytest.mark.parametrize("world", _worlds())
def test_single_process_peer_access(world):
    g = PeerGroup(world)
    try:
        for i, (tokens, hidden, quant) in enumerate([(8, 8192, 4), (8, 8192, 3), (129, 1024, 1), (1024, 8192, 3),
                                                     (8, 8192, 3), (37, 7168, 2), (2048, 7168, 3), (1, 4096, 0)]):
            parts, res, w = util.random_case(world, tokens, hidden, torch.bfloat16, seed=world * 100 + i)
            static = 0.05 if quant == 4 else None
            outs = g.fused(parts, res, w, 1e-6, quant, static)
            want = eo.epilogue_t1(parts, res, w, 1e-6, quant, static)
            for got in outs:
                util.check_against_oracle(got, want, quant)
                assert torch.equal(got[1].view(torch.uint8), outs[0][1].view(torch.uint8))
    finally:
        g.close()


@needs2
@pytest.mark.parametrize("world", _worlds())
def test_single_process_exchange_through_symmetric_memory(world):
    """The pull variant (peer loads, rank-order sum) of the exchange through symmetric memory over real NVLink."""
    g = PeerGroup(world)
    try:
        g.attach_symmetric(2048 * 7168 * 2, 1)
        for i, (tokens, hidden, quant) in enumerate([(1024, 8192, 3), (129, 1024, 1), (2048, 7168, 3), (1024, 8192, 3), (37, 7168, 0)]):
            parts, res, w = util.random_case(world, tokens, hidden, torch.bfloat16, seed=world * 200 + i)
            outs = g.fused(parts, res, w, 1e-6, quant)
            want = eo.epilogue_t1(parts, res, w, 1e-6, quant)
            for got in outs:
                util.check_against_oracle(got, want, quant)
                assert torch.equal(got[1].view(torch.uint8), outs[0][1].view(torch.uint8))
    finally:
        g.close()


def _check_benchmark_config(g, key, world, sample_every):
    """One call on real GPUs with the benchmark's own seeded inputs: residual_out must equal
    T(T1 sum + residual) on ALL rows bit for bit, FP8 codes and scales are compared with the oracle
    on every `sample_every`-th row, and all ranks must hold identical bytes."""
    from gpuk_b200 import workloads as oin
    cfg = oin.CONFIGS[key]
    parts, res, w = oin.make_case(cfg, world)
    outs = g.fused(parts, res, w, cfg.eps, cfg.quant_type, cfg.static_scale)
    total = eo.allreduce_t1(parts)
    want_res = total + res
    for r, got in enumerate(outs):
        assert torch.equal(got[0].view(torch.int16), want_res.view(torch.int16)), (key, world, r)
        assert torch.equal(got[1].view(torch.uint8), outs[0][1].view(torch.uint8)), (key, world, r)
    idx = torch.arange(0, cfg.tokens, sample_every)
    want = eo.add_rms_quant(total[idx], res[idx], w, cfg.eps, cfg.quant_type, cfg.static_scale)
    got = outs[world - 1]
    util.check_against_oracle((got[0][idx], got[1][idx], got[2][idx] if cfg.quant_type != 4 else got[2]), want, cfg.quant_type)


@needs2
@pytest.mark.parametrize("world", sorted({2, max(_worlds())}))
def test_benchmark_configs_with_their_own_seeds_on_real_gpus(world):
    """Configs 2, 3 and 5 in full and config 4 (16384 x 7168, 0.1 % outliers x 20) in full: the shapes, seeds
    and distributions bench.py times, here with their results checked."""
    g = PeerGroup(world, max_bytes=224 << 20)
    try:
        for key, every in (("c2", 1), ("c5", 1), ("c3", 1), ("c4", 16)):
            _check_benchmark_config(g, key, world, every)
    finally:
        g.close()


@needs2
@pytest.mark.parametrize("world", sorted({2, max(_worlds())}))
def test_exchange_starts_before_its_input_is_complete_on_real_gpus(world):
    """Ready words over real NVLink: every rank's kernel is launched first, then the rows of its partial and
    their ready words arrive block by block through the copy engine, in a different scrambled order per rank."""
    from cuda.bindings import runtime as cudart  # noqa: F401  (imported before any kernel waits)
    from gpuk_b200 import cabi
    tokens, hidden, rows_per_word = 1200, 4096, 128
    nwords = -(-tokens // rows_per_word)
    parts, res, w = util.random_case(world, tokens, hidden, torch.bfloat16, seed=world + 77)
    want = eo.epilogue_t1(parts, res, w, 1e-6, 3)
    pinned = [p.pin_memory() for p in parts]
    flag = torch.tensor([1], dtype=torch.int32).pin_memory()
    g = PeerGroup(world)
    try:
        dev = [(torch.full((tokens, hidden), float("nan"), dtype=torch.bfloat16, device=f"cuda:{r}"), res.cuda(r), w.cuda(r))
               for r in range(world)]
        words = [torch.zeros(nwords, dtype=torch.int32, device=f"cuda:{r}") for r in range(world)]
        outs = [util.alloc_outputs(dev[r][0], 3) for r in range(world)]
        # streams are created before the launches (creating one can wait for the device to go idle)
        gen = torch.Generator().manual_seed(world)
        orders = [torch.randperm(nwords, generator=gen).tolist() for _ in range(world)]
        feeders = [torch.cuda.Stream(device=r) for r in range(world)]
        for r in range(world):
            torch.cuda.synchronize(r)
        for r in range(world):
            with torch.cuda.device(r):
                x, rr, ww = dev[r]
                cabi.check(cabi.lib.gpuk_ws_set_ready_words(g.ws[r], ctypes.c_void_p(words[r].data_ptr()), rows_per_word, 1))
                cabi.check(cabi.lib.gpuk_allreduce_rms(
                    g.ws[r], util.ptr(x), util.ptr(rr), util.ptr(ww), util.ptr(outs[r][0]), util.ptr(outs[r][1]), util.ptr(outs[r][2]),
                    x.numel(), hidden, cabi.DTYPE_BF16, 1e-6, 3, ctypes.c_void_p(torch.cuda.current_stream(r).cuda_stream)))
        for step in range(nwords):
            for r in range(world):
                i = orders[r][step]
                lo, hi = i * rows_per_word, min((i + 1) * rows_per_word, tokens)
                with torch.cuda.device(r):
                    util.h2d_async(dev[r][0][lo:hi], pinned[r][lo:hi], feeders[r])
                    util.h2d_async(words[r][i:i + 1], flag, feeders[r])
        for r in range(world):
            torch.cuda.synchronize(r)
        for r in range(world):
            out = (ctypes.c_uint32 * 8)()
            assert cabi.lib.gpuk_ws_status(g.ws[r], out) == 0, list(out)
            got = (outs[r][0].cpu(), outs[r][1].cpu(), outs[r][2].cpu())
            util.check_against_oracle(got, want, 3)
    finally:
        g.close()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _ipc_worker(rank, world, port, cases, q):
    import torch.distributed as dist
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    import gpuk_b200
    from gpuk_b200 import cabi
    env = gpuk_b200.GPUKDistEnv(group=None, device_id=rank, max_size_in_bytes=64 << 20, symmetric_bytes=40 << 20)
    failures = []
    try:
        for i, (tokens, hidden, fp8_out) in enumerate(cases):
            parts, res, w = util.random_case(world, tokens, hidden, torch.bfloat16, seed=900 + i)
            x = parts[rank].cuda()
            r_d, w_d = res.cuda(), w.cuda()
            # large cases go through symmetric memory, read with plain peer loads (bit-exact)
            env.set_option("sym_multicast", 0)
            env.set_option("sym_min_bytes", 1 << 20 if i % 2 == 0 else 0)
            got = env.allreduce_add_rms_fused(x.clone(), r_d, w_d, 1e-6, fp8_out)
            nat = env.allreduce_add_rms_native(x.clone(), r_d, w_d, 1e-6, fp8_out)
            torch.cuda.synchronize()
            quant = 3 if fp8_out else 0
            want = eo.epilogue_t1(parts, res, w, 1e-6, quant)
            got_c = (got[0].cpu(), got[1].cpu(), got[2].cpu() if fp8_out else None)
            try:
                util.check_against_oracle(got_c, want, quant)
                if world == 2:   # a two-rank bf16 collective is a single add: the live path must agree too
                    nat_c = (nat[0].cpu(), nat[1].cpu(), nat[2].cpu() if fp8_out else None)
                    util.check_against_oracle(got_c, nat_c, quant)
                plain = env.allreduce(x)
                assert torch.equal(plain.cpu().view(torch.int16), eo.allreduce_t1(parts).view(torch.int16))
            except AssertionError as e:   # pragma: no cover
                failures.append(f"case {i} {tokens}x{hidden}: {e}")
        # host-buffer API: rows pipelined in pieces, every piece a full exchange
        parts, res, w = util.random_case(world, 300, 4096, torch.bfloat16, seed=777)
        out = (torch.empty_like(res).pin_memory(), torch.empty(res.shape, dtype=torch.float8_e4m3fn).pin_memory(),
               torch.empty(300, 1).pin_memory())
        env.allreduce_add_rms_fused_host(parts[rank].pin_memory(), res.pin_memory(), w.cuda(), 1e-6, out, chunks=4)
        try:
            util.check_against_oracle(out, eo.epilogue_t1(parts, res, w, 1e-6, 3), 3)
        except AssertionError as e:   # pragma: no cover
            failures.append(f"host api: {e}")
        if env.multicast:
            # The same exchange reduced inside the NVSwitch.  The switch rounds 16-bit sums its own way
            # (ties away from zero), so about one sum in seven is off by one unit in the last place:
            # outside the parity bars, therefore opt-in, and checked here for closeness only.
            env.set_option("sym_multicast", 1)
            env.set_option("sym_min_bytes", 1)
            parts, res, w = util.random_case(world, 700, 4096, torch.bfloat16, seed=4242)
            got = env.allreduce_add_rms_fused(parts[rank].cuda(), res.cuda(), w.cuda(), 1e-6, False)
            torch.cuda.synchronize()
            want = eo.epilogue_t1(parts, res, w, 1e-6, 0)
            try:
                torch.testing.assert_close(got[0].cpu().float(), want[0].float(), atol=4e-2, rtol=2e-2)
                torch.testing.assert_close(got[1].cpu().float(), want[1].float(), atol=4e-2, rtol=2e-2)
            except AssertionError as e:   # pragma: no cover
                failures.append(f"multicast: {e}")
            env.set_option("sym_min_bytes", 0)
        out = (ctypes.c_uint32 * 8)()
        rc = cabi.lib.gpuk_ws_status(ctypes.c_void_p(env.fptr), out)
        if rc:
            failures.append(f"status {list(out)}")
    finally:
        q.put((rank, failures))
        env.barrier()
        del env
        dist.destroy_process_group()


def _graph_worker(rank, world, port, q):
    """Two fused calls captured into one CUDA graph through GPUKDistEnv, replayed on new data."""
    import torch.distributed as dist
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    import gpuk_b200
    # the two-shot gather goes through the NVSwitch multicast address where the fabric has one (asked for
    # explicitly: by default it is used from four ranks)
    env = gpuk_b200.GPUKDistEnv(group=None, device_id=rank, max_size_in_bytes=64 << 20, gather_multicast=True)
    failures = []
    try:
        shapes = [(8, 8192), (300, 8192)]        # one-shot over a cluster, two-shot
        x = [torch.zeros(t, h, dtype=torch.bfloat16, device="cuda") for t, h in shapes]
        r = [torch.zeros(t, h, dtype=torch.bfloat16, device="cuda") for t, h in shapes]
        w = [torch.ones(h, dtype=torch.bfloat16, device="cuda") for _, h in shapes]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            for i in range(2):                   # warm-up outside the capture (both staging parities)
                [env.allreduce_add_rms_fused(x[k], r[k], w[k], 1e-6, True) for k in range(2)]
            torch.cuda.synchronize()
            env.barrier()
            with env.capture():
                with torch.cuda.graph(graph, stream=side):
                    outs = [env.allreduce_add_rms_fused(x[k], r[k], w[k], 1e-6, True) for k in range(2)]
        torch.cuda.current_stream().wait_stream(side)
        for rep in range(3):
            cases = [util.random_case(world, t, h, torch.bfloat16, seed=5000 + 10 * rep + k) for k, (t, h) in enumerate(shapes)]
            for k, (parts, res, wt) in enumerate(cases):
                x[k].copy_(parts[rank])
                r[k].copy_(res)
                w[k].copy_(wt)
            torch.cuda.synchronize()
            env.barrier()
            graph.replay()
            if rep == 1:
                graph.replay()      # twice on the same data: the device-side call counter must still be in step
            torch.cuda.synchronize()
            for k, (parts, res, wt) in enumerate(cases):
                want = eo.epilogue_t1(parts, res, wt, 1e-6, 3)
                got = tuple(t.cpu() for t in outs[k])
                try:
                    util.check_against_oracle(got, want, 3)
                except AssertionError as e:   # pragma: no cover
                    failures.append(f"replay {rep} shape {shapes[k]}: {e}")
        try:
            env.check()
        except RuntimeError as e:   # pragma: no cover
            failures.append(str(e))
    finally:
        q.put((rank, failures))
        env.barrier()
        del env
        dist.destroy_process_group()


@needs2
@pytest.mark.parametrize("world", sorted({2, max(_worlds())}))
def test_cuda_graph_replay_across_ranks_follows_new_data(world):
    """The registration-free design rests on this: a graph that holds fused calls of several ranks can be
    replayed any number of times and stays in step, because the call counter lives on the device
    (the reference registers and IPC-maps captured inputs instead, all_reduce_fusion.cpp:105-137, 168-233;
    gpuk/__init__.py:98-129)."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_graph_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
    for rank, failures in results:
        assert not failures, (rank, failures)
    assert all(p.exitcode == 0 for p in procs)


@needs2
@pytest.mark.parametrize("world", _worlds())
def test_one_process_per_gpu_over_ipc(world):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    cases = [(8, 8192, True), (1, 4096, True), (1024, 8192, True), (1024, 8192, True), (1100, 7168, False), (512, 7168, True),
             (901, 2056, True), (129, 1024, True)]
    port = _free_port()
    procs = [ctx.Process(target=_ipc_worker, args=(r, world, port, cases, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
    for rank, failures in results:
        assert not failures, (rank, failures)
    assert all(p.exitcode == 0 for p in procs)
