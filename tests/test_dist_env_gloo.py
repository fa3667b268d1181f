"""GPUKDistEnv's host logic on CPU ranks (gloo, world size 2): the bootstrap exchanges every
rank's handles in rank order, unsupported group sizes leave the workspace unset, and the
live-collective oracle (T2) agrees with the fp32-accumulating oracle (T1) at two ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class FakeOps:
    """Records the operator calls GPUKDistEnv makes; stands in for torch.ops.gpuk on CPU."""

    def __init__(self, rank):
        self.rank = rank
        self.calls = []
        self.opened = {}

    def set_device(self, d):
        self.calls.append(("set_device", d))

    def synchronize(self, d):
        self.calls.append(("synchronize", d))

    def is_capturing(self):
        return False

    def init_ar_fusion(self, device_id, rank, world, max_bytes, buf_len):
        self.calls.append(("init", device_id, rank, world, max_bytes, buf_len))
        return 4242 + rank

    def destroy_ar_fusion(self, fptr):
        self.calls.append(("destroy", fptr))

    def get_ar_fusion_barrier_handle(self, fptr):
        return torch.full((64,), 10 + self.rank, dtype=torch.uint8)

    def get_ar_fusion_data_handle(self, fptr):
        return torch.full((64,), 20 + self.rank, dtype=torch.uint8)

    def open_ar_fusion_barrier_handles(self, fptr, handles):
        self.opened["barrier"] = [int(h[0]) for h in handles]

    def open_ar_fusion_data_handles(self, fptr, handles):
        self.opened["data"] = [int(h[0]) for h in handles]

    def get_ar_fusion_captured_handles(self, fptr):
        return []

    def get_ar_fusion_captured_offsets(self, fptr):
        return torch.empty(0, dtype=torch.int64)

    def ar_fusion_capture_clear(self, fptr):
        self.calls.append(("capture_clear", fptr))


def _worker(rank, world, port, q):
    torch.set_num_threads(1)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    import gpuk_b200
    from oracle import epilogue_oracle as eo
    out = {}
    fake = FakeOps(rank)
    env = gpuk_b200.GPUKDistEnv(group=None, device_id=rank, max_size_in_bytes=1 << 20, _ops=fake)
    out["fptr"] = env.fptr
    out["opened"] = fake.opened
    out["init"] = [c for c in fake.calls if c[0] == "init"]
    with env.capture():
        pass
    out["cleared"] = ("capture_clear", env.fptr) in fake.calls

    # native path over gloo (T2) against the oracle (T1)
    g = torch.Generator().manual_seed(3)
    parts = [torch.randn(16, 512, generator=g).to(torch.bfloat16) for _ in range(world)]
    res = torch.randn(16, 512, generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(512, generator=g)).to(torch.bfloat16)
    nat = env.allreduce_add_rms_native(parts[rank].clone(), res, w, 1e-6, True)
    want = eo.epilogue_t1(parts, res, w, 1e-6, gpuk_b200.fp8_policy_id)
    out["t2_equals_t1"] = (torch.equal(nat[0], want[0]) and torch.equal(nat[2], want[2])
                           and torch.equal(nat[1].view(torch.uint8), want[1].view(torch.uint8)))
    q.put((rank, out))
    dist.barrier()
    env.fptr = None
    dist.destroy_process_group()


def test_bootstrap_and_native_path_over_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank in range(world):
        r = results[rank]
        assert r["fptr"] == 4242 + rank
        assert r["opened"] == {"barrier": [10, 11], "data": [20, 21]}     # every rank's handle, in rank order
        assert r["init"] == [("init", rank, rank, 2, 1 << 20, 1024 * 256)]
        assert r["cleared"]
        assert r["t2_equals_t1"]


def _solo_worker(port, q):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    import gpuk_b200
    fake = FakeOps(0)
    env = gpuk_b200.GPUKDistEnv(group=None, device_id=0, _ops=fake)
    q.put((env.fptr, [c[0] for c in fake.calls]))
    dist.destroy_process_group()


def test_group_of_one_creates_no_workspace():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_solo_worker, args=(_free_port(), q))
    p.start()
    fptr, calls = q.get(timeout=120)
    p.join(timeout=60)
    assert fptr is None and "init" not in calls       # gpuk/__init__.py:72-73


def test_fp8_policy_table_matches_the_reference():
    import gpuk_b200
    assert gpuk_b200._POLICIES["e4m3fn_240"][1:] == (240, 1)       # gpuk/__init__.py:42-51
    assert gpuk_b200._POLICIES["e4m3fnuz_120"][1:] == (120, 2)
    gpuk_b200.set_fp8_policy("e4m3fnuz_120")
    assert gpuk_b200.fp8 is torch.float8_e4m3fnuz and gpuk_b200.fp8_max_val == 120 and gpuk_b200.fp8_policy_id == 2
    gpuk_b200.set_fp8_policy("e4m3fn_448")
    with pytest.raises(ValueError):
        gpuk_b200.set_fp8_policy("e5m2")
