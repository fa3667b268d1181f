"""One GPU, no communication: residual add + RMSNorm + FP8 through the C ABI vs the CPU oracle."""
import glob
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import epilogue_oracle as eo          # noqa: E402
from gpuk_b200 import workloads as oin                  # noqa: E402
from tests import util                            # noqa: E402
from tests.test_oracle import GOLDEN, load_golden  # noqa: E402


def _run(x, res, w, eps, quant, static_scale=None):
    got = util.k1(x.cuda(), res.cuda(), w.cuda(), eps, quant, static_scale)
    want = eo.add_rms_quant(x, res, w, eps, quant, static_scale)
    return got, want


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_golden_vectors_from_the_reference(path):
    """The collective's own output from the golden file stands in for the sum."""
    c = load_golden(path)
    got = util.k1(c["allreduce_out"].cuda(), c["residual"].cuda(), c["weight"].cuda(), c["eps"], c["quant"])
    want = (c["residual_out"], c["norm_out"], c["scale"])
    util.check_against_oracle(got, want, c["quant"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("quant", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("tokens,hidden", [(1, 4096), (129, 1024), (128, 1024), (8, 8192), (37, 7168), (3, 8), (5, 2056)])
def test_shapes_dtypes_policies(tokens, hidden, quant, dtype):
    """Shapes of the reference's own test list (test/test_all_reduce_fusion.py:166-208) plus
    the benchmark's hidden sizes, the smallest legal row and a row that fills no tile evenly."""
    if dtype == torch.float32 and hidden % 4:
        pytest.skip("row not a multiple of 16 bytes")
    if dtype != torch.float32 and hidden % 8:
        pytest.skip("row not a multiple of 16 bytes")
    parts, res, w = util.random_case(1, tokens, hidden, dtype, seed=tokens * 31 + hidden + quant)
    got, want = _run(parts[0], res, w, 1e-6, quant, 0.05 if quant == 4 else None)
    util.check_against_oracle(got, want, quant)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("quant", [0, 3, 4])
@pytest.mark.parametrize("tokens,hidden", [(2368, 1024), (5000, 2048), (2400, 8192), (2501, 7168), (3000, 136)])
def test_many_rows_staged_through_shared_memory(tokens, hidden, quant, dtype):
    """Row counts from sixteen times the SM count up run on persistent CTAs that fetch rows into a
    shared-memory ring with bulk copies: ring wrap-around (several rows per CTA), a ragged last
    round, rows whose size is not a power of two, and a narrow row (two warps per CTA)."""
    parts, res, w = util.random_case(1, tokens, hidden, dtype, seed=tokens + hidden + quant)
    got, want = _run(parts[0], res, w, 1e-6, quant, 0.05 if quant == 4 else None)
    util.check_against_oracle(got, want, quant, exact_residual=True)


def test_long_rows():
    for hidden in (16384, 32768):
        parts, res, w = util.random_case(1, 4, hidden, torch.bfloat16, seed=hidden)
        got, want = _run(parts[0], res, w, 1e-6, 3)
        util.check_against_oracle(got, want, 3)


def test_empty_and_zero_rows():
    bf = torch.bfloat16
    x = torch.zeros(0, 1024, dtype=bf)
    got = util.k1(x.cuda(), x.cuda(), torch.ones(1024, dtype=bf).cuda(), 1e-6, 3)
    assert got[0].shape == (0, 1024)
    z = torch.zeros(4, 1024, dtype=bf)
    got, want = _run(z, z, torch.ones(1024, dtype=bf), 1e-6, 3)
    assert got[2].tolist() == [[1.0]] * 4            # all-zero rows keep scale 1 (impl.h:217)
    assert int(got[1].view(torch.uint8).max()) == 0


def test_row_maximum_maps_to_fp8_max():
    parts, res, w = util.random_case(1, 64, 4096, torch.bfloat16, seed=3)
    for quant, top in ((1, 240.0), (2, 120.0), (3, 448.0)):
        got, _ = _run(parts[0], res, w, 1e-6, quant)
        assert torch.all(got[1].float().abs().amax(dim=-1) == top)


def test_rejects_bad_arguments():
    from gpuk_b200 import cabi
    x = torch.zeros(4, 1024, dtype=torch.bfloat16, device="cuda")
    s = torch.zeros(4, dtype=torch.float32, device="cuda")
    args = lambda h, q, xin=x: (util.ptr(xin), util.ptr(x), util.ptr(x), util.ptr(x), util.ptr(x), util.ptr(s),
                                x.numel(), h, 0, 1e-6, q, util.stream_ptr())
    assert cabi.lib.gpuk_residual_rms_quant(*args(1020, 3)) == cabi.ERR_UNSUPPORTED      # 1020 % 8 != 0
    assert cabi.lib.gpuk_residual_rms_quant(*args(1000, 3)) in (cabi.ERR_INVALID_ARGUMENT, cabi.ERR_UNSUPPORTED)
    assert cabi.lib.gpuk_residual_rms_quant(*args(1024, 9)) == cabi.ERR_INVALID_ARGUMENT  # unknown policy
    mis = x.view(-1)[4:4 + 2048].view(2, 1024)                                            # 8-byte offset
    assert cabi.lib.gpuk_residual_rms_quant(util.ptr(mis), util.ptr(x), util.ptr(x), util.ptr(x), util.ptr(x),
                                            util.ptr(s), 2048, 1024, 0, 1e-6, 3, util.stream_ptr()) == cabi.ERR_INVALID_ARGUMENT
    torch.cuda.synchronize()


def test_through_the_operator_library_with_a_group_of_one():
    """torch.ops.gpuk.allreduce_rms with a null workspace = the no-communication kernel."""
    import gpuk_b200
    parts, res, w = util.random_case(1, 33, 4096, torch.bfloat16, seed=9)
    x, r, g = parts[0].cuda(), res.cuda(), w.cuda()
    res_out, norm_out, scale = util.alloc_outputs(x, 3)
    gpuk_b200.allreduce_rms(0, x, r, g, res_out, norm_out, scale, 1e-6, 3)
    torch.cuda.synchronize()
    want = eo.add_rms_quant(parts[0], res, w, 1e-6, 3)
    util.check_against_oracle((res_out.cpu(), norm_out.cpu(), scale.cpu()), want, 3)


@pytest.mark.parametrize("tokens,chunks,static", [(1000, 4, None), (37, 8, None), (5, 16, None), (256, 3, 0.05)])
def test_host_buffer_api_pipelines_row_pieces(tokens, chunks, static):
    """GPUKDistEnv.allreduce_add_rms_fused_host: pinned host tensors in, pinned host tensors out, rows
    cut into pieces (the last one ragged, more pieces than rows clamps) -- same results as one call."""
    import torch.distributed as dist
    import gpuk_b200
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29571")
        dist.init_process_group("gloo", rank=0, world_size=1)
    env = gpuk_b200.GPUKDistEnv(group=None, device_id=0)
    parts, res, w = util.random_case(1, tokens, 2048, torch.bfloat16, seed=tokens + chunks)
    out = (torch.empty_like(res).pin_memory(), torch.empty(res.shape, dtype=torch.float8_e4m3fn).pin_memory(),
           torch.full((tokens, 1), -1.0).pin_memory())
    st = None if static is None else torch.tensor([static], dtype=torch.float32, device="cuda")
    for _ in range(2):   # second call reuses the cached device buffers and streams
        env.allreduce_add_rms_fused_host(parts[0].pin_memory(), res.pin_memory(), w.cuda(), 1e-6, out, chunks=chunks,
                                         static_scale=st)
    quant = 4 if static is not None else 3
    want = eo.add_rms_quant(parts[0], res, w, 1e-6, quant, static)
    got = (out[0], out[1], out[2] if static is None else torch.tensor([static]))
    util.check_against_oracle(got, want, quant)


@pytest.mark.parametrize("name,rows", [("c2", None), ("c3", None), ("c4", 16384), ("c5", None)])
def test_benchmark_configs_full_size(name, rows):
    """Full benchmark shapes.  The oracle checks a sample of rows; size-independent properties
    cover the rest: every row's largest FP8 magnitude is the format maximum, dequantised
    values reproduce the unquantised norm within one FP8 step, residual_out = x + residual."""
    cfg = oin.CONFIGS[name]
    x = oin.make_partial(cfg, 0, 1)
    res = oin.make_residual(cfg)
    w = oin.make_weight(cfg)
    got = util.k1(x.cuda(), res.cuda(), w.cuda(), cfg.eps, cfg.quant_type, cfg.static_scale)
    sample = torch.arange(0, cfg.tokens, max(1, cfg.tokens // 256))
    want = eo.add_rms_quant(x[sample], res[sample], w, cfg.eps, cfg.quant_type, cfg.static_scale)
    sub = (got[0][sample], got[1][sample], got[2][sample] if cfg.quant_type != 4 else got[2])
    util.check_against_oracle(sub, want, cfg.quant_type)
    assert torch.equal(got[0], x + res)
    if cfg.quant_type == 3:
        assert torch.all(got[1].float().abs().amax(dim=-1) == 448.0)
        assert torch.all(got[2] > 0)
    # idempotence of the no-quant norm scale: re-running gives the same bits
    again = util.k1(x.cuda(), res.cuda(), w.cuda(), cfg.eps, cfg.quant_type, cfg.static_scale)
    assert torch.equal(again[1].view(torch.uint8), got[1].view(torch.uint8))
