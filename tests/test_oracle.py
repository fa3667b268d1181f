"""The CPU oracle against the reference: golden vectors and the reference's FP8 cast."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import epilogue_oracle as eo
from oracle import ref_fp8

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def _t(arr, dtype):
    if dtype in (torch.bfloat16, torch.float16):
        return torch.from_numpy(arr.view(np.int16).copy()).view(dtype)
    if dtype in (torch.float8_e4m3fn, torch.float8_e4m3fnuz):
        return torch.from_numpy(arr.copy()).view(dtype)
    return torch.from_numpy(arr.copy())


def load_golden(path):
    z = np.load(path)
    world, tokens, hidden, fp8_max, _seed = [int(v) for v in z["meta"]]
    dtype = getattr(torch, str(z["dtype"]))
    fp8_s = str(z["fp8"])
    fp8 = getattr(torch, fp8_s) if fp8_s else None
    quant = 0
    if fp8 is torch.float8_e4m3fnuz:
        quant = 2
    elif fp8 is torch.float8_e4m3fn:
        quant = 1 if fp8_max == 240 else 3
    case = dict(
        world=world, tokens=tokens, hidden=hidden, dtype=dtype, quant=quant, eps=float(z["eps"]),
        parts=[_t(z[f"part{r}"], dtype) for r in range(world)],
        residual=_t(z["residual"], dtype), weight=_t(z["weight"], dtype),
        allreduce_out=_t(z["allreduce_out"], dtype), residual_out=_t(z["residual_out"], dtype),
        norm_out=_t(z["norm_out"], fp8 if fp8 is not None else dtype),
        scale=torch.from_numpy(z["scale"].copy()) if fp8 is not None else None,
    )
    return case


def test_golden_fixtures_present():
    assert len(GOLDEN) >= 11


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_post_collective_sequence_is_bit_exact(path):
    """add_rms_quant on the collective's own output reproduces the reference bit for bit."""
    c = load_golden(path)
    res, norm, scale = eo.add_rms_quant(c["allreduce_out"], c["residual"], c["weight"], c["eps"], c["quant"])
    assert torch.equal(res.view(torch.uint8), c["residual_out"].view(torch.uint8))
    assert torch.equal(norm.view(torch.uint8), c["norm_out"].view(torch.uint8))
    if c["scale"] is not None:
        assert torch.equal(scale, c["scale"])


@pytest.mark.parametrize("path", [p for p in GOLDEN if "/n2_" in p],
                         ids=[os.path.basename(p)[:-4] for p in GOLDEN if "/n2_" in p])
def test_t1_allreduce_equals_live_collective_at_two_ranks(path):
    """With two ranks a bf16 collective is a single add: T1 must equal it exactly."""
    c = load_golden(path)
    got = eo.allreduce_t1(c["parts"])
    assert torch.equal(got.view(torch.uint8), c["allreduce_out"].view(torch.uint8))
    out = eo.epilogue_t1(c["parts"], c["residual"], c["weight"], c["eps"], c["quant"])
    assert torch.equal(out[1].view(torch.uint8), c["norm_out"].view(torch.uint8))


@pytest.mark.parametrize("path", [p for p in GOLDEN if "/n4_" in p or "/n8_" in p],
                         ids=[os.path.basename(p)[:-4] for p in GOLDEN if "/n4_" in p or "/n8_" in p])
def test_t1_vs_live_collective_beyond_two_ranks(path):
    """Beyond two ranks the live bf16 collective rounds after every pairwise add; T1 (one
    rounding) stays within the accumulated rounding bound of it and the finished outputs stay
    close to it: the residual inside the reference tolerance (test/test_all_reduce_fusion.py:82-98),
    FP8 codes within one step on >= 98 % of elements and scales within 2e-2."""
    c = load_golden(path)
    got = eo.allreduce_t1(c["parts"])
    d = (got.float() - c["allreduce_out"].float()).abs()
    bound = sum(p.float().abs() for p in c["parts"]) * 2.0 ** -8 * c["world"]
    assert bool((d <= bound).all())
    res, norm, scale = eo.epilogue_t1(c["parts"], c["residual"], c["weight"], c["eps"], c["quant"])
    # pairwise bf16 adds of values of size ~4..8 carry ~0.03 of rounding each: looser than 2e-2
    torch.testing.assert_close(res.float(), c["residual_out"].float(), atol=1e-1, rtol=2e-2)
    d8 = eo.fp8_ulp_distance(norm, c["norm_out"])
    assert (d8 <= 1).float().mean().item() >= 0.98      # the collective's own noise, not the oracle's
    torch.testing.assert_close(scale, c["scale"], atol=0, rtol=2e-2)


def test_rounding_points_hand_case():
    """A two-element row worked by hand: every bf16 rounding point is visible."""
    bf = torch.bfloat16
    parts = [torch.tensor([[1.0, 2.0]], dtype=bf), torch.tensor([[0.00390625, 1.0]], dtype=bf)]
    res = torch.tensor([[0.5, -1.0]], dtype=bf)
    w = torch.tensor([1.5, 0.75], dtype=bf)
    # sum: 1.00390625 -> bf16 keeps 8 significand bits -> 1.0 (tie to even); 3.0
    s = eo.allreduce_t1(parts)
    assert s.tolist() == [[1.0, 3.0]]
    r_out, n_out, scale = eo.add_rms_quant(s, res, w, 0.0, 3)
    assert r_out.tolist() == [[1.5, 2.0]]
    rstd = 1.0 / np.sqrt(np.float32((1.5 ** 2 + 2.0 ** 2) / 2))
    n1 = torch.tensor([1.5 * rstd, 2.0 * rstd], dtype=torch.float32).to(bf)
    n = (w.float() * n1.float()).to(bf)
    amax = n.float().abs().max()
    assert torch.equal(scale, (amax / 448).reshape(1, 1))
    q = (n.float() / scale).clamp(-448, 448).to(torch.float8_e4m3fn)
    assert torch.equal(n_out.view(torch.uint8), q.view(torch.uint8))
    assert n_out.float().abs().max().item() == 448.0


def test_zero_row_keeps_scale_one():
    bf = torch.bfloat16
    z = torch.zeros(2, 64, dtype=bf)
    r, n, s = eo.add_rms_quant(z, z, torch.ones(64, dtype=bf), 1e-6, 3)
    assert s.tolist() == [[1.0], [1.0]]
    assert int(n.view(torch.uint8).max()) == 0


def test_static_scale_policy():
    bf = torch.bfloat16
    g = torch.Generator().manual_seed(5)
    x = torch.randn(4, 256, generator=g).to(bf)
    res = torch.randn(4, 256, generator=g).to(bf)
    w = torch.ones(256, dtype=bf)
    r, n, s = eo.add_rms_quant(x, res, w, 1e-6, 4, static_scale=0.05)
    assert s.shape == (1,) and abs(s.item() - 0.05) < 1e-9
    _, n_ref, _ = eo.add_rms_quant(x, res, w, 1e-6, 0)
    want = (n_ref.float() / torch.tensor(0.05)).clamp(-448, 448).to(torch.float8_e4m3fn)
    assert torch.equal(n.view(torch.uint8), want.view(torch.uint8))
    with pytest.raises(ValueError):
        eo.add_rms_quant(x, res, w, 1e-6, 4)


def test_ulp_distance_metric():
    a = torch.tensor([0.0, -0.0, 1.0, 448.0, -448.0]).to(torch.float8_e4m3fn)
    b = torch.tensor([0.0, 0.0, 1.125, 416.0, -448.0]).to(torch.float8_e4m3fn)
    assert eo.fp8_ulp_distance(a, b).tolist() == [0, 0, 1, 1, 0]


@pytest.mark.skipif(not ref_fp8.available(), reason="oracle/_ref not built (needs the reference checkout)")
class TestAgainstReferenceSoftwareFp8:
    """The oracle's casts against src/common/float8.h compiled from the reference."""

    def _sweep(self):
        g = torch.Generator().manual_seed(7)
        parts = [
            torch.randn(400_000, generator=g) * 60,
            torch.randn(200_000, generator=g) * 0.05,
            torch.linspace(-260, 260, 100_001),
            torch.tensor([0.0, -0.0, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -11, 240.0, 239.9, 248.0, 119.9, 120.0]),
        ]
        return torch.cat(parts).float()

    def test_max_values(self):
        assert ref_fp8.max_values() == (240, 120)

    def test_e4m3fn_240(self):
        x = self._sweep()
        want = ref_fp8.float_to_fp8(x.numpy(), fnuz=False)
        got = x.clamp(-240, 240).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        assert np.array_equal(got, want)

    def test_e4m3fnuz_120_inside_range(self):
        x = self._sweep().clamp(-120, 120)
        want = ref_fp8.float_to_fp8(x.numpy(), fnuz=True)
        got = x.to(torch.float8_e4m3fnuz).view(torch.uint8).numpy()
        assert np.array_equal(got, want)

    def test_fnuz_equals_doubled_fn_with_negative_zero_folded(self):
        """The identity the CUDA kernel uses for the fnuz flavour: code_fnuz(x) = code_fn(2x),
        with the negative-zero pattern 0x80 (NaN in fnuz) folded to 0x00."""
        x = self._sweep().clamp(-120, 120)
        want = ref_fp8.float_to_fp8(x.numpy(), fnuz=True)
        got = (x * 2).to(torch.float8_e4m3fn).view(torch.uint8).numpy().copy()
        got[got == 0x80] = 0
        assert np.array_equal(got, want)

    def test_decode_tables(self):
        codes = np.arange(256, dtype=np.uint8)
        ref = ref_fp8.fp8_to_float(codes, fnuz=False)
        mine = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
        ok = np.isfinite(mine) & (np.abs(mine) <= 240)
        assert np.array_equal(ref[ok], mine[ok])
        ref_z = ref_fp8.fp8_to_float(codes, fnuz=True)
        mine_z = torch.from_numpy(codes).view(torch.float8_e4m3fnuz).float().numpy()
        ok = np.isfinite(mine_z)
        assert np.array_equal(ref_z[ok], mine_z[ok])
