"""The numpy oracle against the golden outputs of the unmodified reference."""
import numpy as np
import pytest

from oracle import converse2d_oracle as orc

N_CASES = 20


@pytest.mark.parametrize("i", range(N_CASES))
def test_oracle_matches_reference_fp64(golden, i):
    c, x, w, b, ref32, ref64 = golden.case(i)
    out = orc.converse2d_forward(x, w, b, c["s"], c["p"], c["mode"], c["eps"], dtype=np.float64)
    assert out.shape == ref64.shape
    assert orc.rel_l2(out, ref64) <= 1e-10


@pytest.mark.parametrize("i", range(N_CASES))
def test_oracle_matches_reference_fp32(golden, i):
    c, x, w, b, ref32, ref64 = golden.case(i)
    out = orc.converse2d_forward(x, w, b, c["s"], c["p"], c["mode"], c["eps"], dtype=np.float32)
    assert out.dtype == np.float32
    # fp32 FFT libraries differ in rounding; the reference's own fp32-vs-fp64 drift is the yardstick
    drift = orc.rel_l2(ref32, ref64)
    assert orc.rel_l2(out, ref64) <= max(1e-4, 4 * drift)


def test_fixture_count(golden):
    assert len(golden) == N_CASES


def test_uncropped_solve_contract(golden):
    # torch.ops.converse2d.forward returns the uncropped plane; cropping it gives the module output
    c, x, w, b, ref32, ref64 = golden.case(1)
    y = orc.boundary_pad(x.astype(np.float64), c["p"], c["mode"])
    full = orc.converse2d_solve(y, orc.nearest_upsample(y, c["s"]), w, b, c["s"], c["eps"], np.float64)
    assert full.shape[-2:] == (y.shape[-2] * c["s"], y.shape[-1] * c["s"])
    k = c["p"] * c["s"]
    assert orc.rel_l2(full[..., k:-k, k:-k], ref64) <= 1e-10


def test_bad_arguments():
    x = np.zeros((1, 2, 4, 4), np.float32)
    w, b = orc.init_weight(2, 3, np.random.default_rng(0))
    with pytest.raises(ValueError):
        orc.converse2d_forward(x, w, b, 1, 5, "circular")
    with pytest.raises(ValueError):
        orc.converse2d_forward(x, w, b, 1, 2, "nope")
    with pytest.raises(ValueError):
        orc.converse2d_solve(x, x, w, b, 0, 1e-5)
