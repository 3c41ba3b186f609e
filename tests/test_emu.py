"""Host emulation of the CUDA block bodies against the oracle and the golden vectors.

The kernels' per-thread phase functions are compiled for the host (tests/emu) and
run thread by thread.  This checks index arithmetic and the transfer-table
algebra without a GPU; it is not a product path and the package cannot load it.
"""
import ctypes
import numpy as np
import pytest

from oracle import converse2d_oracle as orc
from tests.emu.build_emu import build_emu

PAD = {"circular": 0, "replicate": 1, "reflect": 2, "constant": 3}


@pytest.fixture(scope="module")
def emu():
    lib = ctypes.CDLL(build_emu())
    lib.emu_build_transfer.restype = ctypes.c_int
    lib.emu_converse2d_fwd.restype = ctypes.c_int
    return lib


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def emu_forward(lib, x, w, b, s, p, mode, eps, gelu=0, nthr=96, variant=0, strip=False, strip2=False):
    B, C, H, W = x.shape
    k = w.shape[-1]
    h, wd = H + 2 * p, W + 2 * p
    table = np.zeros((C * h * wd + h + wd + 6 * 128, 2), np.float32)  # room for the large-prime tables
    wf = np.ascontiguousarray(w.reshape(C, k, k), np.float32)
    bf = np.ascontiguousarray(b.reshape(C), np.float32)
    rc = lib.emu_build_transfer(_ptr(wf), _ptr(bf), C, k, s, h, wd, ctypes.c_float(eps), _ptr(table))
    assert rc == 0
    xf = np.ascontiguousarray(x, np.float32)
    out = np.full((B, C, H * s, W * s), np.nan, np.float32)
    if strip2:
        rc = lib.emu_converse2d_strip2(_ptr(xf), _ptr(out), _ptr(table), _ptr(wf), B, C, H, W, k, s, p,
                                       PAD[mode], gelu, nthr)
    elif strip:
        rc = lib.emu_converse2d_strip(_ptr(xf), _ptr(out), _ptr(table), _ptr(wf), B, C, H, W, k, s, p,
                                      PAD[mode], gelu, nthr)
    else:
        rc = lib.emu_converse2d_fwd(_ptr(xf), _ptr(out), _ptr(table), _ptr(wf), B, C, H, W, k, s, p,
                                    PAD[mode], gelu, nthr, variant)
    assert rc == 0, rc
    return out


@pytest.mark.parametrize("i", range(20))
def test_emu_matches_reference_golden(emu, golden, i):
    c, x, w, b, ref32, ref64 = golden.case(i)
    out = emu_forward(emu, x, w, b, c["s"], c["p"], c["mode"], c["eps"], nthr=64 + 32 * (i % 3))
    assert np.isfinite(out).all()
    assert orc.rel_l2(out, ref64) <= 2e-5
    assert orc.rel_l2(out, ref32) <= 1e-4


@pytest.mark.parametrize("shape,k,s,p,mode", [
    ((2, 2, 64, 64), 5, 2, 2, "circular"),    # cfg-2 plane: compile-time plan 68 = 17*4
    ((3, 1, 64, 64), 5, 1, 2, "replicate"),   # odd batch: last pair has one plane
    ((1, 2, 30, 38), 5, 1, 2, "reflect"),     # 34 x 42 = (17*2) x (7*6)
    ((2, 1, 32, 40), 3, 3, 2, "constant"),    # 36 x 44 = (6*6) x (11*4)
])
def test_emu_static_plan_body(emu, shape, k, s, p, mode):
    rng = np.random.default_rng(7)
    x = rng.standard_normal(shape).astype(np.float32)
    w, b = orc.init_weight(shape[1], k, rng)
    b = (9.0 + rng.standard_normal(b.shape)).astype(np.float32)
    ref = orc.converse2d_forward(x, w, b, s, p, mode, 1e-5, dtype=np.float64)
    for variant in (0, 1, 2, 3):  # bit 0: compile-time plan body, bit 1: epilogue re-reads x instead of shared memory
        out = emu_forward(emu, x, w, b, s, p, mode, 1e-5, nthr=160, variant=variant)
        assert orc.rel_l2(out, ref) <= 2e-5, variant


@pytest.mark.parametrize("B,s", [(5, 2), (4, 1), (7, 2)])
def test_emu_persistent_body(emu, B, s):
    # blocks loop over plane pairs with the double-buffered staging of x (copies emulated by memcpy)
    rng = np.random.default_rng(B)
    x = rng.standard_normal((B, 3, 64, 64)).astype(np.float32)
    w, b = orc.init_weight(3, 5, rng)
    ref = orc.converse2d_forward(x, w, b, s, 2, "replicate", 1e-5, dtype=np.float64)
    out = emu_forward(emu, x, w, b, s, 2, "replicate", 1e-5, nthr=272, variant=4)
    assert orc.rel_l2(out, ref) <= 2e-5


@pytest.mark.parametrize("i", [0, 3, 5, 8, 11, 12, 13, 15, 16, 17])
def test_emu_strip_path_golden(emu, golden, i):
    # the multi-pass (workspace) path on the golden cases
    c, x, w, b, ref32, ref64 = golden.case(i)
    out = emu_forward(emu, x, w, b, c["s"], c["p"], c["mode"], c["eps"], nthr=64, strip=True)
    assert np.isfinite(out).all()
    assert orc.rel_l2(out, ref64) <= 2e-5


@pytest.mark.parametrize("shape,k,s,p,mode", [
    ((2, 2, 54, 82), 5, 1, 2, "circular"),    # 58 x 86 = (29*2) x (43*2): direct large-prime butterflies
    ((3, 1, 25, 33), 3, 2, 2, "replicate"),   # 29 x 37: prime lengths, upsampling epilogue with halo
    ((1, 2, 63, 30), 7, 1, 2, "reflect"),     # 67 x 34
])
def test_emu_strip_path_large_primes(emu, shape, k, s, p, mode):
    rng = np.random.default_rng(17)
    x = rng.standard_normal(shape).astype(np.float32)
    w, b = orc.init_weight(shape[1], k, rng)
    ref = orc.converse2d_forward(x, w, b, s, p, mode, 1e-5, dtype=np.float64)
    out = emu_forward(emu, x, w, b, s, p, mode, 1e-5, nthr=96, strip=True)     # Rader stages
    assert orc.rel_l2(out, ref) <= 3e-5
    out = emu_forward(emu, x, w, b, s, p, mode, 1e-5, nthr=-96, strip=True)    # direct O(R^2) butterflies
    assert orc.rel_l2(out, ref) <= 3e-5


@pytest.mark.parametrize("shape,k,s,p,mode", [
    ((3, 2, 30, 38), 5, 1, 2, "replicate"),   # 34 x 42: register radices, fused global stages
    ((2, 1, 30, 38), 3, 2, 2, "circular"),    # upsampling epilogue with halo columns
    ((3, 1, 54, 82), 5, 1, 2, "reflect"),     # 58 x 86: Rader first stages (29, 43)
    ((1, 2, 54, 82), 2, 2, 2, "replicate"),
])
def test_emu_strip_compile_time_axis_plans(emu, shape, k, s, p, mode):
    rng = np.random.default_rng(23)
    x = rng.standard_normal(shape).astype(np.float32)
    w, b = orc.init_weight(shape[1], k, rng)
    ref = orc.converse2d_forward(x, w, b, s, p, mode, 1e-5, dtype=np.float64)
    out = emu_forward(emu, x, w, b, s, p, mode, 1e-5, nthr=128, strip2=True)
    assert np.isfinite(out).all()
    assert orc.rel_l2(out, ref) <= 3e-5


def test_emu_gelu_epilogue(emu):
    from math import erf
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 2, 16, 18)).astype(np.float32)
    w, b = orc.init_weight(2, 3, rng)
    for s in (1, 2):
        ref = orc.converse2d_forward(x, w, b, s, 1, "circular", 1e-5, dtype=np.float64)
        ref = 0.5 * ref * (1.0 + np.vectorize(erf)(ref / np.sqrt(2.0)))
        out = emu_forward(emu, x, w, b, s, 1, "circular", 1e-5, gelu=1)
        assert orc.rel_l2(out, ref) <= 2e-5


@pytest.mark.parametrize("shape,k,s", [((2, 2, 20, 26), 5, 2), ((1, 3, 24, 24), 3, 1), ((1, 2, 18, 22), 2, 2),
                                       ((1, 2, 15, 20), 5, 3)])
def test_emu_x0_term_table(emu, shape, k, s):
    """Table of the arbitrary-x0 term: running the scale-1 forward with it must give
    IFFT2(FFT2(e) / (alias mean |FK|^2 + lambda)) (`models/util_converse.py:183-184`)."""
    rng = np.random.default_rng(41)
    B, C, h, wd = shape
    e = rng.standard_normal(shape).astype(np.float32)
    w, b = orc.init_weight(C, k, rng)
    b = (b + 0.5 * rng.standard_normal(b.shape)).astype(np.float32)
    table = np.zeros((C * h * wd + h + wd + 6 * 128, 2), np.float32)
    wf = np.ascontiguousarray(w.reshape(C, k, k), np.float32)
    bf = np.ascontiguousarray(b.reshape(C), np.float32)
    emu.emu_build_x0_table.restype = ctypes.c_int
    assert emu.emu_build_x0_table(_ptr(wf), _ptr(bf), C, k, s, h, wd, ctypes.c_float(1e-5), _ptr(table)) == 0
    out = np.full(shape, np.nan, np.float32)
    rc = emu.emu_converse2d_fwd(_ptr(e), _ptr(out), _ptr(table), _ptr(wf), B, C, h, wd, k, 1, 0, PAD["circular"],
                                0, 96, 0)
    assert rc == 0
    FB = orc.psf2otf(w.astype(np.float64), (h * s, wd * s))
    lam = orc.lam_from_bias(b.astype(np.float64), 1e-5, np.float64)
    ref = np.real(np.fft.ifft2(np.fft.fft2(e.astype(np.float64)) / (orc.block_mean(np.abs(FB) ** 2, s) + lam)))
    assert orc.rel_l2(out, ref) <= 2e-6


def test_emu_gelu_matches_the_erf_definition(emu):
    """The kernels' branch-free GELU against 0.5 x (1 + erf(x / sqrt 2)) in fp64 (`nn.GELU()` of
    `models/util_converse.py:280-287`): within the rounding of an fp32 result."""
    from math import erf, sqrt
    x = np.concatenate([np.linspace(-10, 10, 200001), np.array([0.0, -0.0, 1e-20, -1e-20, 30.0, -30.0])]).astype(np.float32)
    out = np.empty_like(x)
    assert emu.emu_gelu(_ptr(x), _ptr(out), x.size) == 0
    ref = np.array([0.5 * v * (1.0 + erf(v / sqrt(2.0))) for v in x.astype(np.float64)])
    assert np.abs(out - ref).max() <= 5e-7
    small = np.abs(x) < 1.0
    assert np.abs(out[small] - ref[small]).max() <= 1.2e-7
    assert np.all(out[x > 6] == x[x > 6]) and np.abs(out[x < -6]).max() < 1e-8


@pytest.mark.parametrize("shape,p,mode,nseg,direct", [
    ((3, 2, 30, 38), 2, "replicate", 2, 0),   # 34 x 42
    ((4, 1, 64, 64), 2, "circular", 1, 0),    # 68 x 68
    ((2, 2, 20, 26), 0, "circular", 2, 0),    # no padding
    ((5, 1, 32, 40), 2, "reflect", 3, 0),     # 36 x 44, uneven segments
    ((5, 2, 32, 40), 2, "reflect", 3, 1),     # the large-plane form: sums straight into one slab
])
def test_emu_cross_spectrum(emu, shape, p, mode, nseg, direct):
    # D[c] = sum_b FFT2(pad(x)) conj(FFT2(q)) in natural frequency order, the reduction behind dL/dweight
    rng = np.random.default_rng(31)
    B, C, H, W = shape
    h, w = H + 2 * p, W + 2 * p
    x = rng.standard_normal(shape).astype(np.float32)
    q = rng.standard_normal((B, C, h, w)).astype(np.float32)
    tw = np.zeros((h + w, 2), np.float32)
    for n, base in ((h, 0), (w, h)):
        a = 2.0 * np.pi * np.arange(n) / n
        tw[base:base + n, 0] = np.cos(a)
        tw[base:base + n, 1] = np.sin(a)
    out = np.zeros((1, C, h, w, 2), np.float32) if direct else np.full((nseg, C, h, w, 2), np.nan, np.float32)
    emu.emu_cross_spectrum.restype = ctypes.c_int
    rc = emu.emu_cross_spectrum(_ptr(x), _ptr(q), _ptr(tw), _ptr(out), nseg, B, C, H, W, p, PAD[mode], 96, direct)
    assert rc == 0
    got = (out[..., 0] + 1j * out[..., 1]).sum(0)
    y = orc.boundary_pad(x.astype(np.float64), p, mode) if p else x.astype(np.float64)
    ref = (np.fft.fft2(y) * np.conj(np.fft.fft2(q.astype(np.float64)))).sum(0)
    assert np.isfinite(out).all()
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 2e-5
