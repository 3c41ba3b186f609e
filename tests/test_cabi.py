"""C-ABI checks that need no GPU: the library loads, exports what the header declares,
plans FFT lengths, and rejects bad arguments before touching the device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from conversenet_b200 import _cabi
    if not os.path.exists(_cabi.LIB_PATH):
        from conversenet_b200.build import build
        build(verbose=False)
    return _cabi.load()


def test_header_symbols_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "converse_b200.h")).read()
    names = sorted(set(re.findall(r"\b(cvb_[a-z0-9_]+)\s*\(", hdr)))
    assert len(names) >= 9
    from conversenet_b200 import _cabi
    for n in names:
        assert hasattr(lib, n), n
        assert n in _cabi.SIGNATURES, "binding table lacks " + n


def test_version_and_strerror(lib):
    assert lib.cvb_version() >= 100
    assert lib.cvb_strerror(0) == b"success"
    for code in range(-7, 0):
        assert len(lib.cvb_strerror(code)) > 5


@pytest.mark.parametrize("n,expect", [(68, [17, 4]), (132, [12, 11]), (136, [17, 8]), (512, [8, 8, 8]),
                                      (20, [20]), (44, [11, 4])])
def test_plans(lib, n, expect):
    r = (ctypes.c_int * 8)()
    k = lib.cvb_plan_radices(n, r, 8)
    assert list(r[:k]) == expect


def test_plan_products(lib):
    r = (ctypes.c_int * 8)()
    for n in range(2, 700):
        k = lib.cvb_plan_radices(n, r, 8)
        if k:
            prod = 1
            for v in r[:k]:
                prod *= v
            assert prod == n


def test_argument_validation_without_device(lib):
    one = ctypes.c_void_p(16)  # never dereferenced: validation fails first
    f = lib.cvb_converse2d_fwd
    # null input
    assert f(None, one, one, one, 1, 1, 8, 8, 3, 1, 1, 0, 0, 0, None, 0, None) == -1
    # circular padding wider than the plane
    assert f(one, one, one, one, 1, 1, 4, 4, 3, 1, 5, 0, 0, 0, None, 0, None) == -2
    # reflect padding must be smaller than the plane
    assert f(one, one, one, one, 1, 1, 4, 4, 3, 1, 4, 2, 0, 0, None, 0, None) == -2
    # unknown dtype
    assert f(one, one, one, one, 1, 1, 8, 8, 3, 1, 1, 0, 7, 0, None, 0, None) == -1
    # scale > 1 needs the taps
    assert f(one, one, one, None, 1, 1, 8, 8, 3, 2, 1, 0, 0, 0, None, 0, None) == -1
    assert lib.cvb_build_transfer(None, one, 1, 3, 1, 8, 8, 1e-5, one, None) == -1
    assert lib.cvb_build_transfer(one, one, 1, 9, 1, 8, 8, 1e-5, one, None) == -6
    # kernel_size above the 15 taps the table build keeps per thread: refused before any launch
    assert lib.cvb_build_transfer(one, one, 1, 17, 1, 32, 32, 1e-5, one, None) == -6
    assert lib.cvb_build_x0_table(one, one, 1, 17, 1, 32, 32, 1e-5, one, None) == -6
    assert lib.cvb_transfer_bytes(2, 68, 68) == (2 * 68 * 68 + 136) * 8
    assert lib.cvb_transfer_bytes(0, 68, 68) == 0


def test_module_mirror_cpu_behaviour():
    import torch
    from conversenet_b200 import Converse2D, ConverseBlock, ConverseBlockAlphaVariant
    m = Converse2D(3, 3, 5, scale=2, padding=2)
    assert tuple(m.weight.shape) == (1, 3, 5, 5) and tuple(m.bias.shape) == (1, 3, 1, 1)
    assert torch.allclose(m.weight.sum(dim=(-2, -1)), torch.ones(1, 3))
    assert float(m.bias.abs().sum()) == 0.0
    with pytest.raises(ValueError):
        Converse2D(3, 3, 5, backend="nope")
    with pytest.raises(AssertionError):
        Converse2D(3, 4, 5)
    with pytest.raises(RuntimeError):
        m(torch.zeros(1, 3, 8, 8))  # no CPU path: must fail loudly
    blk = ConverseBlock(4, 4, kernel_size=3)
    keys = set(blk.state_dict().keys())
    for k in ["conv1.0.weight", "conv1.1.weight", "conv1.3.weight", "conv1.3.bias", "conv1.5.bias",
              "conv2.0.bias", "conv2.1.weight", "conv2.3.weight"]:
        assert k in keys
    assert "alpha1" in ConverseBlockAlphaVariant(4, 4).state_dict()
