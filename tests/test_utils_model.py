"""Host logic of the test-time drivers (pad / split / x8), checked on CPU with small stand-in
models; the reference's own helpers are used as a second opinion when its tree is present."""
import os
import sys

import pytest
import torch
import torch.nn.functional as F

from conversenet_b200 import utils_model as um


def _img(h, w, b=2, c=3, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.rand(b, c, h, w, generator=g)


def test_symmetry_table_matches_rot90_definitions():
    x = _img(5, 7)
    want = [x, x.rot90(1, [2, 3]).flip([2]), x.flip([2]), x.rot90(3, [2, 3]), x.rot90(2, [2, 3]).flip([2]),
            x.rot90(1, [2, 3]), x.rot90(2, [2, 3]), x.rot90(3, [2, 3]).flip([2])]
    for mode in range(8):
        assert torch.equal(um.augment_img_tensor4(x, mode), want[mode]), mode


def test_every_symmetry_is_undone():
    x = _img(6, 9)
    for mode in range(8):
        back = um.augment_img_tensor4(um.augment_img_tensor4(x, mode), um._inverse_mode(mode))
        assert torch.equal(back, x), mode


def test_pad_crops_back_and_model_sees_multiples():
    seen = []

    def model(t):
        seen.append(tuple(t.shape[-2:]))
        return F.interpolate(t, scale_factor=2, mode="nearest")

    x = _img(13, 18)
    out = um.test_pad(model, x, modulo=8, sf=2)
    assert seen == [(16, 24)]
    assert out.shape == (2, 3, 26, 36)
    assert torch.equal(out, F.interpolate(x, scale_factor=2, mode="nearest"))


@pytest.mark.parametrize("sf", [1, 2])
@pytest.mark.parametrize("hw", [(40, 56), (70, 45), (96, 96)])
def test_split_of_a_pointwise_model_is_exact(hw, sf):
    def model(t):
        y = 2.0 * t + 1.0
        return F.interpolate(y, scale_factor=sf, mode="nearest") if sf > 1 else y

    x = _img(*hw)
    out = um.test_split(model, x, refield=8, min_size=16, sf=sf)
    assert torch.equal(out, model(x))


def test_split_respects_the_receptive_field():
    # 3x3 box filter with zero padding: quadrants overlap by >= refield, so interior seams are exact
    k = torch.ones(3, 1, 3, 3) / 9.0

    def model(t):
        return F.conv2d(t, k, padding=1, groups=3)

    x = _img(48, 64)
    out = um.test_split(model, x, refield=8, min_size=24)
    assert torch.allclose(out, model(x), atol=1e-6)


def test_x8_of_an_equivariant_model_is_the_model():
    k = torch.tensor([[1.0, 2.0, 1.0], [2.0, 4.0, 2.0], [1.0, 2.0, 1.0]]).repeat(3, 1, 1, 1) / 16.0

    def model(t):  # symmetric kernel, circular padding: commutes with all eight symmetries
        return F.conv2d(F.pad(t, (1, 1, 1, 1), mode="circular"), k, groups=3)

    x = _img(12, 20)
    assert torch.allclose(um.test_x8(model, x), model(x), atol=1e-6)
    assert torch.allclose(um.test_split_x8(model, x, refield=4, min_size=64), model(x), atol=1e-6)


def test_mode_dispatch_and_bad_mode():
    x = _img(8, 8)
    model = lambda t: t + 1.0
    for mode in range(5):
        assert torch.equal(um.test_mode(model, x, mode=mode, refield=4, min_size=4), x + 1.0) or mode in (3, 4)
    assert torch.allclose(um.test_mode(model, x, mode=3), x + 1.0)
    with pytest.raises(ValueError):
        um.test_mode(model, x, mode=7)


def test_against_the_reference_helpers_when_present():
    from oracle.build_ref import default_reference_root
    ref_root = default_reference_root()
    if not os.path.isdir(os.path.join(ref_root, "utils")):
        pytest.skip("reference tree not present")
    sys.path.insert(0, ref_root)
    try:
        sys.dont_write_bytecode = True
        import types
        for name in ("matplotlib", "matplotlib.pyplot", "mpl_toolkits", "mpl_toolkits.mplot3d"):
            if name not in sys.modules:   # plotting is not used by the helpers under test
                try:
                    __import__(name)
                except Exception:
                    mod = types.ModuleType(name)
                    mod.Axes3D = object
                    sys.modules[name] = mod
        from utils import utils_model as ref  # noqa
    except Exception as e:  # missing optional dependency of the reference's image helpers
        pytest.skip("reference helpers not importable: %s" % e)
    finally:
        sys.path.remove(ref_root)
    k = torch.rand(3, 1, 5, 5, generator=torch.Generator().manual_seed(3))

    def model(t):
        return F.interpolate(F.conv2d(t, k, padding=2, groups=3), scale_factor=2, mode="nearest")

    x = _img(50, 38, seed=4)
    for mode in range(5):
        a = um.test_mode(model, x, mode=mode, refield=8, min_size=16, sf=2, modulo=4)
        b = ref.test_mode(model, x, mode=mode, refield=8, min_size=16, sf=2, modulo=4)
        assert a.shape == b.shape
        assert torch.allclose(a, b, atol=1e-6), mode


@pytest.mark.gpu
def test_x8_on_the_cuda_layer_with_non_square_planes():
    """A Converse2D layer whose taps are invariant under the eight symmetries (odd kernel,
    circular padding) commutes with them, so the x8 ensemble must reproduce the plain output;
    half of the eight runs see the transposed, H != W plane."""
    from conversenet_b200 import Converse2D
    torch.manual_seed(7)
    layer = Converse2D(8, 8, 5, scale=1, padding=2, padding_mode="circular").cuda().eval()
    w = layer.weight.data
    sym = sum(um.augment_img_tensor4(w, m) for m in range(8)) / 8.0
    layer.weight.data.copy_(sym)
    x = torch.rand(2, 8, 40, 56, device="cuda")
    with torch.no_grad():
        plain = layer(x)
        ens = um.test_x8(layer, x)
        split = um.test_split_x8(layer, x, refield=8, min_size=64)
    rel = lambda a, b: ((a - b).norm() / b.norm()).item()
    assert rel(ens, plain) < 1e-5            # fp32 round-off of eight differently ordered runs
    assert split.shape == plain.shape
