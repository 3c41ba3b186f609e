"""Caller-side data path against fixtures made with the reference's own helpers
(`tests/golden/make_image_golden.py`): conversions, PSNR, SSIM, wrap-around blur."""
import os

import numpy as np
import pytest
import torch

from conversenet_b200 import utils_image as ui

FIX = np.load(os.path.join(os.path.dirname(__file__), "golden", "image_ref_cases.npz"))
DEVICES = ["cpu"] + (["cuda"] if torch.cuda.is_available() else [])


@pytest.mark.parametrize("i", range(3))
def test_conversions(i):
    a = FIX["a%d" % i]
    assert np.array_equal(ui.uint2tensor4(a).numpy(), FIX["t4_%d" % i])
    f = torch.from_numpy(FIX["f%d" % i])
    assert np.array_equal(ui.tensor2uint(f), FIX["u8_%d" % i])
    back = ui.tensor2uint(ui.uint2tensor4(a))
    assert np.array_equal(back, a.squeeze())
    # batched forms agree with the per-image ones
    stack = np.stack([a, a[::-1].copy()])
    t = ui.batch_uint2tensor(stack)
    assert torch.equal(t[0:1], ui.uint2tensor4(a))
    assert torch.equal(ui.batch_tensor2uint(t)[1].permute(1, 2, 0).squeeze(), torch.from_numpy(a[::-1].copy()).squeeze())


@pytest.mark.parametrize("i", range(3))
@pytest.mark.parametrize("border", [0, 4])
def test_psnr_ssim_single_image_calling_convention(i, border):
    a, b = FIX["a%d" % i], FIX["b%d" % i]
    assert ui.calculate_psnr(a, b, border=border) == pytest.approx(float(FIX["psnr%d_%d" % (i, border)]), rel=1e-12)
    assert ui.calculate_ssim(a, b, border=border) == pytest.approx(float(FIX["ssim%d_%d" % (i, border)]), rel=1e-9)
    assert ui.calculate_psnr(a, a) == float("inf")
    with pytest.raises(ValueError):
        ui.calculate_psnr(a, b[:-1])


def _batched(device):
    # two RGB images of the same size in one batch
    a, b = FIX["a1"], FIX["b1"]
    ta = torch.from_numpy(np.stack([a, b])).permute(0, 3, 1, 2).to(device)
    tb = torch.from_numpy(np.stack([b, b])).permute(0, 3, 1, 2).to(device)
    return ta, tb


@pytest.mark.parametrize("device", ["cpu"])
def test_psnr_ssim_batched_cpu(device):
    ta, tb = _batched(device)
    p = ui.calculate_psnr(ta, tb, border=4)
    s = ui.calculate_ssim(ta, tb, border=4)
    assert p.shape == (2,) and s.shape == (2,)
    assert float(p[0]) == pytest.approx(float(FIX["psnr1_4"]), rel=1e-12) and float(p[1]) == float("inf")
    assert float(s[0]) == pytest.approx(float(FIX["ssim1_4"]), rel=1e-9) and float(s[1]) == pytest.approx(1.0)


@pytest.mark.gpu
def test_psnr_ssim_blur_on_the_gpu():
    ta, tb = _batched("cuda")
    p = ui.calculate_psnr(ta, tb, border=0)
    s = ui.calculate_ssim(ta, tb, border=0)
    assert p.is_cuda and s.is_cuda
    assert float(p[0]) == pytest.approx(float(FIX["psnr1_0"]), rel=1e-12)
    assert float(s[0]) == pytest.approx(float(FIX["ssim1_0"]), rel=1e-9)
    _check_blur("cuda")


def _check_blur(device):
    img = torch.from_numpy(FIX["blur_in"]).permute(2, 0, 1).unsqueeze(0).to(device)
    for kname, oname in (("blur_k", "blur_out"), ("blur_k2", "blur_out2")):   # odd and even kernel sizes
        k = torch.from_numpy(FIX[kname]).to(device)
        out = ui.circular_blur(img, k)[0].permute(1, 2, 0).cpu().numpy()
        assert np.abs(out - FIX[oname]).max() <= 1e-12
    # one kernel per image
    ks = torch.from_numpy(np.stack([FIX["blur_k"], FIX["blur_k"][::-1].copy()])).unsqueeze(1).to(device)
    two = ui.circular_blur(torch.cat([img, img]), ks)
    assert np.abs(two[0].permute(1, 2, 0).cpu().numpy() - FIX["blur_out"]).max() <= 1e-12
    assert not torch.allclose(two[0], two[1])


def test_blur_noise_downsample_cpu():
    _check_blur("cpu")
    g = torch.Generator().manual_seed(0)
    x = torch.zeros(2, 1, 64, 64)
    n = ui.add_gaussian_noise(x, 25 / 255.0, generator=g)
    assert abs(float(n.std()) - 25 / 255.0) < 2e-3
    assert ui.downsample(torch.arange(36.0).reshape(1, 1, 6, 6), 2).tolist() == [[[[0.0, 2.0, 4.0], [12.0, 14.0, 16.0],
                                                                                   [24.0, 26.0, 28.0]]]]
