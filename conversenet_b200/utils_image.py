"""Caller-side data path of the test scripts as batched tensor ops: uint8 <-> float tensors,
degradations, PSNR and SSIM.

Same names and numbers as the reference's per-image numpy / OpenCV helpers
(`utils/utils_image.py:293-313` conversions, `:626-694` PSNR / SSIM;
`main_test_converse_dncnn.py:120-127` noise, `main_test_converse_usrnet.py:141-143` blur and
decimation), but every function also takes a (B,C,H,W) tensor on any device and then returns one
value per image, so that a whole test set is scored without leaving the GPU.  Metrics are
evaluated in float64.
"""
import math

import numpy as np
import torch
import torch.nn.functional as F


# ---- uint8 / float arrays <-> tensors -------------------------------------------------
def uint2single(img):
    return np.float32(img / 255.0)


def single2uint(img):
    return np.uint8((img.clip(0, 1) * 255.0).round())


def uint2tensor4(img):
    """HxW or HxWxC uint8 array -> (1,C,H,W) float tensor in [0,1]."""
    if img.ndim == 2:
        img = np.expand_dims(img, axis=2)
    return torch.from_numpy(np.ascontiguousarray(img)).permute(2, 0, 1).float().div(255.0).unsqueeze(0)


def single2tensor4(img):
    """HxW or HxWxC float array -> (1,C,H,W) float tensor."""
    if img.ndim == 2:
        img = np.expand_dims(img, axis=2)
    return torch.from_numpy(np.ascontiguousarray(img)).permute(2, 0, 1).float().unsqueeze(0)


def tensor2single(img):
    img = img.detach().squeeze().float().cpu().numpy()
    if img.ndim == 3:
        img = np.transpose(img, (1, 2, 0))
    return img


def tensor2uint(img):
    """2/3/4-dimensional tensor in [0,1] -> uint8 array (HxW or HxWxC); rounds half to even as numpy does."""
    img = img.detach().squeeze().float().clamp(0, 1).cpu().numpy()
    if img.ndim == 3:
        img = np.transpose(img, (1, 2, 0))
    return np.uint8((img * 255.0).round())


def batch_uint2tensor(imgs, device=None):
    """(B,H,W) or (B,H,W,C) uint8 array -> (B,C,H,W) float tensor in [0,1] on `device`."""
    t = torch.from_numpy(np.ascontiguousarray(imgs))
    if t.dim() == 3:
        t = t.unsqueeze(-1)
    t = t.permute(0, 3, 1, 2)
    if device is not None:
        t = t.to(device, non_blocking=True)
    return t.float().div(255.0)


def batch_tensor2uint(t):
    """(B,C,H,W) tensor in [0,1] -> (B,C,H,W) uint8 tensor on the same device (round half to even)."""
    return (t.detach().float().clamp(0, 1) * 255.0).round().to(torch.uint8)


# ---- degradations ---------------------------------------------------------------------
def add_gaussian_noise(img, sigma, generator=None):
    """img + N(0, sigma^2) with sigma on the [0,1] scale (`noise_level_img / 255`)."""
    noise = torch.randn(img.shape, dtype=img.dtype, device=img.device, generator=generator)
    return img + sigma * noise


def circular_blur(img, kernel):
    """Convolution of every channel with `kernel` (kh,kw) or one kernel per image (B,1,kh,kw), wrap-around
    boundary: `scipy.ndimage.convolve(img, k[..., None], mode='wrap')` of the USRNet script."""
    B, C, H, W = img.shape
    k = kernel if kernel.dim() == 4 else kernel.reshape(1, 1, *kernel.shape[-2:]).expand(B, 1, -1, -1)
    kh, kw = k.shape[-2:]
    # ndimage's origin: the kernel centre sits at index size // 2; convolution = correlation with the flip
    ph, pw = kh // 2, kw // 2
    x = F.pad(img, (kw - 1 - pw, pw, kh - 1 - ph, ph), mode="circular")
    wgt = k.flip(-2, -1).to(img.dtype).repeat_interleave(C, dim=0)          # (B*C,1,kh,kw)
    out = F.conv2d(x.reshape(1, B * C, *x.shape[-2:]), wgt, groups=B * C)
    return out.reshape(B, C, H, W)


def downsample(img, sf):
    """s-fold decimation from phase 0 (`img[0::sf, 0::sf]`)."""
    return img[..., 0::sf, 0::sf]


# ---- metrics --------------------------------------------------------------------------
def _as_batch(img):
    """numpy HxW / HxWxC (one image, the reference's calling convention) or (B,C,H,W) tensor ->
    (B,C,H,W) float64 tensor, and whether the caller passed a single array."""
    if isinstance(img, np.ndarray):
        a = torch.from_numpy(np.ascontiguousarray(img)).double()
        if a.dim() == 2:
            a = a.unsqueeze(-1)
        return a.permute(2, 0, 1).unsqueeze(0), True
    if img.dim() != 4:
        raise ValueError("tensors must be (B,C,H,W)")
    return img.double(), False


def _crop(a, border):
    h, w = a.shape[-2:]
    return a[..., border:h - border, border:w - border]


def calculate_psnr(img1, img2, border=0):
    """PSNR on the [0,255] scale.  One array pair -> float; tensors -> (B,) float64 tensor."""
    a, single = _as_batch(img1)
    b, _ = _as_batch(img2)
    if a.shape != b.shape:
        raise ValueError("Input images must have the same dimensions.")
    mse = ((_crop(a, border) - _crop(b, border)) ** 2).mean(dim=(1, 2, 3))
    psnr = torch.where(mse == 0, torch.full_like(mse, float("inf")), 20.0 * torch.log10(255.0 / mse.sqrt()))
    return float(psnr[0]) if single else psnr


def _gaussian_window(dtype, device):
    g = torch.tensor([math.exp(-((i - 5) ** 2) / (2.0 * 1.5 ** 2)) for i in range(11)], dtype=dtype, device=device)
    return g / g.sum()


def calculate_ssim(img1, img2, border=0):
    """SSIM on the [0,255] scale with the 11-tap sigma-1.5 Gaussian window over the valid region, averaged over
    channels (MATLAB's definition, as the reference's).  One array pair -> float; tensors -> (B,) tensor."""
    a, single = _as_batch(img1)
    b, _ = _as_batch(img2)
    if a.shape != b.shape:
        raise ValueError("Input images must have the same dimensions.")
    a, b = _crop(a, border), _crop(b, border)
    if a.size(1) not in (1, 3):
        raise ValueError("Wrong input image dimensions.")
    B, C, H, W = a.shape
    g = _gaussian_window(a.dtype, a.device)

    def blur(t):   # separable, valid
        t = t.reshape(B * C, 1, H, W)
        t = F.conv2d(t, g.view(1, 1, 11, 1))
        t = F.conv2d(t, g.view(1, 1, 1, 11))
        return t.reshape(B, C, H - 10, W - 10)

    C1, C2 = (0.01 * 255) ** 2, (0.03 * 255) ** 2
    mu1, mu2 = blur(a), blur(b)
    s1 = blur(a * a) - mu1 * mu1
    s2 = blur(b * b) - mu2 * mu2
    s12 = blur(a * b) - mu1 * mu2
    smap = ((2 * mu1 * mu2 + C1) * (2 * s12 + C2)) / ((mu1 * mu1 + mu2 * mu2 + C1) * (s1 + s2 + C2))
    val = smap.mean(dim=(2, 3)).mean(dim=1)
    return float(val[0]) if single else val
