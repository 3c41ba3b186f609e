"""Restatement of the reference's networks in plain torch ops.  TEST INFRASTRUCTURE ONLY.

The reference's Python package cannot travel to a machine that has no checkout of it, so
the network wiring is restated here, layer by layer, with the same state-dict keys:

  * `solve`              -- the closed-form solve of `models/util_converse.py:171-187`
                            (= `Converse2D/torch_converse2d/converse2d.cpp:186-207`) in torch.fft;
                            when `oracle/_ref/converse2d_ref.so` (the reference's own C++ op,
                            compiled by oracle/build_ref.py) has been loaded, the shared-kernel
                            case calls that op instead (`use_reference_op`)
  * `RefConverse2D`      -- `models/util_converse.py:98-192` (pad, x0, solve, crop)
  * `RefLayerNorm`       -- `models/util_converse.py:42-68`, channels_first
  * `RefBlock`           -- `models/util_converse.py:253-323` (alpha=True: the alpha variant)
  * `RefDnCNN`           -- `models/converse_dncnn.py:11-35`
  * `RefSRResNet`        -- `models/converse_srresnet.py:50-80`
  * `RefDataNet`, `RefKernelNet`, `RefUSRNet`, `RefConverseNet`
                         -- `models/converse_usrnet.py:33-68,125-142,150-169,178-214`

Uses: the CPU baseline of the benchmark (the networks on the host cores), the library
baseline (the same modules on CUDA tensors: cuFFT + ATen, what the reference's PyTorch
path does on a GPU), and as a second checker next to the stored outputs of the unmodified
reference (`tests/golden/model_fullsize_cases.npz`).  tests/test_ref_networks.py pins every
class here to the imported reference (bit-identical on CPU) where the checkout exists, and
to the stored outputs everywhere.  Nothing in the shipped package imports this file.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

_use_ref_op = False


def use_reference_op(flag=True):
    """Route `solve` with a shared kernel through `torch.ops.converse2d.forward` (the
    reference's C++ op, which the caller has loaded from oracle/_ref)."""
    global _use_ref_op
    _use_ref_op = bool(flag) and hasattr(torch.ops, "converse2d") and hasattr(torch.ops.converse2d, "forward")
    return _use_ref_op


def _splits_mean(a, s):
    # mean over the s*s aliases: out[u, v] = mean a[u + i*h, v + j*w]  (`util_converse.py:182-183,194-215`)
    *lead, Nh, Nw = a.shape
    return a.reshape(*lead, s, Nh // s, s, Nw // s).mean(dim=(-4, -2))


def _p2o(psf, shape):
    # `util_converse.py:218-235`
    otf = torch.zeros(psf.shape[:-2] + tuple(shape), dtype=psf.dtype, device=psf.device)
    otf[..., :psf.shape[-2], :psf.shape[-1]] = psf
    otf = torch.roll(otf, (-int(psf.shape[-2] / 2), -int(psf.shape[-1] / 2)), dims=(-2, -1))
    return torch.fft.fftn(otf, dim=(-2, -1))


def solve(y, x0, weight, lam, s):
    """Uncropped closed-form solve on a padded plane; `weight` (1 or B, C, k, k), `lam` (1,C,1,1)."""
    B, C, h, w = y.shape
    STy = torch.zeros((B, C, h * s, w * s), dtype=y.dtype, device=y.device)
    STy[..., ::s, ::s] = y
    FB = _p2o(weight, (h * s, w * s))
    FBC = torch.conj(FB)
    F2B = torch.abs(FB) ** 2
    FR = FBC * torch.fft.fftn(STy, dim=(-2, -1)) + torch.fft.fftn(lam * x0, dim=(-2, -1))
    x1 = FB * FR
    invWBR = _splits_mean(x1, s) / (_splits_mean(F2B, s) + lam)
    FX = (FR - FBC * invWBR.repeat(1, 1, s, s)) / lam
    return torch.real(torch.fft.ifftn(FX, dim=(-2, -1)))


class RefConverse2D(nn.Module):
    def __init__(self, channels, kernel_size, scale=1, padding=2, padding_mode="circular", eps=1e-5):
        super().__init__()
        self.kernel_size, self.scale, self.padding = kernel_size, scale, padding
        self.padding_mode, self.eps = padding_mode, eps
        w = torch.randn(1, channels, kernel_size, kernel_size)
        self.weight = nn.Parameter(F.softmax(w.view(1, channels, -1), dim=-1).view_as(w))
        self.bias = nn.Parameter(torch.zeros(1, channels, 1, 1))

    def forward(self, x):
        p, s = self.padding, self.scale
        y = F.pad(x, [p, p, p, p], mode=self.padding_mode) if p > 0 else x
        x0 = y if s == 1 else F.interpolate(y, scale_factor=s, mode="nearest")
        if _use_ref_op:
            out = torch.ops.converse2d.forward(y, x0, self.weight, self.bias, int(s), float(self.eps))
        else:
            out = solve(y, x0, self.weight, torch.sigmoid(self.bias - 9.0) + self.eps, s)
        return out[..., p * s:-p * s, p * s:-p * s] if p > 0 else out


class RefLayerNorm(nn.Module):
    def __init__(self, channels, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(channels))
        self.bias = nn.Parameter(torch.zeros(channels))
        self.eps = eps

    def forward(self, x):
        u = x.mean(1, keepdim=True)
        v = (x - u).pow(2).mean(1, keepdim=True)
        x = (x - u) / torch.sqrt(v + self.eps)
        return self.weight[:, None, None] * x + self.bias[:, None, None]


class RefBlock(nn.Module):
    def __init__(self, c, kernel_size=3, padding=2, padding_mode="replicate", eps=1e-5, alpha=False):
        super().__init__()
        self.conv1 = nn.Sequential(RefLayerNorm(c), nn.Conv2d(c, 2 * c, 1), nn.GELU(),
                                   RefConverse2D(2 * c, kernel_size, 1, padding, padding_mode, eps), nn.GELU(),
                                   nn.Conv2d(2 * c, c, 1))
        self.conv2 = nn.Sequential(RefLayerNorm(c), nn.Conv2d(c, 2 * c, 1), nn.GELU(), nn.Conv2d(2 * c, c, 1))
        if alpha:
            self.alpha1 = nn.Parameter(torch.zeros(1, c, 1, 1))
            self.alpha2 = nn.Parameter(torch.zeros(1, c, 1, 1))
        self.has_alpha = alpha

    def forward(self, x):
        if self.has_alpha:
            x = self.alpha1 * self.conv1(x) + x
            return self.alpha2 * self.conv2(x) + x
        x = self.conv1(x) + x
        return self.conv2(x) + x


class RefDnCNN(nn.Module):
    def __init__(self):
        super().__init__()
        self.m_head = nn.Sequential(nn.Conv2d(1, 64, 1))
        self.m_body = nn.Sequential(*[RefBlock(64, 7, 6, "circular") for _ in range(20)])
        self.m_tail = nn.Sequential(nn.Conv2d(64, 1, 1))

    def forward(self, x):
        return self.m_tail(self.m_body(self.m_head(x)))


class RefSRResNet(nn.Module):
    def __init__(self):
        super().__init__()
        blk = lambda: RefBlock(64, 5, 4, "replicate")
        self.conv_first = nn.Conv2d(3, 64, 1)
        self.conv_body = nn.Sequential(*[blk() for _ in range(16)])
        self.upconv1 = blk()
        self.up1 = RefConverse2D(64, 2, 2, 2, "replicate", 1e-3)
        self.upconv2 = blk()
        self.up2 = RefConverse2D(64, 2, 2, 2, "replicate", 1e-3)
        self.conv_hres = blk()
        self.conv_last = nn.Conv2d(64, 3, 1, bias=False)
        self.gelu = nn.GELU()

    def forward(self, x):
        x1 = self.conv_body(self.gelu(self.conv_first(x)))
        x1 = self.gelu(self.up1(self.upconv1(x1)))
        x1 = self.gelu(self.up2(self.upconv2(x1)))
        x1 = self.conv_last(self.gelu(self.conv_hres(x1)))
        return x1 + F.interpolate(x, scale_factor=4, mode="bilinear", align_corners=False)


class RefDataNet(nn.Module):
    def __init__(self, eps=1e-3):
        super().__init__()
        self.alpha = nn.Parameter(torch.zeros(1, 64, 1, 1))
        self.eps = eps

    def forward(self, x, k, sf):
        lam = torch.sigmoid(self.alpha - 9.0) + self.eps
        x0 = x if sf == 1 else F.interpolate(x, scale_factor=sf, mode="nearest")
        return solve(x, x0, k, lam, int(sf))


class RefKernelNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1, self.fc2, self.fc3 = nn.Linear(49, 64), nn.Linear(64, 64), nn.Linear(64, 16 * 49)
        self.gelu = nn.GELU()

    def forward(self, k):
        b = k.shape[0]
        k = k.to(self.fc1.weight.dtype).view(b, -1)
        return self.fc3(self.gelu(self.fc2(self.gelu(self.fc1(k))))).view(b, 16, 7, 7)


class _Body(nn.Module):
    def __init__(self, alpha):
        super().__init__()
        self.m_body = nn.Sequential(*[RefBlock(64, 3, 2, "circular", alpha=alpha) for _ in range(7)])

    def forward(self, x):
        return self.m_body(x)


class RefConverseNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.p = _Body(False)
        self.conv1, self.conv2 = nn.Conv2d(3, 64, 1), nn.Conv2d(64, 3, 1)

    def forward(self, x):
        x = self.conv1(x)
        for _ in range(5):
            x = self.p(x)
        return self.conv2(x)


class RefUSRNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.d = RefDataNet()
        self.p = _Body(True)
        self.conv1, self.conv2 = nn.Conv2d(3, 64, 1), nn.Conv2d(64, 3, 1)
        self.kernelnet = RefKernelNet()
        self.convs = nn.ModuleList([nn.Conv2d(16, 64, 1) for _ in range(5)])

    def forward(self, x, k, sf):
        b, _, h, w = k.shape
        k = self.kernelnet(k)
        x = self.conv1(x)
        x = self.p(self.d(x, self.convs[0](k).view(b, 64, h, w), sf))
        for i in range(1, 5):
            x = self.p(self.d(x, self.convs[i](k).view(b, 64, h, w), 1))
        return self.conv2(x)


NETWORKS = {"dncnn": RefDnCNN, "srresnet": RefSRResNet, "usrnet": RefUSRNet, "conversenet": RefConverseNet}
