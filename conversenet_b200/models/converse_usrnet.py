"""Converse-USRNet / ConverseNet (`models/converse_usrnet.py`)."""
import torch
import torch.nn as nn

from .. import functional as CF
from ..util_converse import sequential, ConverseBlock, ConverseBlockAlphaVariant


class MultiConverseBlock(nn.Module):
    def __init__(self, in_channels=64, num_blocks=7, kernel_size=3, scale=1, padding=2, padding_mode="circular"):
        super().__init__()
        self.m_body = sequential(*[ConverseBlock(in_channels, in_channels, kernel_size, scale, padding, padding_mode)
                                   for _ in range(num_blocks)])

    def forward(self, x):
        return self.m_body(x)


class MultiConverseBlockAlphaVariant(nn.Module):
    def __init__(self, in_channels=64, num_blocks=7, kernel_size=3, scale=1, padding=2, padding_mode="circular"):
        super().__init__()
        self.m_body = sequential(*[ConverseBlockAlphaVariant(in_channels, in_channels, kernel_size, scale, padding,
                                                             padding_mode) for _ in range(num_blocks)])

    def forward(self, x):
        return self.m_body(x)


class ConvReverseDataNet(nn.Module):
    """Data step of USRNet (`models/converse_usrnet.py:33-68`): the Converse2D solve with a
    different k x k kernel per (sample, channel) and lambda from `alpha (1,64,1,1)`.

    Every (sample, channel) plane has its own transfer table, so the planes are handed to
    the kernels as one batch entry with B*C channels."""

    def __init__(self, eps=1e-3):
        super().__init__()
        self.alpha = nn.Parameter(torch.zeros(1, 64, 1, 1))
        self.eps = eps

    def forward(self, x, k, sf, padding=0, padding_mode="circular"):
        if not x.is_cuda:
            raise RuntimeError("ConvReverseDataNet needs CUDA tensors; this build has no CPU path")
        B, C, H, W = x.shape
        if k.dim() != 4 or k.size(0) != B or k.size(1) != C or k.size(2) != k.size(3):
            raise RuntimeError("k must be (B,C,kh,kh) matching x")
        self.biaseps = torch.sigmoid(self.alpha.detach() - 9.0) + self.eps
        ks = k.size(2)
        h, w = H + 2 * padding, W + 2 * padding
        weight = k.reshape(1, B * C, ks, ks)
        bias = self.alpha.expand(B, C, 1, 1).reshape(1, B * C, 1, 1)
        table, wf = CF.build_transfer(weight, bias, int(sf), self.eps, h, w)
        planes = x.reshape(1, B * C, H, W)
        if torch.is_grad_enabled() and (x.requires_grad or k.requires_grad or self.alpha.requires_grad):
            # differentiable in x, the kernels and alpha, as the reference's torch.fft data step is
            # (`models/converse_usrnet.py:41-68`)
            from ..autograd import Converse2DFunction
            out = Converse2DFunction.apply(planes, weight, bias, table, wf, ks, int(sf), padding, padding_mode,
                                           self.eps)
        else:
            out = CF.converse2d_forward(planes, table, wf, ks, int(sf), padding, padding_mode)
        return out.reshape(B, C, H * int(sf), W * int(sf))


class KernelNet(nn.Module):
    """MLP 49 -> 64 -> 64 -> 16*49 on the flattened blur kernel (`models/converse_usrnet.py:125-142`)."""

    def __init__(self, kernel_size=7):
        super().__init__()
        self.kernel_size = kernel_size
        self.fc1 = nn.Linear(kernel_size ** 2, 64)
        self.fc2 = nn.Linear(64, 64)
        self.fc3 = nn.Linear(64, 16 * (kernel_size ** 2))
        self.gelu = nn.GELU()

    def forward(self, k):
        k = k.to(torch.float)
        b = k.shape[0]
        k = k.view(b, -1)
        k = self.gelu(self.fc1(k))
        k = self.gelu(self.fc2(k))
        k = self.fc3(k)
        return k.view(b, 16, self.kernel_size, self.kernel_size)


class ConverseNet(nn.Module):
    """Blind variant: 1x1, `num_iterations` passes through the same 7 blocks, 1x1
    (`models/converse_usrnet.py:150-169`)."""

    def __init__(self, num_iterations=5, in_channels=64, num_blocks=7):
        super().__init__()
        self.p = MultiConverseBlock(in_channels=in_channels, num_blocks=num_blocks)
        self.conv1 = nn.Conv2d(3, in_channels, 1, 1, 0)
        self.conv2 = nn.Conv2d(in_channels, 3, 1, 1, 0)
        self.num_iterations = num_iterations

    def forward(self, x):
        x = self.conv1(x)
        for _ in range(self.num_iterations):
            x = self.p(x)
        return self.conv2(x)


class ConverseUSRNet(nn.Module):
    """Non-blind deblurring / SR (`models/converse_usrnet.py:178-214`): kernel MLP, then
    `num_iterations` x [data step with per-sample kernels, 7 shared alpha-variant blocks]."""

    def __init__(self, num_iterations=5, in_channels=64, num_blocks=7):
        super().__init__()
        self.d = ConvReverseDataNet()
        self.p = MultiConverseBlockAlphaVariant(in_channels=in_channels, num_blocks=num_blocks)
        self.conv1 = nn.Conv2d(3, 64, 1, 1, 0)
        self.conv2 = nn.Conv2d(64, 3, 1, 1, 0)
        self.kernelnet = KernelNet()
        self.num_iterations = num_iterations
        self.convs = nn.ModuleList([nn.Conv2d(16, 64, 1, 1, 0) for _ in range(num_iterations)])

    def forward(self, x, k, sf):
        b, c, h, w = k.shape
        k = self.kernelnet(k)
        x = self.conv1(x)
        x = self.d(x, self.convs[0](k).view(b, 64, h, w), sf)
        x = self.p(x)
        for i in range(1, self.num_iterations):
            x = self.d(x, self.convs[i](k).view(b, 64, h, w), 1)
            x = self.p(x)
        return self.conv2(x)
