"""Drop-in for the reference's `models/util_converse.py`: same class names, constructor
signatures, parameter names/shapes and forward semantics; the arithmetic runs in
hand-written sm_100a kernels behind the C ABI.  Forward only."""
import os
from collections import OrderedDict

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import functional as CF


# False: ConverseBlock runs its layers one by one (PyTorch LayerNorm / 1x1 / GELU around the native
# operator) instead of the fused block kernels; the tests compare the two.
BLOCK_FUSION = True


class _exact_fp32:
    """PyTorch's 1x1 convolutions (cuDNN / cuBLAS) in full fp32 for a block of code.  The unfused route of
    ConverseBlock (channel counts other than 64, or autograd) must hold the operator's 1e-4 bar, which
    TF32 (10-bit mantissa, on by default for cuDNN convolutions) does not."""

    def __enter__(self):
        self.saved = (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32)
        torch.backends.cudnn.allow_tf32 = False
        torch.backends.cuda.matmul.allow_tf32 = False

    def __exit__(self, *exc):
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = self.saved
        return False


class LayerNorm(nn.Module):
    """channels_last / channels_first LayerNorm (`models/util_converse.py:42-68`)."""

    def __init__(self, normalized_shape, eps=1e-6, data_format="channels_last"):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(normalized_shape))
        self.bias = nn.Parameter(torch.zeros(normalized_shape))
        self.eps = eps
        self.data_format = data_format
        if self.data_format not in ["channels_last", "channels_first"]:
            raise NotImplementedError
        self.normalized_shape = (normalized_shape,)

    def forward(self, x):
        if self.data_format == "channels_last":
            return F.layer_norm(x, self.normalized_shape, self.weight, self.bias, self.eps)
        u = x.mean(1, keepdim=True)
        s = (x - u).pow(2).mean(1, keepdim=True)
        x = (x - u) / torch.sqrt(s + self.eps)
        return self.weight[:, None, None] * x + self.bias[:, None, None]


def sequential(*args):
    """Flattening `nn.Sequential` builder (`models/util_converse.py:71-91`)."""
    if len(args) == 1:
        if isinstance(args[0], OrderedDict):
            raise NotImplementedError("sequential does not support OrderedDict input.")
        return args[0]
    modules = []
    for module in args:
        if isinstance(module, nn.Sequential):
            modules.extend(module.children())
        elif isinstance(module, nn.Module):
            modules.append(module)
    return nn.Sequential(*modules)


class Converse2D(nn.Module):
    """Depthwise reverse convolution (`models/util_converse.py:98-192`).

    `Converse2D(in_channels, out_channels, kernel_size, scale=1, padding=2,
    padding_mode='circular', eps=1e-5, backend='auto')`, parameters
    `weight (1,C,k,k)` (softmax-normalised normal draw) and `bias (1,C,1,1)`
    (zeros), `forward(x: (B,C,H,W)) -> (B,C,H*scale,W*scale)`.

    With autograd enabled and an input or parameter that requires a gradient the call is
    differentiable (`conversenet_b200/autograd.py`: dL/dx through the native kernels).

    `backend` is accepted for compatibility: 'auto' and 'cuda' run the native
    kernels; 'pytorch' (or CONVERSE2D_BACKEND=pytorch) raises, because this build
    carries no torch.fft path.  The output is contiguous (the reference returns a
    cropped view)."""

    _TABLE_SLOTS = 8

    def __init__(self, in_channels, out_channels, kernel_size, scale=1, padding=2, padding_mode="circular",
                 eps=1e-5, backend="auto"):
        super().__init__()
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = kernel_size
        self.scale = scale
        self.padding = padding
        self.padding_mode = padding_mode
        self.eps = eps
        self.backend = backend.lower()
        if self.backend not in ("auto", "cuda", "pytorch"):
            raise ValueError(f"backend must be 'auto' | 'cuda' | 'pytorch', got: {self.backend}")
        assert self.out_channels == self.in_channels  # depthwise
        self.weight = nn.Parameter(torch.randn(1, self.in_channels, self.kernel_size, self.kernel_size))
        self.bias = nn.Parameter(torch.zeros(1, self.in_channels, 1, 1))
        self.weight.data = F.softmax(self.weight.data.view(1, self.in_channels, -1), dim=-1).view(
            1, self.in_channels, self.kernel_size, self.kernel_size)
        self._tables = OrderedDict()
        self.fuse_gelu = False  # set by ConverseBlock: apply the following GELU inside the kernel

    # -- transfer-table cache: rebuilt when a parameter is modified in place or replaced
    def _table_for(self, h, w, device):
        key = (h, w, device, self.weight.data_ptr(), self.bias.data_ptr(), self.weight._version,
               self.bias._version, int(self.scale), float(self.eps))
        hit = self._tables.get(key)
        if hit is not None:
            self._tables.move_to_end(key)
            return hit
        table, wf = CF.build_transfer(self.weight, self.bias, self.scale, self.eps, h, w)
        self.biaseps = torch.sigmoid(self.bias.detach() - 9.0) + self.eps
        self._tables[key] = (table, wf)
        while len(self._tables) > self._TABLE_SLOTS:
            self._tables.popitem(last=False)
        return table, wf

    def clear_cache(self):
        self._tables.clear()

    def forward(self, x):
        backend = (os.environ.get("CONVERSE2D_BACKEND", "") or self.backend).lower()
        if backend == "pytorch":
            raise RuntimeError("Converse2D backend='pytorch' is not available: this build only has the "
                               "native sm_100a path")
        if backend not in ("auto", "cuda"):
            raise ValueError(f"backend must be 'auto' | 'cuda' | 'pytorch', got: {backend}")
        if not x.is_cuda:
            raise RuntimeError("Converse2D backend='cuda' but the input is not a CUDA tensor.")
        if x.dim() != 4 or x.size(1) != self.in_channels:
            raise RuntimeError("x must be (B,%d,H,W)" % self.in_channels)
        h, w = x.size(2) + 2 * self.padding, x.size(3) + 2 * self.padding
        table, wf = self._table_for(h, w, x.device)
        if torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad or self.bias.requires_grad):
            # differentiable route (the reference is differentiable through torch.fft, converse2d.cpp:223)
            from .autograd import Converse2DFunction
            out = Converse2DFunction.apply(x, self.weight, self.bias, table, wf, self.kernel_size, self.scale,
                                           self.padding, self.padding_mode, self.eps)
            return F.gelu(out) if self.fuse_gelu else out
        return CF.converse2d_forward(x, table, wf, self.kernel_size, self.scale, self.padding,
                                     self.padding_mode, fuse_gelu=self.fuse_gelu)


class ConverseBlock(nn.Module):
    """`x + conv1(x)` then `x + conv2(x)` (`models/util_converse.py:253-293`); children and
    state-dict keys as in the reference (conv1.{0,1,3,5}, conv2.{0,1,3})."""

    def __init__(self, in_channels, out_channels, kernel_size=3, scale=1, padding=2, padding_mode="replicate",
                 eps=1e-5):
        super().__init__()
        self.conv1 = nn.Sequential(LayerNorm(in_channels, eps=1e-5, data_format="channels_first"),
                                   nn.Conv2d(in_channels, 2 * out_channels, 1, 1, 0),
                                   nn.GELU(),
                                   Converse2D(2 * out_channels, 2 * out_channels, kernel_size, scale=scale,
                                              padding=padding, padding_mode=padding_mode, eps=eps),
                                   nn.GELU(),
                                   nn.Conv2d(2 * out_channels, out_channels, 1, 1, 0))
        self.conv2 = nn.Sequential(LayerNorm(in_channels, eps=1e-5, data_format="channels_first"),
                                   nn.Conv2d(out_channels, 2 * out_channels, 1, 1, 0),
                                   nn.GELU(),
                                   nn.Conv2d(2 * out_channels, out_channels, 1, 1, 0))

    def _branch1(self, x):
        c = self.conv1
        t = c[2](c[1](c[0](x)))
        conv = c[3]
        conv.fuse_gelu = True  # c[4] runs inside the Converse2D kernel
        try:
            t = conv(t)
        finally:
            conv.fuse_gelu = False
        return c[5](t)

    def _fusable(self, x):
        c1, c2 = self.conv1, self.conv2
        if torch.is_grad_enabled() and (x.requires_grad or any(q.requires_grad for q in self.parameters())):
            return False  # the fused block kernels are forward-only
        return (x.is_cuda and x.dim() == 4 and x.size(1) == 64 and c1[1].out_channels == 128 and
                c1[5].out_channels == 64 and c1[3].scale == 1 and x.dtype in (torch.float32, torch.bfloat16) and
                c1[1].bias is not None and c1[5].bias is not None and c2[1].bias is not None and
                c2[3].bias is not None and BLOCK_FUSION)

    def _forward_fused(self, x, alpha1=None, alpha2=None):
        # three kernels per block: LN+1x1+GELU, Converse2D(+GELU), 1x1+residual+LN+1x1+GELU+1x1+residual
        c1, c2 = self.conv1, self.conv2
        t = CF.ln_pw_gelu(x, c1[0], c1[1])
        conv = c1[3]
        conv.fuse_gelu = True
        try:
            t = conv(t)
        finally:
            conv.fuse_gelu = False
        return CF.pw_res_mlp(t, x, c1[5], c2[0], c2[1], c2[3], alpha1, alpha2)

    def forward(self, x):
        if self._fusable(x):
            return self._forward_fused(x)
        with _exact_fp32():
            x = self._branch1(x) + x
            x = self.conv2(x) + x
        return x


class ConverseBlockAlphaVariant(ConverseBlock):
    """ConverseBlock with learned per-channel branch scales (`models/util_converse.py:297-323`)."""

    def __init__(self, in_channels, out_channels, kernel_size=3, scale=1, padding=2, padding_mode="replicate",
                 eps=1e-5):
        super().__init__(in_channels, out_channels, kernel_size, scale, padding, padding_mode, eps)
        self.alpha1 = nn.Parameter(torch.zeros((1, out_channels, 1, 1)), requires_grad=True)
        self.alpha2 = nn.Parameter(torch.zeros((1, out_channels, 1, 1)), requires_grad=True)

    def forward(self, x):
        if self._fusable(x):
            return self._forward_fused(x, self.alpha1, self.alpha2)
        with _exact_fp32():
            x = self.alpha1 * self._branch1(x) + x
            x = self.alpha2 * self.conv2(x) + x
        return x
