"""Importing this module registers `torch.ops.converse2d.forward` and
`torch.ops.converse2d.clear_cache` with the reference's schema
(`Converse2D/torch_converse2d/converse2d.cpp:218-227`), backed by the native library.

    forward(Tensor x, Tensor x0, Tensor weight, Tensor bias, int scale, float eps=1e-5) -> Tensor

`x` is the already padded plane batch (B,C,h,w), the result is the UNCROPPED
(B,C,s*h,s*w) solve, as in the reference.  The fused kernels implement the solve for
`x0 = nearest-upsample(x)`, which is what `Converse2D.forward` passes
(`models/util_converse.py:166`).  The operator is linear in (x, x0), so any other `x0` is
answered as  solve(x, nearest(x)) + T(d),  d = x0 - nearest(x), with
    T(d) = d - corr(K, zero_insert_s(q)),   q = IFFT2( FFT2(decimate_s(K * d)) / (alias mean |FK|^2 + lambda) )
(`models/util_converse.py:178-187` with x = 0): the two FFTs are the forward kernel at scale 1 with the
table of `cvb_build_x0_table`, the k x k correlations are PyTorch convolutions.
Differentiable as the reference's op is (CompositeImplicitAutograd there): separate partial derivatives
for `x` and `x0` through the native kernels (see `_backward`), parameter gradients through the `torch.fft`
restatement in `conversenet_b200/autograd.py`.  Deciding whether `x0` equals the up-sampled `x` takes one
device comparison (a synchronisation) per forward call unless the two are the same tensor at scale 1.

Do not import this module in a process that also loads the reference's own extension:
a schema can be defined once.
"""
from collections import OrderedDict

import torch
import torch.nn.functional as F

from . import functional as CF

_CACHE_SLOTS = 64  # as the reference's FB cache (`converse2d.cpp:52`)
_cache = OrderedDict()

_lib = torch.library.Library("converse2d", "DEF")
_lib.define("forward(Tensor x, Tensor x0, Tensor weight, Tensor bias, int scale, float eps=1e-5) -> Tensor")
_lib.define("clear_cache() -> ()")


def _forward(x, x0, weight, bias, scale, eps=1e-5):
    if x.dim() != 4:
        raise RuntimeError("x must be (B,C,H,W)")
    if x0.dim() != 4:
        raise RuntimeError("x0 must be (B,C,Hs,Ws)")
    if weight.dim() != 4 or weight.size(0) != 1:
        raise RuntimeError("weight must be (1,C,kh,kw)")
    if bias.dim() != 4 or bias.size(0) != 1 or bias.size(2) != 1 or bias.size(3) != 1:
        raise RuntimeError("bias must be (1,C,1,1)")
    if not (x.device == x0.device == weight.device == bias.device):
        raise RuntimeError("tensors on same device")
    if scale < 1:
        raise RuntimeError("scale must be >= 1")
    if not x.is_cuda:
        raise RuntimeError("converse2d.forward: this build only has the native CUDA path")
    x = x.contiguous()
    B, C, h, w = x.shape
    if tuple(x0.shape) != (B, C, h * scale, w * scale):
        raise RuntimeError("x0 must be (B,C,scale*H,scale*W)")
    same = x0.data_ptr() == x.data_ptr() if scale == 1 else False
    d = None
    if not same:
        ref = x if scale == 1 else F.interpolate(x, scale_factor=scale, mode="nearest")
        if not torch.equal(x0, ref):
            d = (x0 - ref).float()
    key = (x.device, weight.data_ptr(), weight._version, bias.data_ptr(), bias._version, C, h, w, int(scale),
           float(eps))
    hit = _cache.get(key)
    if hit is None:
        hit = CF.build_transfer(weight, bias, int(scale), float(eps), h, w)
        _cache[key] = hit
        while len(_cache) > _CACHE_SLOTS:
            _cache.popitem(last=False)
    else:
        _cache.move_to_end(key)
    table, wf = hit
    # padding 0: the solve on the plane as given, nothing cropped
    out = CF.converse2d_forward(x, table, wf, weight.size(2), int(scale), 0, "circular")
    if d is not None:
        out = out + _x0_term(d, weight, bias, wf, int(scale), float(eps), h, w).to(out.dtype)
    return out


def _x0_term(d, weight, bias, wf, s, eps, h, w):
    """T(d) for d = x0 - nearest(x), (B,C,s*h,s*w) fp32."""
    C, k = wf.size(0), wf.size(1)
    c = k // 2
    key = ("x0", d.device, weight.data_ptr(), weight._version, bias.data_ptr(), bias._version, C, h, w, s, eps)
    tab = _cache.get(key)
    if tab is None:
        tab = CF.build_transfer(weight, bias, s, eps, h, w, x0_term=True)[0]
        _cache[key] = tab
    # e[m] = (K * d)[s m] = sum_a K[a] d[s m - a + c], circular
    dp = F.pad(d, (k - 1 - c, c, k - 1 - c, c), mode="circular")
    e = F.conv2d(dp, wf.flip(-2, -1).reshape(C, 1, k, k), stride=s, groups=C).contiguous()
    q = CF.converse2d_forward(e, tab, wf, k, 1, 0, "circular")
    z = torch.zeros_like(d)
    z[..., ::s, ::s] = q
    zp = F.pad(z, (c, k - 1 - c, c, k - 1 - c), mode="circular")
    return d - F.conv2d(zp, wf.reshape(C, 1, k, k), groups=C)


def _clear_cache():
    _cache.clear()


def _setup_context(ctx, inputs, output):
    x, x0, weight, bias, scale, eps = inputs
    ctx.save_for_backward(x, weight, bias)
    ctx.cfg = (int(scale), float(eps))


def _backward(ctx, g):
    """True partial derivatives.  The op is out = (F - T N) x + T x0 with F the fused operator for
    x0 = N x (N = nearest up-sampling) and T the self-adjoint x0-term operator of `_x0_term`:
        dL/dx0 = T g,      dL/dx = F^T g - N^T (T g),
    so that x0 = interpolate(x) in the caller's graph adds N^T (T g) back and x receives F^T g in total,
    while a detached or independent x0 gets exactly its own share.  Parameter gradients go through the
    `torch.fft` restatement and are written for the tied case (x0 = N x), the only one the reference's
    module produces."""
    from .autograd import grad_input, spectral_forward
    x, weight, bias = ctx.saved_tensors
    scale, eps = ctx.cfg
    gx = gx0 = gw = gb = None
    if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
        B, C, h, w = x.shape
        k = weight.size(-1)
        wf = weight.detach().reshape(C, k, k).to(torch.float32).contiguous()
        tg = _x0_term(g.float().contiguous(), weight, bias, wf, scale, eps, h, w)
        if ctx.needs_input_grad[1]:
            gx0 = tg.to(g.dtype)
        if ctx.needs_input_grad[0]:
            gx = grad_input(g, weight, bias, scale, 0, "circular", eps, x.shape)
            back = tg if scale == 1 else F.avg_pool2d(tg, scale) * float(scale * scale)
            gx = gx - back.to(gx.dtype)
    if ctx.needs_input_grad[2] or ctx.needs_input_grad[3]:
        with torch.enable_grad():
            w_ = weight.detach().float().requires_grad_(True)
            b_ = bias.detach().float().requires_grad_(True)
            out = spectral_forward(x.detach().float(), w_, b_, scale, 0, "circular", eps)
            gw, gb = torch.autograd.grad(out, (w_, b_), g.float())
        gw = gw.to(weight.dtype) if ctx.needs_input_grad[2] else None
        gb = gb.to(bias.dtype) if ctx.needs_input_grad[3] else None
    return gx, gx0, gw, gb, None, None


_lib.impl("forward", _forward, "CUDA")
_lib.impl("forward", _forward, "CPU")  # raises: no CPU path
_lib.impl("clear_cache", _clear_cache, "CompositeExplicitAutograd")
torch.library.register_autograd("converse2d::forward", _backward, setup_context=_setup_context, lib=_lib)
