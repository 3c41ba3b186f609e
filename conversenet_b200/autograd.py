"""Gradients of Converse2D.

The reference gets its backward from autograd through `torch.fft`
(`Converse2D/torch_converse2d/csrc/converse2d.cpp:223`, CompositeImplicitAutograd;
`test/test_error.py:50-54` pins grad-x against the Python path).  Here the operator runs
in the native kernels, so its gradient is written out.

With y = pad(x), r = IFFT2(P . FFT2(y)) on the h x w grid, and
    out = crop( nearest_s(y) + corr(K, zero_insert_s(r)) )          (scale s >= 2)
    out = crop( IFFT2(G . FFT2(y)) )                                (scale 1),
the operator is linear in x.  Its adjoint, applied to g = dL/dout, is
    g_full = zero-extend g to the s*h x s*w grid                    (adjoint of the crop)
    s >= 2:  u = sum of g_full over s x s cells                     (adjoint of nearest_s)
             v = (K convolved with g_full, circular) at every s-th sample   (adjoint of corr o zero-insert)
             g_y = u + IFFT2( conj(P) . FFT2(v) )
    s == 1:  g_y = IFFT2( conj(G) . FFT2(g_full) )
    dL/dx = adjoint of the padding applied to g_y.
The two FFTs and the multiply are the forward kernel itself (scale 1, no padding) run with the
conjugated transfer table; u, v and the padding adjoint are small PyTorch tensor ops.

dL/dweight and dL/dbias.  The parameters act through the multiplier M (G or P, one (C,h,w) complex
tensor) and, at scale >= 2, through the taps of the epilogue's correlation:
    L = (1 / (h w)) Re sum_f M[f] D[f]  (+ terms without M),
    D[f] = sum_b FFT2(y_b)[f] conj(FFT2(q_b)[f]),   q = g_full (scale 1) or v (scale >= 2).
D, the reduction over the batch, is one native kernel (`functional.cross_spectrum`); the chain rule
from D to the k x k taps and lambda runs through `transfer_multiplier`, the closed form of M written
with `torch.fft` on that single (C, s h, s w) tensor.  The direct tap term of scale >= 2,
dK[a] = sum_m g_full[s m - a + c] r[m], needs r = IFFT2(P . FFT2(y)): the forward kernel at scale 1
on the padded planes, followed by k^2 strided products.  Planes the cross-spectrum kernel does not
take (two planes must fit shared memory) fall back to autograd through `spectral_forward`, the
whole operator restated with `torch.fft` (library kernels).
"""
import torch
import torch.nn.functional as F

from . import functional as CF


# False: parameter gradients always take the `spectral_forward` route (tests compare the two)
NATIVE_PARAM_GRADS = True


def _pad(x, p, mode):
    if p == 0:
        return x
    if mode == "constant":
        return F.pad(x, (p, p, p, p), mode="constant", value=0.0)
    return F.pad(x, (p, p, p, p), mode=mode)


def transfer_multiplier(weight, bias, scale, eps, h, w):
    """The operator's multiplier on the h x w grid, (1,C,h,w) complex, natural frequency order,
    differentiable in `weight` (1,C,k,k) and `bias` (1,C,1,1): G at scale 1, P at scale >= 2."""
    s = int(scale)
    C, k = weight.size(1), weight.size(-1)
    c = k // 2
    lam = torch.sigmoid(bias - 9.0) + eps                                    # (1,C,1,1)
    # kernel spectrum on the s*h x s*w grid, kernel centre (k//2, k//2) at the origin
    psf = torch.zeros(1, C, s * h, s * w, dtype=weight.dtype, device=weight.device)
    psf[..., :k, :k] = weight
    psf = torch.roll(psf, shifts=(-c, -c), dims=(-2, -1))
    FK = torch.fft.fft2(psf)
    if s == 1:
        return (FK.conj() + lam) / (FK.real ** 2 + FK.imag ** 2 + lam)
    # box factor of the nearest upsampling, alias means over the s x s copies of the h x w spectrum
    box = torch.zeros(s * h, s * w, dtype=weight.dtype, device=weight.device)
    box[:s, :s] = 1.0
    D = torch.fft.fft2(box)

    def alias_mean(Z):
        return Z.reshape(*Z.shape[:-2], s, h, s, w).mean(dim=(-4, -2))

    return (1.0 - alias_mean(FK * D)) / (alias_mean(FK.real ** 2 + FK.imag ** 2) + lam)


def spectral_forward(x, weight, bias, scale, padding, padding_mode, eps):
    """The operator written with `torch.fft` in its collapsed form (differentiable in every
    argument; any device and float dtype).  Fallback for parameter gradients; used by the tests."""
    s, p = int(scale), int(padding)
    B, C, H, W = x.shape
    k = weight.size(-1)
    c = k // 2
    y = _pad(x, p, padding_mode)
    h, w = y.shape[-2:]
    M = transfer_multiplier(weight.to(x.dtype), bias.to(x.dtype), s, eps, h, w)
    if s == 1:
        return torch.fft.ifft2(M * torch.fft.fft2(y)).real[..., p:p + H, p:p + W]
    r = torch.fft.ifft2(M * torch.fft.fft2(y)).real                           # (B,C,h,w)
    z = torch.zeros(B, C, s * h, s * w, dtype=x.dtype, device=x.device)
    z[..., ::s, ::s] = r
    # corr(K, z)[i] = sum_a K[a] z[i + a - c], circular
    zp = F.pad(z, (c, k - 1 - c, c, k - 1 - c), mode="circular")
    corr = F.conv2d(zp, weight.reshape(C, 1, k, k).to(x.dtype), groups=C)
    up = y.repeat_interleave(s, dim=-2).repeat_interleave(s, dim=-1)
    full = up + corr
    return full[..., p * s:(p + H) * s, p * s:(p + W) * s]


def _conjugated(table, n_entries):
    """Copy of a transfer table with the multiplier conjugated (the twiddle tables behind it untouched)."""
    t = table.clone()
    t.view(torch.float32)[: 2 * n_entries].view(-1, 2)[:, 1].neg_()
    return t


class _Cotangent:
    """g = dL/dout prepared once per backward call: zero-extended to the padded grid (adjoint of the
    crop) and, at scale >= 2, v[m] = sum_a K[a] g_full[s m - a + c] (adjoint of corr(K, zero_insert(.)):
    a strided cross-correlation with the flipped kernel).  dL/dx and the parameter gradients share it."""

    def __init__(self, g, wf, k, s, p):
        ps = p * s
        self.g_full = (F.pad(g, (ps, ps, ps, ps)) if ps else g).float().contiguous()
        self.v = None
        if s > 1:
            c = k // 2
            C = wf.size(0)
            gp = F.pad(self.g_full, (k - 1 - c, c, k - 1 - c, c), mode="circular")
            self.v = F.conv2d(gp, wf.flip(-2, -1).reshape(C, 1, k, k), stride=s, groups=C).contiguous()


def grad_input(g, weight, bias, scale, padding, padding_mode, eps, in_shape, table=None, cot=None):
    """dL/dx for g = dL/dout (B,C,sH,sW) through the native kernels.  `table`: the forward's
    transfer table for the padded size, if the caller has it."""
    s, p = int(scale), int(padding)
    B, C, H, W = in_shape
    h, w = H + 2 * p, W + 2 * p
    k = weight.size(-1)
    if table is None:
        table, _ = CF.build_transfer(weight, bias, s, eps, h, w)
    wf = weight.detach().reshape(C, k, k).to(torch.float32).contiguous()
    ctab = _conjugated(table, C * h * w)
    if cot is None:
        cot = _Cotangent(g, wf, k, s, p)
    if s == 1:
        g_y = CF.converse2d_forward(cot.g_full, ctab, wf, k, 1, 0, "circular")
    else:
        u = F.avg_pool2d(cot.g_full, s) * float(s * s)
        g_y = u + CF.converse2d_forward(cot.v, ctab, wf, k, 1, 0, "circular")
    g_y = g_y.to(g.dtype)
    if p == 0:
        return g_y
    # adjoint of the boundary padding: PyTorch's own pad backward (a gather / scatter-add)
    probe = torch.zeros(in_shape, dtype=g_y.dtype, device=g_y.device, requires_grad=True)
    with torch.enable_grad():
        padded = _pad(probe, p, padding_mode)
    return torch.autograd.grad(padded, probe, g_y)[0]


def grad_params(x, g, weight, bias, scale, padding, padding_mode, eps, table=None, cot=None):
    """(dL/dweight, dL/dbias) in fp32 for g = dL/dout, batch reductions in the native kernels; None when
    the cross-spectrum kernel does not take the padded plane (the caller then falls back)."""
    s, p = int(scale), int(padding)
    B, C, H, W = x.shape
    h, w = H + 2 * p, W + 2 * p
    if not CF.cross_spectrum_supported(h, w):
        return None
    k = weight.size(-1)
    if table is None:
        table, _ = CF.build_transfer(weight, bias, s, eps, h, w)
    wf = weight.detach().reshape(C, k, k).to(torch.float32).contiguous()
    xf = x.detach().float().contiguous()
    if cot is None:
        cot = _Cotangent(g, wf, k, s, p)
    D = CF.cross_spectrum(xf, cot.g_full if s == 1 else cot.v, table, p, padding_mode)   # (C,h,w) complex
    with torch.enable_grad():
        w_ = weight.detach().float().requires_grad_(True)
        b_ = bias.detach().float().requires_grad_(True)
        M = transfer_multiplier(w_, b_, s, eps, h, w)[0]
        proxy = (M * D).real.sum() / float(h * w)
        gw, gb = torch.autograd.grad(proxy, (w_, b_))
    if s > 1:
        # direct dependence of corr(K, zero_insert(r)) on the taps; r = the forward at scale 1 on the padded planes
        y = _pad(xf, p, padding_mode).contiguous()
        r = CF.converse2d_forward(y, table, wf, k, 1, 0, "circular")
        gw = gw + CF.tap_gradient(cot.g_full, r, k, s).reshape(1, C, k, k)
    return gw, gb


class Converse2DFunction(torch.autograd.Function):
    """Native forward; native dL/dx; parameter gradients from the native batch-summed cross spectrum
    (`grad_params`), through `spectral_forward` for planes that kernel does not take."""

    @staticmethod
    def forward(ctx, x, weight, bias, table, wf, kernel_size, scale, padding, padding_mode, eps):
        ctx.save_for_backward(x, weight, bias)
        ctx.table = table
        ctx.cfg = (int(kernel_size), int(scale), int(padding), padding_mode, float(eps))
        return CF.converse2d_forward(x, table, wf, kernel_size, scale, padding, padding_mode)

    @staticmethod
    def backward(ctx, g):
        x, weight, bias = ctx.saved_tensors
        k, s, p, mode, eps = ctx.cfg
        gx = gw = gb = None
        C = weight.size(1)
        cot = _Cotangent(g, weight.detach().reshape(C, k, k).to(torch.float32), k, s, p)
        if ctx.needs_input_grad[0]:
            gx = grad_input(g, weight, bias, s, p, mode, eps, x.shape, table=ctx.table, cot=cot)
        if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
            native = (grad_params(x, g, weight, bias, s, p, mode, eps, table=ctx.table, cot=cot)
                      if NATIVE_PARAM_GRADS else None)
            if native is not None:
                gw, gb = native
            else:
                with torch.enable_grad():
                    w_ = weight.detach().float().requires_grad_(True)
                    b_ = bias.detach().float().requires_grad_(True)
                    out = spectral_forward(x.detach().float(), w_, b_, s, p, mode, eps)
                    gw, gb = torch.autograd.grad(out, (w_, b_), g.float())
            gw = gw.to(weight.dtype) if ctx.needs_input_grad[1] else None
            gb = gb.to(bias.dtype) if ctx.needs_input_grad[2] else None
        return gx, gw, gb, None, None, None, None, None, None, None
