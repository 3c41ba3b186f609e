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

dL/dweight and dL/dbias go through the table (P depends on K and lambda) and are not
written natively: when a parameter requires a gradient they come from autograd through a
`torch.fft` restatement of the same closed form (`spectral_forward`, library kernels).
"""
import torch
import torch.nn.functional as F

from . import functional as CF


def _pad(x, p, mode):
    if p == 0:
        return x
    if mode == "constant":
        return F.pad(x, (p, p, p, p), mode="constant", value=0.0)
    return F.pad(x, (p, p, p, p), mode=mode)


def spectral_forward(x, weight, bias, scale, padding, padding_mode, eps):
    """The operator written with `torch.fft` in its collapsed form (differentiable in every
    argument; any device and float dtype).  Used for parameter gradients and by the tests."""
    s, p = int(scale), int(padding)
    B, C, H, W = x.shape
    k = weight.size(-1)
    c = k // 2
    y = _pad(x, p, padding_mode)
    h, w = y.shape[-2:]
    lam = torch.sigmoid(bias - 9.0) + eps                                    # (1,C,1,1)
    # kernel spectrum on the s*h x s*w grid, kernel centre (k//2, k//2) at the origin
    psf = torch.zeros(1, C, s * h, s * w, dtype=x.dtype, device=x.device)
    psf[..., :k, :k] = weight
    psf = torch.roll(psf, shifts=(-c, -c), dims=(-2, -1))
    FK = torch.fft.fft2(psf)
    if s == 1:
        G = (FK.conj() + lam) / (FK.real ** 2 + FK.imag ** 2 + lam)
        return torch.fft.ifft2(G * torch.fft.fft2(y)).real[..., p:p + H, p:p + W]
    # box factor of the nearest upsampling, alias means over the s x s copies of the h x w spectrum
    box = torch.zeros(s * h, s * w, dtype=x.dtype, device=x.device)
    box[:s, :s] = 1.0
    D = torch.fft.fft2(box)

    def alias_mean(Z):
        return Z.reshape(*Z.shape[:-2], s, h, s, w).mean(dim=(-4, -2))

    P = (1.0 - alias_mean(FK * D)) / (alias_mean(FK.real ** 2 + FK.imag ** 2) + lam)
    r = torch.fft.ifft2(P * torch.fft.fft2(y)).real                           # (B,C,h,w)
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


def grad_input(g, weight, bias, scale, padding, padding_mode, eps, in_shape, table=None):
    """dL/dx for g = dL/dout (B,C,sH,sW) through the native kernels.  `table`: the forward's
    transfer table for the padded size, if the caller has it."""
    s, p = int(scale), int(padding)
    B, C, H, W = in_shape
    h, w = H + 2 * p, W + 2 * p
    k = weight.size(-1)
    c = k // 2
    if table is None:
        table, _ = CF.build_transfer(weight, bias, s, eps, h, w)
    wf = weight.detach().reshape(C, k, k).to(torch.float32).contiguous()
    ctab = _conjugated(table, C * h * w)
    g = g.contiguous()
    ps = p * s
    g_full = F.pad(g, (ps, ps, ps, ps)) if ps else g                          # zeros outside the crop
    if s == 1:
        g_y = CF.converse2d_forward(g_full, ctab, wf, k, 1, 0, "circular")
    else:
        u = F.avg_pool2d(g_full.float(), s) * float(s * s)
        # v[m] = sum_a K[a] g_full[s m - a + c]: a strided cross-correlation with the flipped kernel
        gp = F.pad(g_full.float(), (k - 1 - c, c, k - 1 - c, c), mode="circular")
        v = F.conv2d(gp, wf.flip(-2, -1).reshape(C, 1, k, k), stride=s, groups=C)
        g_y = u + CF.converse2d_forward(v.contiguous(), ctab, wf, k, 1, 0, "circular")
        g_y = g_y.to(g.dtype)
    if p == 0:
        return g_y
    # adjoint of the boundary padding: PyTorch's own pad backward (a gather / scatter-add)
    probe = torch.zeros(in_shape, dtype=g_y.dtype, device=g_y.device, requires_grad=True)
    with torch.enable_grad():
        padded = _pad(probe, p, padding_mode)
    return torch.autograd.grad(padded, probe, g_y)[0]


class Converse2DFunction(torch.autograd.Function):
    """Native forward; native dL/dx; parameter gradients through `spectral_forward`."""

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
        if ctx.needs_input_grad[0]:
            gx = grad_input(g, weight, bias, s, p, mode, eps, x.shape, table=ctx.table)
        if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
            with torch.enable_grad():
                w_ = weight.detach().float().requires_grad_(True)
                b_ = bias.detach().float().requires_grad_(True)
                out = spectral_forward(x.detach().float(), w_, b_, s, p, mode, eps)
                gw, gb = torch.autograd.grad(out, (w_, b_), g.float())
            gw = gw.to(weight.dtype) if ctx.needs_input_grad[1] else None
            gb = gb.to(bias.dtype) if ctx.needs_input_grad[2] else None
        return gx, gw, gb, None, None, None, None, None, None, None
