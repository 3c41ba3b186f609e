"""Tensor-level entry points over the C ABI (device memory and streams come from torch)."""

import torch

from . import _cabi


def _stream_ptr(device):
    return torch.cuda.current_stream(device).cuda_stream


def _io_dtype(t):
    if t.dtype == torch.float32:
        return _cabi.CVB_F32
    if t.dtype == torch.bfloat16:
        return _cabi.CVB_BF16
    raise RuntimeError("Converse2D supports float32 and bfloat16 tensors, got %s" % t.dtype)


def build_transfer(weight, bias, scale, eps, h, w, x0_term=False):
    """Transfer table for `weight` (1,C,k,k) / `bias` (1,C,1,1) at padded size h x w.
    `x0_term`: the real table 1 / (alias mean of |FK|^2 + lambda) that the term of an
    arbitrary `x0` needs (`cvb_build_x0_table`) instead of the operator's multiplier.

    Plays the role of the reference's cached kernel spectrum
    (`converse2d.cpp:58-102`), but holds the complete weights-only multiplier.
    Returns a uint8 CUDA tensor owned by the caller."""
    lib = _cabi.load()
    if not weight.is_cuda:
        raise RuntimeError("Converse2D parameters must live on a CUDA device")
    if weight.dim() != 4 or weight.size(0) != 1:
        raise RuntimeError("weight must be (1,C,kh,kw)")
    C, k = weight.size(1), weight.size(2)
    if weight.size(3) != k:
        raise RuntimeError("only square kernels are supported")
    if bias.dim() != 4 or bias.size(0) != 1 or bias.size(1) != C or bias.size(2) != 1 or bias.size(3) != 1:
        raise RuntimeError("bias must be (1,C,1,1)")
    if scale < 1:
        raise RuntimeError("scale must be >= 1")
    nbytes = lib.cvb_transfer_bytes(C, h, w)
    if nbytes == 0:
        raise RuntimeError("padded plane %dx%d is not supported by the FFT engine" % (h, w))
    wf = weight.detach().reshape(C, k, k).to(torch.float32).contiguous()
    bf = bias.detach().reshape(C).to(torch.float32).contiguous()
    table = torch.empty(nbytes, dtype=torch.uint8, device=weight.device)
    with torch.cuda.device(weight.device):
        fn = lib.cvb_build_x0_table if x0_term else lib.cvb_build_transfer
        rc = fn(wf.data_ptr(), bf.data_ptr(), C, k, int(scale), h, w, float(eps), table.data_ptr(),
                _stream_ptr(weight.device))
    _cabi.check(rc, "cvb_build_transfer")
    return table, wf


def converse2d_forward(x, table, weight_f32, kernel_size, scale, padding, padding_mode, fuse_gelu=False,
                       out=None):
    """Fused pad -> solve -> crop (`models/util_converse.py:142-192`) on a CUDA tensor."""
    lib = _cabi.load()
    if not x.is_cuda:
        raise RuntimeError("Converse2D needs a CUDA tensor; this build has no CPU path")
    if x.dim() != 4:
        raise RuntimeError("x must be (B,C,H,W)")
    if padding_mode not in _cabi.PAD_MODES:
        raise RuntimeError("unknown padding_mode %r" % (padding_mode,))
    x = x.contiguous()
    B, C, H, W = x.shape
    io = _io_dtype(x)
    s = int(scale)
    if out is None:
        out = torch.empty((B, C, H * s, W * s), dtype=x.dtype, device=x.device)
    ws_bytes = lib.cvb_converse2d_workspace_bytes(B, C, H, W, s, int(padding), io)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device) if ws_bytes else None
    with torch.cuda.device(x.device):
        rc = lib.cvb_converse2d_fwd(x.data_ptr(), out.data_ptr(), table.data_ptr(), weight_f32.data_ptr(),
                                    B, C, H, W, int(kernel_size), s, int(padding),
                                    _cabi.PAD_MODES[padding_mode], io, 1 if fuse_gelu else 0,
                                    ws.data_ptr() if ws is not None else None, ws_bytes,
                                    _stream_ptr(x.device))
    _cabi.check(rc, "cvb_converse2d_fwd")
    return out


def cross_spectrum_supported(h, w):
    """True when `cross_spectrum` has a kernel for the padded plane h x w."""
    return _cabi.load().cvb_cross_spectrum_supported(int(h), int(w)) in (1, 2)


def cross_spectrum(x, q, table, padding, padding_mode):
    """sum_b FFT2(pad(x[b]))  * conj(FFT2(q[b])) per channel, complex64 (C,h,w), natural frequency order.

    x (B,C,H,W), q (B,C,h,w) with h = H + 2*padding: the batch reduction behind dL/dweight and
    dL/dbias (the reference leaves it to autograd through `torch.fft`, `converse2d.cpp:223`).
    `table`: a transfer table of the same (C,h,w) (its twiddle tables are used)."""
    lib = _cabi.load()
    if not (x.is_cuda and q.is_cuda):
        raise RuntimeError("cross_spectrum needs CUDA tensors; this build has no CPU path")
    if padding_mode not in _cabi.PAD_MODES:
        raise RuntimeError("unknown padding_mode %r" % (padding_mode,))
    x = x.detach().to(torch.float32).contiguous()
    q = q.detach().to(torch.float32)
    B, C, H, W = x.shape
    p = int(padding)
    h, w = H + 2 * p, W + 2 * p
    if tuple(q.shape) != (B, C, h, w):
        raise RuntimeError("q must be (B,C,H+2p,W+2p)")
    # The kernel transforms z = pad(x) + i q as one complex plane and separates the two spectra
    # afterwards; a q far smaller than x (a gradient of a mean loss) would drown in the rounding of
    # |Z|^2, so each channel of q is brought to the magnitude of x first and the result scaled back.
    xn = x.square().sum(dim=(0, 2, 3)).sqrt()
    qn = q.square().sum(dim=(0, 2, 3)).sqrt()
    gain = torch.where((qn > 0) & (xn > 0), xn / qn.clamp_min(1e-38), torch.ones_like(qn))
    q = (q * gain.view(1, C, 1, 1)).contiguous()
    props = torch.cuda.get_device_properties(x.device)
    nseg = max(1, min(B, (2 * props.multi_processor_count + C - 1) // C))
    # large planes (kind 2): the blocks add into one slab, which the library zero-fills
    slabs = 1 if lib.cvb_cross_spectrum_supported(h, w) == 2 else nseg
    out = torch.empty((slabs, C, h, w, 2), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib.cvb_cross_spectrum(x.data_ptr(), q.data_ptr(), table.data_ptr(), out.data_ptr(), nseg, B, C, H, W,
                                    p, _cabi.PAD_MODES[padding_mode], _stream_ptr(x.device))
    _cabi.check(rc, "cvb_cross_spectrum")
    d = torch.view_as_complex(out.sum(0) if slabs > 1 else out[0])
    return d / gain.view(C, 1, 1)


def tap_gradient(g_full, r, kernel_size, scale):
    """sum_{n,m} g_full[n,c,(s m - a + k//2) mod] r[n,c,m] -> (C,k,k): the direct dependence of the scale >= 2
    epilogue on the taps (`cvb_tap_gradient`)."""
    lib = _cabi.load()
    g_full = g_full.detach().to(torch.float32).contiguous()
    r = r.detach().to(torch.float32).contiguous()
    B, C, h, w = r.shape
    k, s = int(kernel_size), int(scale)
    if tuple(g_full.shape) != (B, C, s * h, s * w):
        raise RuntimeError("g_full must be (B,C,s*h,s*w) for r (B,C,h,w)")
    props = torch.cuda.get_device_properties(r.device)
    nseg = max(1, min(B, (4 * props.multi_processor_count + C - 1) // C))
    out = torch.empty((nseg, C, k, k), dtype=torch.float32, device=r.device)
    with torch.cuda.device(r.device):
        rc = lib.cvb_tap_gradient(g_full.data_ptr(), r.data_ptr(), out.data_ptr(), nseg, B, C, h, w, k, s,
                                  _stream_ptr(r.device))
    _cabi.check(rc, "cvb_tap_gradient")
    return out.sum(0) if nseg > 1 else out[0]


def _f32(t):
    return t.detach().to(torch.float32).contiguous()


def ln_pw_gelu(x, ln, conv):
    """GELU(conv1x1(LayerNorm_channels_first(x))) in one kernel (C = 64 -> 128).
    `ln`: the block's LayerNorm module, `conv`: its 1x1 nn.Conv2d (`models/util_converse.py:278-280`)."""
    lib = _cabi.load()
    x = x.contiguous()
    B, C, H, W = x.shape
    out = torch.empty((B, conv.out_channels, H, W), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib.cvb_ln_pw_gelu_fwd(x.data_ptr(), out.data_ptr(), _f32(ln.weight).data_ptr(), _f32(ln.bias).data_ptr(),
                                    float(ln.eps), _f32(conv.weight).data_ptr(), _f32(conv.bias).data_ptr(),
                                    B, C, H * W, _io_dtype(x), _stream_ptr(x.device))
    _cabi.check(rc, "cvb_ln_pw_gelu_fwd")
    return out


def pw_res_mlp(t, x, conv_out, ln, conv_up, conv_down, alpha1=None, alpha2=None):
    """x1 = x + alpha1*conv_out(t); out = x1 + alpha2*conv_down(GELU(conv_up(LayerNorm(x1)))) in one kernel
    (`models/util_converse.py:283-292`, alphas `:321-322`)."""
    lib = _cabi.load()
    t = t.contiguous()
    x = x.contiguous()
    B, C, H, W = x.shape
    bk = lib.cvb_get_option(_cabi.OPT_BLOCK_KERNELS)
    if (H * W) % 128 == 0 and (bk >= 2 or (bk == 1 and x.dtype == torch.float32)):
        # tensor-core route: three tcgen05 kernels (1x1 + residual, LN + 1x1 + GELU, 1x1 + residual)
        x1 = pw_res(t, x, conv_out, alpha1)
        hid = ln_pw_gelu(x1, ln, conv_up)
        return pw_res(hid, x1, conv_down, alpha2)
    out = torch.empty_like(x)
    keep = [_f32(conv_out.weight), _f32(conv_out.bias), _f32(ln.weight), _f32(ln.bias), _f32(conv_up.weight),
            _f32(conv_up.bias), _f32(conv_down.weight), _f32(conv_down.bias)]
    a1 = _f32(alpha1).reshape(-1) if alpha1 is not None else None
    a2 = _f32(alpha2).reshape(-1) if alpha2 is not None else None
    with torch.cuda.device(x.device):
        rc = lib.cvb_pw_res_mlp_fwd(t.data_ptr(), x.data_ptr(), out.data_ptr(), keep[0].data_ptr(), keep[1].data_ptr(),
                                    a1.data_ptr() if a1 is not None else None, keep[2].data_ptr(), keep[3].data_ptr(),
                                    float(ln.eps), keep[4].data_ptr(), keep[5].data_ptr(), keep[6].data_ptr(),
                                    keep[7].data_ptr(), a2.data_ptr() if a2 is not None else None,
                                    B, C, H * W, _io_dtype(x), _stream_ptr(x.device))
    _cabi.check(rc, "cvb_pw_res_mlp_fwd")
    return out


def pw_res(t, res, conv, alpha=None):
    """res + alpha * conv1x1(t) on the tensor cores (128 -> 64 channels, fp32, whole 128-pixel tiles)."""
    lib = _cabi.load()
    t = t.contiguous()
    res = res.contiguous()
    B, C, H, W = res.shape
    out = torch.empty_like(res)
    w, b = _f32(conv.weight), _f32(conv.bias)
    a = _f32(alpha).reshape(-1) if alpha is not None else None
    with torch.cuda.device(res.device):
        rc = lib.cvb_pw_res_fwd(t.data_ptr(), res.data_ptr(), out.data_ptr(), w.data_ptr(), b.data_ptr(),
                                a.data_ptr() if a is not None else None, B, C, H * W, _io_dtype(res),
                                _stream_ptr(res.device))
    _cabi.check(rc, "cvb_pw_res_fwd")
    return out
