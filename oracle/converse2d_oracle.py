"""CPU oracle for the Converse2D forward path.  TEST INFRASTRUCTURE ONLY.

This file restates, in numpy, the algorithm of the reference's PyTorch path
(`models/util_converse.py:142-192`, helpers `:194-245`) and of the identical
C++ op (`Converse2D/torch_converse2d/converse2d.cpp:165-209`).  It is the
checker that the CUDA path is compared against; nothing in the shipped
package may import it.  Only tests, the smoke check and the CPU-baseline leg
of the benchmark use it.

Parity pin: `tests/golden/converse2d_ref_cases.npz` holds inputs and outputs
of the unmodified reference (fp32 and fp64) produced by
`tests/golden/make_golden.py`; `tests/test_oracle.py` checks this oracle
against every case there (fp64: <= 1e-10 relative L2; fp32: <= 1e-4).

Every function works on numpy arrays laid out (B, C, H, W) like the
reference's tensors and follows the reference step by step -- including the
full-size complex FFTs the CUDA path avoids -- so that it stays an independent
statement of the operator.
"""
import numpy as np

_PAD_MODES = {"circular": "wrap", "replicate": "edge", "reflect": "reflect", "constant": "constant"}


def boundary_pad(x, p, mode):
    """`F.pad(x, [p, p, p, p], mode)` on the two spatial axes
    (`models/util_converse.py:144-145`)."""
    if p == 0:
        return x
    if mode not in _PAD_MODES:
        raise ValueError(f"unknown padding_mode {mode!r}")
    if mode == "circular" and (p > x.shape[-2] or p > x.shape[-1]):
        raise ValueError("circular padding wider than the plane")
    if mode == "reflect" and (p >= x.shape[-2] or p >= x.shape[-1]):
        raise ValueError("reflect padding must be smaller than the plane")
    return np.pad(x, ((0, 0), (0, 0), (p, p), (p, p)), mode=_PAD_MODES[mode])


def lam_from_bias(bias, eps, dtype):
    """lambda = sigmoid(bias - 9) + eps, shape (1, C, 1, 1)
    (`models/util_converse.py:147`, `converse2d.cpp:186`)."""
    b = np.asarray(bias, dtype=dtype).reshape(1, -1, 1, 1)
    one = dtype(1)
    return (one / (one + np.exp(-(b - dtype(9.0))))).astype(dtype) + dtype(eps)


def zero_insert(y, s):
    """s-fold zero-insertion upsampler, phase 0 (`models/util_converse.py:237-245`)."""
    B, C, h, w = y.shape
    z = np.zeros((B, C, h * s, w * s), dtype=y.dtype)
    z[..., ::s, ::s] = y
    return z


def nearest_upsample(y, s):
    """`F.interpolate(y, scale_factor=s, mode='nearest')` for integer s: pixel
    replication (`models/util_converse.py:172-173`)."""
    if s == 1:
        return y
    return np.repeat(np.repeat(y, s, axis=-2), s, axis=-1)


def psf2otf(weight, shape):
    """Kernel spectrum (`models/util_converse.py:218-235`): embed the k x k taps
    in the top-left corner of a zero plane, roll by -floor(k/2) on both axes,
    full 2-D FFT."""
    kh, kw = weight.shape[-2:]
    otf = np.zeros(weight.shape[:-2] + tuple(shape), dtype=weight.dtype)
    otf[..., :kh, :kw] = weight
    otf = np.roll(otf, (-(kh // 2), -(kw // 2)), axis=(-2, -1))
    return np.fft.fft2(otf)


def block_mean(a, s):
    """The reference's `splits(...)` followed by a mean over the s*s aliases
    (`models/util_converse.py:182-183,194-215`):
    out[u, v] = mean_{i,j<s} a[u + i*h, v + j*w]."""
    *lead, N_h, N_w = a.shape
    h, w = N_h // s, N_w // s
    return a.reshape(*lead, s, h, s, w).mean(axis=(-4, -2))


def converse2d_solve(y, x0, weight, bias, scale, eps, dtype=np.float32):
    """The closed-form solve on an already padded plane, returning the
    UNCROPPED result (the contract of `torch.ops.converse2d.forward`,
    `converse2d.cpp:165-209`).  `y`: (B,C,h,w); `x0`: (B,C,s*h,s*w)."""
    dtype = np.dtype(dtype).type
    y = np.asarray(y, dtype=dtype)
    x0 = np.asarray(x0, dtype=dtype)
    weight = np.asarray(weight, dtype=dtype)
    if y.ndim != 4 or x0.ndim != 4:
        raise ValueError("x and x0 must be 4-D")
    if weight.ndim != 4 or weight.shape[0] != 1:
        raise ValueError("weight must be (1,C,kh,kw)")
    if scale < 1:
        raise ValueError("scale must be >= 1")
    s = int(scale)
    _, _, h, w = y.shape
    lam = lam_from_bias(bias, eps, dtype)
    STy = zero_insert(y, s)
    FB = psf2otf(weight, (h * s, w * s))
    FBC = np.conj(FB)
    F2B = np.abs(FB) ** 2
    FBFy = FBC * np.fft.fft2(STy)
    FR = FBFy + np.fft.fft2(lam * x0)
    x1 = FB * FR
    FBR = block_mean(x1, s)
    invW = block_mean(F2B, s)
    invWBR = FBR / (invW + lam)
    FCBinvWBR = FBC * np.tile(invWBR, (1, 1, s, s))
    FX = (FR - FCBinvWBR) / lam
    return np.real(np.fft.ifft2(FX)).astype(dtype)


def converse2d_forward(x, weight, bias, scale=1, padding=2, padding_mode="circular",
                       eps=1e-5, dtype=np.float32):
    """`Converse2D.forward` (`models/util_converse.py:142-192`): pad, solve with
    x0 = nearest-upsample of the padded input, crop `[p*s : -p*s]`."""
    dtype = np.dtype(dtype).type
    x = np.asarray(x, dtype=dtype)
    y = boundary_pad(x, padding, padding_mode)
    x0 = nearest_upsample(y, scale)
    out = converse2d_solve(y, x0, weight, bias, scale, eps, dtype)
    if padding > 0:
        c = padding * scale
        out = out[..., c:-c, c:-c]
    return np.ascontiguousarray(out)


def init_weight(C, k, rng):
    """The reference's parameter init (`models/util_converse.py:137-139`): softmax
    over the k*k taps of a normal draw; bias zeros.  `rng` is a
    numpy Generator -- the draw differs from torch's, only the distribution is
    the same."""
    w = rng.standard_normal((1, C, k * k)).astype(np.float32)
    w = np.exp(w - w.max(axis=-1, keepdims=True))
    w /= w.sum(axis=-1, keepdims=True)
    return w.reshape(1, C, k, k).astype(np.float32), np.zeros((1, C, 1, 1), np.float32)


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))
