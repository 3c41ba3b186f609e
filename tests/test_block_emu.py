"""Host emulation of the fused ConverseBlock kernels against a plain PyTorch fp32/fp64 reference."""
import ctypes

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from tests.emu.build_emu import build_emu

C, M = 64, 128


@pytest.fixture(scope="module")
def emu():
    return ctypes.CDLL(build_emu())


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def ln_cf(x, w, b, eps):
    # channels_first LayerNorm of the reference (models/util_converse.py:60-68)
    u = x.mean(1, keepdim=True)
    s = (x - u).pow(2).mean(1, keepdim=True)
    return w[:, None, None] * ((x - u) / torch.sqrt(s + eps)) + b[:, None, None]


def test_ln_pw_gelu(emu):
    g = torch.Generator().manual_seed(1)
    B, H, W = 2, 9, 7  # odd pixel count: exercises the clamped tail
    x = torch.randn(B, C, H, W, generator=g)
    lw, lb = 1 + 0.3 * torch.randn(C, generator=g), 0.2 * torch.randn(C, generator=g)
    w, b = 0.2 * torch.randn(M, C, generator=g), 0.1 * torch.randn(M, generator=g)
    ref = F.gelu(F.conv2d(ln_cf(x.double(), lw.double(), lb.double(), 1e-5), w.double()[:, :, None, None], b.double()))
    out = np.full((B, M, H, W), np.nan, np.float32)
    arrs = [a.numpy().copy() for a in (x, lw, lb, w, b)]
    rc = emu.emu_ln_pw_gelu(_p(arrs[0]), _p(out), _p(arrs[1]), _p(arrs[2]), ctypes.c_float(1e-5), _p(arrs[3]),
                            _p(arrs[4]), B, H * W, 32)
    assert rc == 0 and np.isfinite(out).all()
    err = np.linalg.norm(out - ref.numpy()) / np.linalg.norm(ref.numpy())
    assert err <= 2e-6


@pytest.mark.parametrize("alphas", [False, True])
def test_pw_res_mlp(emu, alphas):
    g = torch.Generator().manual_seed(2)
    B, H, W = 1, 6, 11
    t2 = torch.randn(B, M, H, W, generator=g)
    x = torch.randn(B, C, H, W, generator=g)
    w2, b2 = 0.1 * torch.randn(C, M, generator=g), 0.1 * torch.randn(C, generator=g)
    lw, lb = 1 + 0.3 * torch.randn(C, generator=g), 0.2 * torch.randn(C, generator=g)
    w3, b3 = 0.2 * torch.randn(M, C, generator=g), 0.1 * torch.randn(M, generator=g)
    w4, b4 = 0.1 * torch.randn(C, M, generator=g), 0.1 * torch.randn(C, generator=g)
    a1 = torch.randn(C, generator=g) if alphas else torch.ones(C)
    a2 = torch.randn(C, generator=g) if alphas else torch.ones(C)
    d = lambda v: v.double()
    x1 = d(x) + d(a1)[:, None, None] * F.conv2d(d(t2), d(w2)[:, :, None, None], d(b2))
    hid = F.gelu(F.conv2d(ln_cf(x1, d(lw), d(lb), 1e-5), d(w3)[:, :, None, None], d(b3)))
    ref = x1 + d(a2)[:, None, None] * F.conv2d(hid, d(w4)[:, :, None, None], d(b4))
    out = np.full((B, C, H, W), np.nan, np.float32)
    A = [v.numpy().copy() for v in (t2, x, w2, b2, a1, lw, lb, w3, b3, w4, b4, a2)]
    rc = emu.emu_pw_res_mlp(_p(A[0]), _p(A[1]), _p(out), _p(A[2]), _p(A[3]), _p(A[4]) if alphas else None,
                            _p(A[5]), _p(A[6]), ctypes.c_float(1e-5), _p(A[7]), _p(A[8]), _p(A[9]), _p(A[10]),
                            _p(A[11]) if alphas else None, B, H * W, 32)
    assert rc == 0 and np.isfinite(out).all()
    err = np.linalg.norm(out - ref.numpy()) / np.linalg.norm(ref.numpy())
    assert err <= 2e-6
