"""Gradients of Converse2D: the torch.fft restatement against the numpy oracle (CPU), and the native
dL/dx against autograd through that restatement (GPU; the comparison `test/test_error.py:50-54` of the
reference makes between its two backends)."""
import numpy as np
import pytest
import torch

from conversenet_b200.autograd import spectral_forward
from oracle import converse2d_oracle as orc

CASES = [
    # B, C, H, W, k, s, p, mode
    (2, 3, 12, 10, 5, 1, 2, "circular"),
    (1, 2, 9, 14, 3, 2, 1, "replicate"),
    (2, 2, 8, 8, 5, 2, 2, "circular"),
    (1, 3, 10, 7, 2, 2, 2, "replicate"),
    (1, 2, 6, 9, 5, 3, 2, "reflect"),
    (1, 2, 11, 11, 7, 1, 3, "constant"),
]


@pytest.mark.parametrize("case", CASES)
def test_spectral_restatement_matches_oracle(case):
    B, C, H, W, k, s, p, mode = case
    rng = np.random.default_rng(11)
    x = rng.standard_normal((B, C, H, W))
    w, b = orc.init_weight(C, k, rng)
    b = b + rng.standard_normal(b.shape) * 0.5
    ref = orc.converse2d_forward(x, w, b, s, p, mode, 1e-5, dtype=np.float64)
    out = spectral_forward(torch.from_numpy(x), torch.from_numpy(w).double(), torch.from_numpy(b).double(),
                           s, p, mode, 1e-5)
    assert orc.rel_l2(out.numpy(), ref) <= 1e-10


@pytest.mark.gpu
@pytest.mark.parametrize("case", [
    (2, 4, 32, 32, 5, 1, 2, "circular"),     # shared-memory kernels
    (3, 2, 64, 64, 5, 2, 2, "circular"),     # test_error.py's setting: scale 2, padding k // 2
    (2, 3, 30, 44, 3, 2, 1, "replicate"),
    (1, 2, 24, 40, 2, 2, 2, "replicate"),    # even kernel
    (1, 2, 40, 24, 5, 3, 2, "reflect"),
    (1, 2, 256, 256, 7, 1, 6, "circular"),   # multi-pass path (268)
])
def test_grad_input_matches_autograd_of_the_restatement(case):
    from conversenet_b200 import Converse2D
    B, C, H, W, k, s, p, mode = case
    torch.manual_seed(3)
    m = Converse2D(C, C, k, scale=s, padding=p, padding_mode=mode, eps=1e-5).cuda()
    with torch.no_grad():
        m.bias.add_(torch.randn_like(m.bias) * 0.5)
    x = torch.randn(B, C, H, W, device="cuda", requires_grad=True)
    y = m(x)
    loss = y.square().mean()
    gx, gw, gb = torch.autograd.grad(loss, (x, m.weight, m.bias))
    # reference gradients: autograd through the restatement in fp64
    x64 = x.detach().double().requires_grad_(True)
    w64 = m.weight.detach().double().requires_grad_(True)
    b64 = m.bias.detach().double().requires_grad_(True)
    y64 = spectral_forward(x64, w64, b64, s, p, mode, 1e-5)
    rx, rw, rb = torch.autograd.grad(y64.square().mean(), (x64, w64, b64))
    rel = lambda a, r: float((a.detach().double() - r).norm() / r.norm())
    assert rel(y, y64) <= 1e-4
    assert rel(gx, rx) <= 1e-4          # native adjoint
    assert rel(gw, rw) <= 1e-3          # parameter gradients: fp32 torch.fft restatement
    # dL/dbias carries sigmoid'(bias - 9) ~ 1e-4 and can sit below fp32 resolution of the O(1) loss
    assert float((gb.double() - rb).norm()) <= 1e-3 * float(rb.norm()) + 1e-8


@pytest.mark.gpu
def test_block_is_differentiable_and_matches_its_inference_path():
    from conversenet_b200 import ConverseBlock
    torch.manual_seed(5)
    blk = ConverseBlock(64, 64, 5, scale=1, padding=4, padding_mode="replicate").cuda()
    x = torch.randn(2, 64, 128, 128, device="cuda")
    with torch.no_grad():
        fused = blk(x)
    xg = x.clone().requires_grad_(True)
    tf32 = (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32)
    torch.backends.cudnn.allow_tf32 = False   # the unfused route runs PyTorch's 1x1 convolutions
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        out = blk(xg)
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = tf32
    assert float((out - fused).norm() / fused.norm()) <= 1e-5
    g = torch.autograd.grad(out.square().mean(), xg)[0]
    assert torch.isfinite(g).all() and float(g.abs().max()) > 0


@pytest.mark.gpu
def test_registered_op_is_differentiable_through_x_and_x0():
    """`torch.ops.converse2d.forward(pad(x), interpolate(pad(x)), ...)`, the way the reference module
    calls its extension (`models/util_converse.py:160-170`): the gradient reaching x must be the total one."""
    import torch.nn.functional as F
    import conversenet_b200.torch_converse2d  # noqa: F401  (registers the op)
    torch.manual_seed(8)
    B, C, H, W, k, s, p = 2, 3, 20, 28, 5, 2, 2
    weight = torch.softmax(torch.randn(1, C, k * k, device="cuda"), -1).view(1, C, k, k)
    bias = torch.randn(1, C, 1, 1, device="cuda") * 0.3
    x = torch.randn(B, C, H, W, device="cuda", requires_grad=True)
    y = F.pad(x, (p, p, p, p), mode="circular")
    x0 = F.interpolate(y, scale_factor=s, mode="nearest")
    out = torch.ops.converse2d.forward(y, x0, weight, bias, s, 1e-5)[..., p * s:-p * s, p * s:-p * s]
    gx = torch.autograd.grad(out.square().mean(), x)[0]
    x64 = x.detach().double().requires_grad_(True)
    ref = spectral_forward(x64, weight.double(), bias.double(), s, p, "circular", 1e-5)
    rx = torch.autograd.grad(ref.square().mean(), x64)[0]
    assert float((out.detach().double() - ref).norm() / ref.norm()) <= 1e-4
    assert float((gx.double() - rx).norm() / rx.norm()) <= 1e-4
