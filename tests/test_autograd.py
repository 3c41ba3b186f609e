"""Gradients of Converse2D against gradients of the unmodified reference.

`tests/golden/converse2d_ref_grads.npz` (written by tests/golden/make_golden.py from the imported
reference, fp64, loss = y^2 mean: the protocol of the reference's `test/test_error.py:50-54`, plus its
gradcheck case `:140-153`) holds dL/dx, dL/dweight and dL/dbias.  CPU: the torch.fft restatement that
is the fallback for parameter gradients is pinned to them; GPU: the module's gradients (native dL/dx,
parameter gradients from the native batch-summed cross spectrum) are."""
import ast
import os

import numpy as np
import pytest
import torch

from conversenet_b200.autograd import spectral_forward
from oracle import converse2d_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _grad_cases():
    z = np.load(os.path.join(ROOT, "tests", "golden", "converse2d_ref_grads.npz"))
    return z, ast.literal_eval(str(z["meta"]))


N_GRAD_CASES = 8


@pytest.mark.parametrize("j", range(N_GRAD_CASES))
def test_restatement_gradients_match_reference_gradients(j):
    z, meta = _grad_cases()
    assert len(meta) == N_GRAD_CASES
    c = meta[j]
    x = torch.from_numpy(z[f"x{j}"]).double().requires_grad_(True)
    w = torch.from_numpy(z[f"w{j}"]).double().requires_grad_(True)
    b = torch.from_numpy(z[f"b{j}"]).double().requires_grad_(True)
    y = spectral_forward(x, w, b, c["s"], c["p"], c["mode"], c["eps"])
    gx, gw, gb = torch.autograd.grad(y.square().mean(), (x, w, b))
    assert orc.rel_l2(y.detach().numpy(), z[f"y{j}"]) <= 1e-9
    assert orc.rel_l2(gx.numpy(), z[f"gx{j}"]) <= 1e-8
    assert orc.rel_l2(gw.numpy(), z[f"gw{j}"]) <= 1e-7
    # dL/dbias is ~1e-12 where lambda is dominated by eps; the reference's own fp64 value then carries
    # the cancellation noise of its division by lambda (`models/util_converse.py:186`), ~1e-15 absolute
    rb = z[f"gb{j}"]
    assert float(np.linalg.norm(gb.numpy() - rb)) <= 1e-7 * float(np.linalg.norm(rb)) + 1e-14


@pytest.mark.gpu
@pytest.mark.parametrize("j", range(N_GRAD_CASES))
def test_module_gradients_match_reference_gradients(j):
    from conversenet_b200 import Converse2D
    z, meta = _grad_cases()
    c = meta[j]
    m = Converse2D(c["C"], c["C"], c["k"], scale=c["s"], padding=c["p"], padding_mode=c["mode"], eps=c["eps"]).cuda()
    with torch.no_grad():
        m.weight.copy_(torch.from_numpy(z[f"w{j}"]))
        m.bias.copy_(torch.from_numpy(z[f"b{j}"]))
    x = torch.from_numpy(z[f"x{j}"]).cuda().requires_grad_(True)
    y = m(x)
    gx, gw, gb = torch.autograd.grad(y.square().mean(), (x, m.weight, m.bias))
    assert orc.rel_l2(y.detach().cpu().numpy(), z[f"y{j}"]) <= 1e-4
    assert orc.rel_l2(gx.cpu().numpy(), z[f"gx{j}"]) <= 1e-4     # native adjoint
    assert orc.rel_l2(gw.cpu().numpy(), z[f"gw{j}"]) <= 1e-3     # parameter gradients in fp32
    rb = z[f"gb{j}"]
    # dL/dbias carries sigmoid'(bias - 9), ~1e-4 at the default bias: below fp32 resolution of the loss
    assert float(np.linalg.norm(gb.cpu().numpy().astype(np.float64) - rb)) <= 1e-3 * float(np.linalg.norm(rb)) + 1e-8


@pytest.mark.gpu
def test_usrnet_data_step_is_differentiable():
    """The data step with per-sample kernels: gradients reach x, the kernels and alpha, as in the
    reference (`models/converse_usrnet.py:41-68`, torch.fft under autograd)."""
    from conversenet_b200.models.converse_usrnet import ConvReverseDataNet
    torch.manual_seed(4)
    B, C, H, W, ks = 2, 64, 16, 20, 7
    d = ConvReverseDataNet().cuda()
    with torch.no_grad():
        d.alpha.copy_(9.0 + torch.randn_like(d.alpha))
    k = torch.softmax(torch.randn(B, C, ks * ks, device="cuda"), -1).view(B, C, ks, ks).requires_grad_(True)
    x = torch.randn(B, C, H, W, device="cuda", requires_grad=True)
    for sf in (1, 2):
        out = d(x, k, sf)
        assert out.grad_fn is not None
        gx, gk, ga = torch.autograd.grad(out.square().mean(), (x, k, d.alpha))
        x64 = x.detach().double().requires_grad_(True)
        k64 = k.detach().double().requires_grad_(True)
        a64 = d.alpha.detach().double().requires_grad_(True)
        ref = spectral_forward(x64.reshape(1, B * C, H, W), k64.reshape(1, B * C, ks, ks),
                               a64.expand(B, C, 1, 1).reshape(1, B * C, 1, 1), sf, 0, "circular", d.eps)
        rx, rk, ra = torch.autograd.grad(ref.square().mean(), (x64, k64, a64))
        rel = lambda a, r: float((a.detach().double() - r).norm() / r.norm())
        assert rel(out.reshape(1, B * C, H * sf, W * sf), ref) <= 1e-4
        assert rel(gx, rx) <= 1e-4
        assert rel(gk, rk) <= 1e-3
        assert rel(ga, ra) <= 1e-2


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
    assert rel(gw, rw) <= 1e-3          # parameter gradients in fp32 (native cross spectrum, or the fallback)
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


@pytest.mark.gpu
@pytest.mark.parametrize("scale", [1, 2])
def test_registered_op_partial_gradients_with_independent_x0(scale):
    """x0 that is NOT the up-sampled x (the raw op accepts it, `converse2d.cpp:165,193`): the gradients of x
    and of x0 are separate partial derivatives, checked against fp64 autograd of the torch.fft restatement
    of the reference's solve (oracle/ref_networks.py)."""
    import conversenet_b200.torch_converse2d  # noqa: F401  (registers the op)
    from oracle import ref_networks as rn
    torch.manual_seed(9)
    B, C, h, w, k = 2, 3, 20, 24, 5
    weight = torch.softmax(torch.randn(1, C, k * k, device="cuda"), -1).view(1, C, k, k)
    bias = torch.randn(1, C, 1, 1, device="cuda") * 0.3
    x = torch.randn(B, C, h, w, device="cuda", requires_grad=True)
    x0 = torch.randn(B, C, scale * h, scale * w, device="cuda", requires_grad=True)
    out = torch.ops.converse2d.forward(x, x0, weight, bias, scale, 1e-5)
    gx, gx0 = torch.autograd.grad(out.square().mean(), (x, x0))
    x64 = x.detach().double().requires_grad_(True)
    x064 = x0.detach().double().requires_grad_(True)
    lam = torch.sigmoid(bias.double() - 9.0) + 1e-5
    ref = rn.solve(x64, x064, weight.double(), lam, scale)
    rx, rx0 = torch.autograd.grad(ref.square().mean(), (x64, x064))
    rel = lambda a, r: float((a.detach().double() - r).norm() / r.norm())
    assert rel(out, ref) <= 1e-4
    assert rel(gx, rx) <= 1e-4
    assert rel(gx0, rx0) <= 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("shape,p,mode", [
    ((3, 4, 30, 38), 2, "replicate"),
    ((16, 64, 64, 64), 2, "circular"),      # the benchmark layer's planes (68 x 68)
    ((2, 3, 64, 64), 6, "reflect"),         # 76 x 76 = (19*4)^2: a ConverseDnCNN training patch
    ((5, 2, 100, 90), 0, "circular"),
    ((6, 3, 128, 128), 4, "replicate"),     # 136 x 136: one plane in shared memory, sums by atomics
    ((3, 2, 128, 128), 2, "circular"),      # 132 x 132
])
def test_cross_spectrum_matches_torch_fft(shape, p, mode):
    from conversenet_b200 import functional as CF
    from conversenet_b200.autograd import _pad
    torch.manual_seed(5)
    B, C, H, W = shape
    h, w = H + 2 * p, W + 2 * p
    assert CF.cross_spectrum_supported(h, w)
    x = torch.randn(shape, device="cuda")
    q = torch.randn(B, C, h, w, device="cuda") * 1e-5     # a gradient's magnitude
    weight = torch.randn(1, C, 3, 3, device="cuda")
    bias = torch.zeros(1, C, 1, 1, device="cuda")
    table, _ = CF.build_transfer(weight, bias, 1, 1e-5, h, w)
    got = CF.cross_spectrum(x, q, table, p, mode)
    ref = (torch.fft.fft2(_pad(x.double(), p, mode)) * torch.fft.fft2(q.double()).conj()).sum(0)
    assert got.shape == ref.shape
    assert float((got.to(torch.complex128) - ref).norm() / ref.norm()) <= 2e-5


@pytest.mark.gpu
def test_cross_spectrum_refuses_planes_it_has_no_kernel_for():
    from conversenet_b200 import functional as CF
    assert not CF.cross_spectrum_supported(268, 268)     # multi-pass planes
    assert not CF.cross_spectrum_supported(264, 264)     # one plane exceeds shared memory
    x = torch.randn(1, 1, 256, 256, device="cuda")
    q = torch.randn(1, 1, 268, 268, device="cuda")
    table, _ = CF.build_transfer(torch.randn(1, 1, 3, 3, device="cuda"), torch.zeros(1, 1, 1, 1, device="cuda"),
                                 1, 1e-5, 268, 268)
    with pytest.raises(RuntimeError):
        CF.cross_spectrum(x, q, table, 6, "circular")


@pytest.mark.gpu
@pytest.mark.parametrize("case", [
    (4, 8, 64, 64, 5, 1, 2, "circular"),
    (16, 64, 64, 64, 5, 2, 2, "circular"),   # the benchmark layer
    (3, 4, 64, 64, 7, 1, 6, "circular"),     # ConverseDnCNN's layer on a 64 x 64 patch
    (2, 3, 30, 44, 3, 2, 1, "replicate"),
    (3, 2, 24, 40, 2, 2, 2, "replicate"),    # even kernel
    (2, 2, 40, 24, 5, 3, 2, "reflect"),
    (2, 2, 33, 45, 3, 1, 0, "circular"),     # odd plane sizes
    (4, 2, 128, 128, 5, 1, 4, "replicate"),  # 136 x 136 (ConverseMSRResNet body on 128 x 128 patches)
    (2, 2, 64, 64, 5, 2, 2, "replicate"),
])
def test_native_parameter_gradients_match_the_torch_fft_route(case):
    """dL/dweight, dL/dbias from the native cross spectrum against autograd through the restatement
    (fp32 on the GPU, and fp64)."""
    from conversenet_b200 import autograd as AG
    B, C, H, W, k, s, p, mode = case
    torch.manual_seed(9)
    weight = torch.randn(1, C, k, k, device="cuda") * 0.2
    bias = torch.randn(1, C, 1, 1, device="cuda") * 0.5
    x = torch.randn(B, C, H, W, device="cuda")
    g = torch.randn(B, C, H * s, W * s, device="cuda")
    native = AG.grad_params(x, g, weight, bias, s, p, mode, 1e-5)
    assert native is not None
    w64 = weight.double().requires_grad_(True)
    b64 = bias.double().requires_grad_(True)
    out = AG.spectral_forward(x.double(), w64, b64, s, p, mode, 1e-5)
    rw, rb = torch.autograd.grad(out, (w64, b64), g.double())
    ew = float((native[0].double() - rw).norm() / rw.norm())
    eb = float((native[1].double() - rb).norm() / rb.norm())
    assert ew <= 2e-5 and eb <= 2e-4, (ew, eb)
    # and the switch really selects the route
    m_w = weight.clone().requires_grad_(True)
    m_b = bias.clone().requires_grad_(True)
    from conversenet_b200 import functional as CF
    table, wf = CF.build_transfer(m_w, m_b, s, 1e-5, H + 2 * p, W + 2 * p)
    outs = []
    for flag in (True, False):
        AG.NATIVE_PARAM_GRADS = flag
        try:
            y = AG.Converse2DFunction.apply(x, m_w, m_b, table, wf, k, s, p, mode, 1e-5)
            outs.append(torch.autograd.grad(y, (m_w, m_b), g))
        finally:
            AG.NATIVE_PARAM_GRADS = True
    assert float((outs[0][0] - outs[1][0]).norm() / outs[1][0].norm()) <= 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("case", [(3, 4, 20, 26, 5, 2), (2, 2, 17, 12, 2, 2), (5, 3, 12, 10, 7, 3), (1, 2, 9, 9, 3, 4),
                                  (2, 2, 14, 11, 4, 2), (2, 1, 10, 10, 9, 2)])
def test_tap_gradient_matches_the_sliced_products(case):
    import torch.nn.functional as F
    from conversenet_b200 import functional as CF
    B, C, h, w, k, s = case
    torch.manual_seed(2)
    g_full = torch.randn(B, C, s * h, s * w, device="cuda")
    r = torch.randn(B, C, h, w, device="cuda")
    got = CF.tap_gradient(g_full, r, k, s)
    c = k // 2
    gp = F.pad(g_full.double(), (k - 1 - c, c, k - 1 - c, c), mode="circular")
    ref = torch.empty(C, k, k, dtype=torch.float64, device="cuda")
    for a in range(k):
        for b in range(k):
            ref[:, a, b] = (gp[..., (k - 1 - a)::s, (k - 1 - b)::s][..., :h, :w] * r.double()).sum(dim=(0, 2, 3))
    assert float((got.double() - ref).norm() / ref.norm()) <= 1e-5
