"""Whole networks (this repo's mirrors on the GPU) against outputs of the unmodified reference.

The fixtures hold the reference's fp32 and fp64 outputs on seeded inputs
(tests/golden/make_model_golden.py); parameters are re-created from the same seed and
checked by a checksum.  At random init the reference's own fp32 run drifts 0.5-2.3e-4
from its fp64 run, so the bar is: ours-vs-fp64 <= max(1e-4, that drift)."""
import os

import numpy as np
import pytest
import torch

from oracle import converse2d_oracle as orc

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def fx():
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    return np.load(os.path.join(ROOT, "tests", "golden", "model_ref_cases.npz"))


def _checksum(m):
    return float(sum(p.detach().double().abs().sum() for p in m.parameters()))


def _seed_alphas(model, seed):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith("alpha1") or n.endswith("alpha2"):
                p.copy_(0.1 * torch.randn(p.shape, generator=g))
            elif n.endswith("d.alpha"):
                p.copy_(9.0 + torch.randn(p.shape, generator=g))


def _check(out, ref32, ref64):
    drift = orc.rel_l2(ref32, ref64)
    assert out.shape == ref64.shape
    assert orc.rel_l2(out, ref64) <= max(1e-4, drift)
    assert orc.rel_l2(out, ref32) <= max(2e-4, 2 * drift)


def test_converse_dncnn(fx):
    from conversenet_b200.models import ConverseDnCNN
    torch.manual_seed(101)
    m = ConverseDnCNN().eval()
    assert abs(_checksum(m) - float(fx["dncnn_sum"])) <= 1e-6 * float(fx["dncnn_sum"])
    with torch.no_grad():
        out = m.cuda()(torch.from_numpy(fx["dncnn_x"]).cuda()).cpu().numpy()
    _check(out, fx["dncnn_ref32"], fx["dncnn_ref64"])


def test_converse_srresnet(fx):
    from conversenet_b200.models import ConverseMSRResNet
    torch.manual_seed(102)
    m = ConverseMSRResNet().eval()
    assert abs(_checksum(m) - float(fx["srres_sum"])) <= 1e-6 * float(fx["srres_sum"])
    with torch.no_grad():
        out = m.cuda()(torch.from_numpy(fx["srres_x"]).cuda()).cpu().numpy()
    _check(out, fx["srres_ref32"], fx["srres_ref64"])


@pytest.mark.parametrize("sf", [1, 2])
def test_converse_usrnet(fx, sf):
    from conversenet_b200.models import ConverseUSRNet
    torch.manual_seed(103)
    m = ConverseUSRNet().eval()
    _seed_alphas(m, 5)
    assert abs(_checksum(m) - float(fx["usr_sum"])) <= 1e-6 * float(fx["usr_sum"])
    with torch.no_grad():
        out = m.cuda()(torch.from_numpy(fx[f"usr{sf}_x"]).cuda(), torch.from_numpy(fx["usr_k"]).cuda(), sf)
    _check(out.cpu().numpy(), fx[f"usr{sf}_ref32"], fx[f"usr{sf}_ref64"])


def test_conversenet_blind(fx):
    from conversenet_b200.models import ConverseNet
    torch.manual_seed(104)
    m = ConverseNet().eval()
    assert abs(_checksum(m) - float(fx["cnet_sum"])) <= 1e-6 * float(fx["cnet_sum"])
    with torch.no_grad():
        out = m.cuda()(torch.from_numpy(fx["cnet_x"]).cuda()).cpu().numpy()
    _check(out, fx["cnet_ref32"], fx["cnet_ref64"])


def test_fused_block_matches_unfused(monkeypatch):
    # ConverseBlock through the three fused kernels vs the same module with torch's LayerNorm / 1x1 / GELU
    from conversenet_b200 import ConverseBlock, ConverseBlockAlphaVariant
    from conversenet_b200 import util_converse as uc
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    for cls in (ConverseBlock, ConverseBlockAlphaVariant):
        torch.manual_seed(3)
        blk = cls(64, 64, kernel_size=5, padding=4, padding_mode="replicate").cuda().eval()
        with torch.no_grad():
            for n, p in blk.named_parameters():
                if "alpha" in n:
                    p.copy_(0.3 * torch.randn_like(p))
                if n in ("conv1.0.weight", "conv2.0.weight", "conv1.0.bias", "conv2.0.bias"):
                    p.add_(0.2 * torch.randn_like(p))
        x = torch.randn(3, 64, 37, 29, device="cuda")
        with torch.no_grad():
            fused = blk(x)
            monkeypatch.setattr(uc, "BLOCK_FUSION", False)
            plain = blk(x)
            monkeypatch.setattr(uc, "BLOCK_FUSION", True)
        assert float((fused - plain).norm() / plain.norm()) <= 5e-6
        with torch.no_grad():
            fb = blk(x.bfloat16()).float()
        assert float((fb - plain).norm() / plain.norm()) <= 2e-2


def test_tensor_core_kernel_matches_cuda_core_kernel(monkeypatch):
    # LN + 1x1 + GELU on tcgen05 (TF32 hi/lo split, three MMAs per product) vs the fp32 CUDA-core kernel
    from conversenet_b200 import functional as CF, _cabi
    from conversenet_b200.util_converse import LayerNorm
    torch.manual_seed(5)
    ln = LayerNorm(64, eps=1e-5, data_format="channels_first").cuda()
    conv = torch.nn.Conv2d(64, 128, 1).cuda()
    with torch.no_grad():
        ln.weight.add_(0.3 * torch.randn_like(ln.weight))
        ln.bias.add_(0.2 * torch.randn_like(ln.bias))
    x = torch.randn(3, 64, 64, 96, device="cuda")   # 6144 pixels per image: whole 128-pixel tiles
    with _cabi.option(_cabi.OPT_BLOCK_KERNELS, 0):
        ref = CF.ln_pw_gelu(x, ln, conv)
    with _cabi.option(_cabi.OPT_BLOCK_KERNELS, 1):    # single-buffered kernel
        out1 = CF.ln_pw_gelu(x, ln, conv)
    assert _cabi.load().cvb_get_option(_cabi.OPT_BLOCK_KERNELS) == 3   # default: operand in tensor memory
    with _cabi.option(_cabi.OPT_BLOCK_KERNELS, 2):    # warp-specialised, operand tiles in shared memory
        out = CF.ln_pw_gelu(x, ln, conv)
    torch.cuda.synchronize()
    assert _cabi.load().cvb_last_device_status(1) == 0
    assert float((out1 - ref).norm() / ref.norm()) <= 3e-6
    assert float((out - ref).norm() / ref.norm()) <= 3e-6
    # 1x1 + residual (128 -> 64) on the tensor cores against PyTorch
    conv2 = torch.nn.Conv2d(128, 64, 1).cuda()
    alpha = torch.randn(1, 64, 1, 1, device="cuda")
    t = torch.randn(3, 128, 64, 96, device="cuda")
    torch.backends.cudnn.allow_tf32 = False
    want2 = x + alpha * conv2(t)
    for mode in (1, 2):
        with _cabi.option(_cabi.OPT_BLOCK_KERNELS, mode):
            got2 = CF.pw_res(t, x, conv2, alpha)
        assert float((got2 - want2).norm() / want2.norm()) <= 5e-6
    assert _cabi.load().cvb_last_device_status(1) == 0
    # torch fp32 reference of the same op
    u = x.mean(1, keepdim=True)
    s = (x - u).pow(2).mean(1, keepdim=True)
    xn = ln.weight[:, None, None] * ((x - u) / torch.sqrt(s + 1e-5)) + ln.bias[:, None, None]
    torch.backends.cudnn.allow_tf32 = False
    want = torch.nn.functional.gelu(conv(xn))
    assert float((out - want).norm() / want.norm()) <= 5e-6


def test_tensor_core_block_kernels_with_bf16_tensors():
    """The tcgen05 1x1 kernels on bf16 tensors (fp32 arithmetic) against the same ops in fp32 PyTorch on the
    bf16-rounded inputs; the only difference is the rounding of the stored result (2^-9 relative)."""
    from conversenet_b200 import functional as CF, _cabi
    from conversenet_b200.util_converse import LayerNorm
    torch.backends.cudnn.allow_tf32 = False
    torch.manual_seed(6)
    ln = LayerNorm(64, eps=1e-5, data_format="channels_first").cuda()
    conv = torch.nn.Conv2d(64, 128, 1).cuda()
    conv2 = torch.nn.Conv2d(128, 64, 1).cuda()
    with torch.no_grad():
        ln.weight.add_(0.3 * torch.randn_like(ln.weight))
        ln.bias.add_(0.2 * torch.randn_like(ln.bias))
    x = torch.randn(2, 64, 64, 96, device="cuda").bfloat16()
    t = torch.randn(2, 128, 64, 96, device="cuda").bfloat16()
    alpha = torch.randn(1, 64, 1, 1, device="cuda")
    out = CF.ln_pw_gelu(x, ln, conv)
    got2 = CF.pw_res(t, x, conv2, alpha)
    torch.cuda.synchronize()
    assert out.dtype == torch.bfloat16 and got2.dtype == torch.bfloat16
    assert _cabi.load().cvb_last_device_status(1) == 0
    with torch.no_grad():
        want = torch.nn.functional.gelu(conv(ln(x.float())))
        want2 = x.float() + alpha * conv2(t.float())
    assert float((out.float() - want).norm() / want.norm()) <= 4e-3
    assert float((got2.float() - want2).norm() / want2.norm()) <= 4e-3
    with _cabi.option(_cabi.OPT_BLOCK_KERNELS, 0):       # the CUDA-core kernel on the same bf16 tensors
        ref = CF.ln_pw_gelu(x, ln, conv)
    assert float((out.float() - ref.float()).norm() / ref.float().norm()) <= 4e-3


def test_graphed_forward_replays_the_eager_result():
    """One CUDA-graph launch per forward (conversenet_b200/graphs.py) must reproduce the eager forward bit for bit,
    also for a second input copied into the static buffers."""
    from conversenet_b200.graphs import GraphedForward
    from conversenet_b200.models import ConverseDnCNN
    torch.backends.cudnn.allow_tf32 = False
    torch.manual_seed(11)
    net = ConverseDnCNN().cuda().eval()
    x1 = torch.rand(2, 1, 40, 56, device="cuda")
    x2 = torch.rand(2, 1, 40, 56, device="cuda")
    with torch.no_grad():
        want1, want2 = net(x1).clone(), net(x2).clone()
    g = GraphedForward(net, x1)
    assert torch.equal(g(x1).clone(), want1)
    assert torch.equal(g(x2).clone(), want2)
    with pytest.raises(RuntimeError):
        g(torch.rand(1, 1, 40, 56, device="cuda"))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_kernels_with_the_operand_in_tensor_memory(dtype):
    """Option value 3 of the block kernels (cp.async ring, LayerNorm inside one thread, operand A staged in TMEM)
    against fp32 PyTorch and against variant 2, on images of many tiles and on a single tile."""
    from conversenet_b200 import functional as CF, _cabi
    from conversenet_b200.util_converse import LayerNorm
    torch.backends.cudnn.allow_tf32 = False
    torch.manual_seed(8)
    ln = LayerNorm(64, eps=1e-5, data_format="channels_first").cuda()
    conv = torch.nn.Conv2d(64, 128, 1).cuda()
    conv2 = torch.nn.Conv2d(128, 64, 1).cuda()
    with torch.no_grad():
        ln.weight.add_(0.3 * torch.randn_like(ln.weight))
        ln.bias.add_(0.2 * torch.randn_like(ln.bias))
    alpha = torch.randn(1, 64, 1, 1, device="cuda")
    tol = 5e-6 if dtype == torch.float32 else 4e-3
    for shape in ((3, 64, 96), (1, 8, 16), (5, 128, 128)):
        B, H, W = shape
        x = torch.randn(B, 64, H, W, device="cuda").to(dtype)
        t = torch.randn(B, 128, H, W, device="cuda").to(dtype)
        with _cabi.option(_cabi.OPT_BLOCK_KERNELS, 3):
            out = CF.ln_pw_gelu(x, ln, conv)
            got2 = CF.pw_res(t, x, conv2, alpha)
        with _cabi.option(_cabi.OPT_BLOCK_KERNELS, 2):
            ref = CF.ln_pw_gelu(x, ln, conv)
            ref2 = CF.pw_res(t, x, conv2, alpha)
        torch.cuda.synchronize()
        assert _cabi.load().cvb_last_device_status(1) == 0
        with torch.no_grad():
            want = torch.nn.functional.gelu(conv(ln(x.float())))
            want2 = x.float() + alpha * conv2(t.float())
        assert float((out.float() - want).norm() / want.norm()) <= tol, shape
        assert float((got2.float() - want2).norm() / want2.norm()) <= tol, shape
        assert float((out.float() - ref.float()).norm() / ref.float().norm()) <= tol
        assert float((got2.float() - ref2.float()).norm() / ref2.float().norm()) <= tol
