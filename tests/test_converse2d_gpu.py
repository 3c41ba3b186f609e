"""Parity of the CUDA path (through the C ABI) with the oracle and the reference's golden outputs."""
import numpy as np
import pytest
import torch

from oracle import converse2d_oracle as orc

pytestmark = pytest.mark.gpu

TOL_FP32 = 1e-4   # relative L2, fp32: the stated bar of this operator against the reference's torch.fft path
TOL_BF16 = 5e-3   # relative L2, bf16 I/O with fp32 spectra


def _module(C, k, s, p, mode, eps, w, b):
    from conversenet_b200 import Converse2D
    m = Converse2D(C, C, k, scale=s, padding=p, padding_mode=mode, eps=eps).cuda().eval()
    with torch.no_grad():
        m.weight.copy_(torch.from_numpy(w))
        m.bias.copy_(torch.from_numpy(b))
    return m


def _run(x, w, b, s, p, mode, eps, dtype=torch.float32):
    m = _module(x.shape[1], w.shape[-1], s, p, mode, eps, w, b)
    with torch.no_grad():
        y = m(torch.from_numpy(x).cuda().to(dtype))
    torch.cuda.synchronize()
    return y.float().cpu().numpy()


@pytest.mark.parametrize("i", range(20))
def test_golden_cases(golden, i):
    c, x, w, b, ref32, ref64 = golden.case(i)
    out = _run(x, w, b, c["s"], c["p"], c["mode"], c["eps"])
    assert out.shape == ref32.shape
    assert orc.rel_l2(out, ref32) <= TOL_FP32
    assert orc.rel_l2(out, ref64) <= TOL_FP32


@pytest.mark.parametrize("i", [1, 4, 13, 15])
def test_golden_cases_forced_runtime_plan(golden, i):
    from conversenet_b200 import _cabi
    c, x, w, b, ref32, ref64 = golden.case(i)
    with _cabi.option(_cabi.OPT_RUNTIME_PLAN, 1):
        out = _run(x, w, b, c["s"], c["p"], c["mode"], c["eps"])
    assert orc.rel_l2(out, ref64) <= TOL_FP32


CONFIGS = {
    # the two single-layer benchmark configurations at full size, SRResNet-style layers reduced in batch
    "cfg1": dict(B=1, C=64, H=128, W=128, k=5, s=1, p=2, mode="circular", eps=1e-5),
    "cfg2": dict(B=16, C=64, H=64, W=64, k=5, s=2, p=2, mode="circular", eps=1e-5),
    "srres_body": dict(B=2, C=128, H=128, W=128, k=5, s=1, p=4, mode="replicate", eps=1e-5),
    "srres_up1": dict(B=2, C=64, H=128, W=128, k=2, s=2, p=2, mode="replicate", eps=1e-3),
    "odd_batch": dict(B=3, C=8, H=64, W=64, k=5, s=2, p=2, mode="circular", eps=1e-5),
}


LARGE = {
    # planes that take the multi-pass path (workspace): layers of the three benchmark networks, batch reduced
    "dncnn_body_268": dict(B=2, C=8, H=256, W=256, k=7, s=1, p=6, mode="circular", eps=1e-5),
    "srres_264": dict(B=2, C=6, H=256, W=256, k=5, s=1, p=4, mode="replicate", eps=1e-5),
    "srres_up2_260": dict(B=2, C=4, H=256, W=256, k=2, s=2, p=2, mode="replicate", eps=1e-3),
    "srres_520": dict(B=1, C=4, H=512, W=512, k=5, s=1, p=4, mode="replicate", eps=1e-5),
    "usrnet_block_516": dict(B=1, C=4, H=512, W=512, k=3, s=1, p=2, mode="circular", eps=1e-5),
    "usrnet_data_512": dict(B=2, C=2, H=512, W=512, k=7, s=1, p=0, mode="circular", eps=1e-3),
    "odd_rect_prime": dict(B=3, C=3, H=83, W=55, k=3, s=3, p=2, mode="reflect", eps=1e-5),  # 87 x 59
    # 268 = 67 * 4: the 67-point stage on the tensor cores; with the upsampling epilogue (halo columns in
    # the 16-line tiles, odd plane count), and mixed with a register-radix axis both ways round
    "tc_268_up2": dict(B=3, C=3, H=264, W=264, k=3, s=2, p=2, mode="replicate", eps=1e-5),
    "tc_268x264": dict(B=2, C=5, H=256, W=252, k=7, s=1, p=6, mode="circular", eps=1e-5),
    "tc_264x268": dict(B=1, C=6, H=252, W=256, k=5, s=1, p=6, mode="reflect", eps=1e-5),
}


@pytest.mark.parametrize("name", list(LARGE))
def test_large_planes_multi_pass(name):
    cfg = LARGE[name]
    x, w, b = _seeded(cfg, 4)
    out = _run(x, w, b, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"])
    ref64 = orc.converse2d_forward(x, w, b, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"], dtype=np.float64)
    assert orc.rel_l2(out, ref64) <= TOL_FP32


def test_tensor_core_stage_bf16_io_and_status_word():
    """268-wide planes with bf16 tensors; the device status word must stay clear (no bounded wait ran out)."""
    from conversenet_b200 import _cabi
    lib = _cabi.load()
    lib.cvb_last_device_status(1)
    cfg = LARGE["dncnn_body_268"]
    x, w, b = _seeded(cfg, 9)
    xb = torch.from_numpy(x).bfloat16()
    out = _run(xb.float().numpy(), w, b, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"], dtype=torch.bfloat16)
    ref = orc.converse2d_forward(xb.float().numpy(), w, b, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"],
                                 dtype=np.float32)
    ref = torch.from_numpy(ref).bfloat16().float().numpy()
    assert orc.rel_l2(out, ref) <= TOL_BF16
    torch.cuda.synchronize()
    assert lib.cvb_last_device_status(0) == 0


def test_forced_multi_pass_matches_shared_memory_path():
    from conversenet_b200 import _cabi
    cfg = CONFIGS["odd_batch"]
    x, w, b = _seeded(cfg, 6)
    for s in (1, 2):
        a = _run(x, w, b, s, cfg["p"], cfg["mode"], cfg["eps"])
        with _cabi.option(_cabi.OPT_MULTIPASS, 1):
            d = _run(x, w, b, s, cfg["p"], cfg["mode"], cfg["eps"])
        assert orc.rel_l2(d, a) <= 2e-6
    xb = torch.from_numpy(x).bfloat16().float().numpy()
    with _cabi.option(_cabi.OPT_MULTIPASS, 1):
        d = _run(xb, w, b, 2, cfg["p"], cfg["mode"], cfg["eps"], dtype=torch.bfloat16)
    a = _run(xb, w, b, 2, cfg["p"], cfg["mode"], cfg["eps"], dtype=torch.bfloat16)
    assert orc.rel_l2(d, a) <= 5e-3


def _seeded(cfg, seed=0):
    rng = np.random.default_rng(seed)
    w, b = orc.init_weight(cfg["C"], cfg["k"], rng)
    x = rng.standard_normal((cfg["B"], cfg["C"], cfg["H"], cfg["W"])).astype(np.float32)
    return x, w, b


@pytest.mark.parametrize("name", list(CONFIGS))
def test_baseline_configs_fp32(name):
    cfg = CONFIGS[name]
    x, w, b = _seeded(cfg)
    out = _run(x, w, b, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"])
    ref32 = orc.converse2d_forward(x, w, b, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"], dtype=np.float32)
    ref64 = orc.converse2d_forward(x, w, b, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"], dtype=np.float64)
    assert orc.rel_l2(out, ref32) <= TOL_FP32
    assert orc.rel_l2(out, ref64) <= TOL_FP32


@pytest.mark.parametrize("name", ["cfg2", "cfg1"])
def test_baseline_configs_bf16_io(name):
    cfg = CONFIGS[name]
    x, w, b = _seeded(cfg)
    xb = torch.from_numpy(x).bfloat16()
    out = _run(xb.float().numpy(), w, b, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"], dtype=torch.bfloat16)
    ref = orc.converse2d_forward(xb.float().numpy(), w, b, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"],
                                 dtype=np.float32)
    ref = torch.from_numpy(ref).bfloat16().float().numpy()
    assert orc.rel_l2(out, ref) <= TOL_BF16


def test_forced_runtime_plan_matches_compiled_plan():
    from conversenet_b200 import _cabi
    cfg = CONFIGS["odd_batch"]
    x, w, b = _seeded(cfg, 5)
    a = _run(x, w, b, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"])
    with _cabi.option(_cabi.OPT_RUNTIME_PLAN, 1):
        d = _run(x, w, b, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"])
    assert orc.rel_l2(a, d) <= 2e-6


def test_persistent_prefetch_kernel_matches():
    # blocks looping over plane pairs with bulk-copy (TMA) prefetch of x; bounded waits must not trip
    from conversenet_b200 import _cabi
    cfg = dict(CONFIGS["cfg2"], B=12)
    x, w, b = _seeded(cfg, 21)
    base = _run(x, w, b, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"])
    with _cabi.option(_cabi.OPT_PERSISTENT, 1):
        pers = _run(x, w, b, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"])
        assert _cabi.load().cvb_last_device_status(1) == 0
        assert orc.rel_l2(pers, base) <= 1e-6
        pers1 = _run(x, w, b, 1, cfg["p"], cfg["mode"], cfg["eps"])
    base1 = _run(x, w, b, 1, cfg["p"], cfg["mode"], cfg["eps"])
    assert _cabi.load().cvb_last_device_status(1) == 0
    assert orc.rel_l2(pers1, base1) <= 1e-6


def test_linearity_and_constant_planes_full_size():
    # size-independent properties at the bench workload's full size
    cfg = CONFIGS["cfg2"]
    x, w, b = _seeded(cfg, 11)
    x2 = np.random.default_rng(12).standard_normal(x.shape).astype(np.float32)
    m = _module(cfg["C"], cfg["k"], cfg["s"], cfg["p"], cfg["mode"], cfg["eps"], w, b)
    with torch.no_grad():
        a = m(torch.from_numpy(x).cuda())
        c = m(torch.from_numpy(x2).cuda())
        ac = m(torch.from_numpy(x + 0.5 * x2).cuda())
        const = m(torch.full(x.shape, 3.25, device="cuda"))
    assert float((ac - (a + 0.5 * c)).norm() / ac.norm()) <= 2e-6
    # a constant plane is a fixed point of the circular solve (the kernel taps sum to one)
    assert float((const - 3.25).abs().max()) <= 2e-4


def test_fused_gelu_matches_separate_gelu():
    cfg = CONFIGS["odd_batch"]
    x, w, b = _seeded(cfg, 2)
    for s in (1, 2):
        m = _module(cfg["C"], cfg["k"], s, cfg["p"], cfg["mode"], cfg["eps"], w, b)
        xt = torch.from_numpy(x).cuda()
        with torch.no_grad():
            plain = m(xt)
            m.fuse_gelu = True
            fused = m(xt)
        assert torch.allclose(fused, torch.nn.functional.gelu(plain), atol=1e-6, rtol=1e-5)


def test_table_follows_in_place_weight_update():
    cfg = CONFIGS["odd_batch"]
    x, w, b = _seeded(cfg, 3)
    m = _module(cfg["C"], cfg["k"], 1, cfg["p"], cfg["mode"], cfg["eps"], w, b)
    xt = torch.from_numpy(x).cuda()
    with torch.no_grad():
        m(xt)
        m.bias.add_(9.0)  # lambda changes from ~1.3e-4 to ~0.5
        out = m(xt).cpu().numpy()
    ref = orc.converse2d_forward(x, w, b + 9.0, 1, cfg["p"], cfg["mode"], cfg["eps"], dtype=np.float64)
    assert orc.rel_l2(out, ref) <= TOL_FP32


def test_error_behaviour_on_device():
    from conversenet_b200 import Converse2D
    m = Converse2D(2, 2, 3, padding=9, padding_mode="circular").cuda()
    with pytest.raises(RuntimeError):
        m(torch.zeros(1, 2, 8, 8, device="cuda"))      # padding wider than the plane
    m = Converse2D(2, 2, 3, padding=1).cuda()
    with pytest.raises(RuntimeError):
        m(torch.zeros(1, 2, 8, 8, device="cuda", dtype=torch.float16))  # unsupported dtype
    with pytest.raises(RuntimeError):
        m(torch.zeros(1, 3, 8, 8, device="cuda"))      # channel mismatch


def test_registered_torch_op_matches_reference_contract(golden):
    # torch.ops.converse2d.forward: padded input in, uncropped plane out (converse2d.cpp:165-209)
    import conversenet_b200.torch_converse2d  # noqa: F401  (registers the op)
    import torch.nn.functional as F
    c, x, w, b, ref32, ref64 = golden.case(9)
    p, s = c["p"], c["s"]
    y = F.pad(torch.from_numpy(x).cuda(), [p, p, p, p], mode="circular")
    x0 = y if s == 1 else F.interpolate(y, scale_factor=s, mode="nearest")
    out = torch.ops.converse2d.forward(y, x0, torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda(), s, c["eps"])
    assert tuple(out.shape) == (y.shape[0], y.shape[1], y.shape[2] * s, y.shape[3] * s)
    crop = out[..., p * s:-p * s, p * s:-p * s].cpu().numpy()
    assert orc.rel_l2(crop, ref64) <= TOL_FP32
    torch.ops.converse2d.clear_cache()
    with pytest.raises(RuntimeError):   # x0 of the wrong shape
        torch.ops.converse2d.forward(y, x0[..., :-1], torch.from_numpy(w).cuda(),
                                     torch.from_numpy(b).cuda(), s, c["eps"])


@pytest.mark.parametrize("shape,k,s", [((2, 3, 20, 26), 5, 2), ((1, 4, 32, 32), 3, 1), ((2, 2, 18, 24), 2, 2),
                                       ((1, 2, 24, 15), 5, 3)])
def test_registered_torch_op_with_an_arbitrary_x0(shape, k, s):
    """The raw operator with an x0 that is NOT the upsampled input (`converse2d.cpp:165,193`; this is what
    `test/test_error.py:30` builds): checked against the oracle's closed-form solve."""
    import conversenet_b200.torch_converse2d  # noqa: F401
    rng = np.random.default_rng(31)
    B, C, h, w = shape
    y = rng.standard_normal(shape).astype(np.float32)
    x0 = rng.standard_normal((B, C, h * s, w * s)).astype(np.float32)
    wt, b = orc.init_weight(C, k, rng)
    b = (b + 0.4 * rng.standard_normal(b.shape)).astype(np.float32)
    ref = orc.converse2d_solve(y, x0, wt, b, s, 1e-5, dtype=np.float64)
    out = torch.ops.converse2d.forward(torch.from_numpy(y).cuda(), torch.from_numpy(x0).cuda(),
                                       torch.from_numpy(wt).cuda(), torch.from_numpy(b).cuda(), s, 1e-5)
    assert orc.rel_l2(out.cpu().numpy(), ref) <= TOL_FP32
