"""The tensor-core multi-pass kernels (padded lengths 4 * R0 with R0 in the registry: 268, 512 and 516)
against the numpy oracle, through the C ABI: square and non-square planes, an unpaired plane (odd
batch), every padding mode, bf16 tensors, the fused GELU and the scale >= 2 epilogue kernel."""
import numpy as np
import pytest
import torch

from oracle import converse2d_oracle as orc

pytestmark = pytest.mark.gpu

CASES = [
    dict(B=2, C=3, H=256, W=256, k=7, s=1, p=6, mode="circular"),      # 268 x 268, the ConverseDnCNN layer
    dict(B=3, C=2, H=256, W=500, k=7, s=1, p=6, mode="reflect"),       # 268 x 512: two plans, unpaired plane
    dict(B=2, C=1, H=512, W=512, k=7, s=1, p=0, mode="circular"),      # 512 x 512, the USRNet data step
    dict(B=1, C=2, H=500, W=256, k=3, s=1, p=6, mode="replicate"),     # 512 x 268
    dict(B=2, C=2, H=264, W=264, k=5, s=2, p=2, mode="constant"),      # 268 x 268 at scale 2: epilogue kernel
    dict(B=2, C=2, H=512, W=512, k=3, s=1, p=2, mode="circular"),      # 516 x 516, the USRNet blocks' layer
    dict(B=1, C=1, H=512, W=264, k=3, s=1, p=2, mode="replicate"),     # 516 x 268
]


def _run(c, x, w, b, dtype=torch.float32, gelu=False):
    from conversenet_b200 import functional as CF
    h, wd = c["H"] + 2 * c["p"], c["W"] + 2 * c["p"]
    table, wf = CF.build_transfer(torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda(), c["s"], 1e-5, h, wd)
    out = CF.converse2d_forward(torch.from_numpy(x).cuda().to(dtype), table, wf, c["k"], c["s"], c["p"], c["mode"],
                                fuse_gelu=gelu)
    torch.cuda.synchronize()
    return out.float().cpu().numpy()


@pytest.mark.parametrize("c", CASES, ids=lambda c: "%dx%d_s%d_%s" % (c["H"] + 2 * c["p"], c["W"] + 2 * c["p"], c["s"], c["mode"]))
def test_tensor_core_multipass_matches_oracle(c):
    from conversenet_b200 import _cabi
    lib = _cabi.load()
    assert lib.cvb_fits_shared(c["H"] + 2 * c["p"], c["W"] + 2 * c["p"]) == 0
    radices = (np.ctypeslib.ctypes.c_int * 8)()
    rng = np.random.default_rng(7)
    w, b = orc.init_weight(c["C"], c["k"], rng)
    b = b + rng.standard_normal(b.shape).astype(np.float32)
    x = rng.standard_normal((c["B"], c["C"], c["H"], c["W"])).astype(np.float32)
    ref = orc.converse2d_forward(x, w, b, c["s"], c["p"], c["mode"], 1e-5, dtype=np.float64)
    out = _run(c, x, w, b)
    assert lib.cvb_last_device_status(1) == 0
    assert orc.rel_l2(out, ref) <= 1e-4          # fp32 bar; measured 2e-6 .. 4e-6 (TF32 hi/lo split products)
    if c["s"] == 1:
        outg = _run(c, x, w, b, gelu=True)
        assert orc.rel_l2(outg, torch.nn.functional.gelu(torch.from_numpy(ref)).numpy()) <= 1e-4
    xb = torch.from_numpy(x).bfloat16().float().numpy()
    refb = orc.converse2d_forward(xb, w, b, c["s"], c["p"], c["mode"], 1e-5, dtype=np.float64)
    outb = _run(c, xb, w, b, dtype=torch.bfloat16)
    assert orc.rel_l2(outb, refb) <= 5e-3        # bf16 tensors, fp32 spectra
    assert lib.cvb_last_device_status(1) == 0
