"""The allocation-free entry point against the regular one.

`cvb_converse2d_fwd_static_scratch` is for callers that cannot allocate device memory
where they run the operator (a plug-in that owns only its input and output buffers, a
region whose memory pool is frozen, a loop that must not take the allocator lock): the
multi-pass kernels then use a fixed scratch array inside the library.  The test drives it
through the C ABI with caller-owned buffers only, twice in a row (the array is shared and
keeps the previous call's contents), and compares with `cvb_converse2d_fwd`.

Collected last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import converse2d_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 1e-4  # relative L2, the fp32 bar used by the other GPU tests
PAD = {"circular": 0, "replicate": 1, "reflect": 2, "constant": 3}


def _buffers(cfg, seed):
    from conversenet_b200 import functional as CF
    rng = np.random.default_rng(seed)
    w, b = orc.init_weight(cfg["C"], cfg["k"], rng)
    x = rng.standard_normal((cfg["B"], cfg["C"], cfg["H"], cfg["W"])).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    h, wd = cfg["H"] + 2 * cfg["p"], cfg["W"] + 2 * cfg["p"]
    table, wf = CF.build_transfer(torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda(), cfg["s"], cfg["eps"], h, wd)
    return x, w, b, xd, table, wf


def _call_static(lib, cfg, xd, table, wf, out):
    stream = torch.cuda.current_stream().cuda_stream
    return lib.cvb_converse2d_fwd_static_scratch(
        xd.data_ptr(), out.data_ptr(), table.data_ptr(), wf.data_ptr(), cfg["B"], cfg["C"], cfg["H"], cfg["W"],
        cfg["k"], cfg["s"], cfg["p"], PAD[cfg["mode"]], 0, 0, ctypes.c_void_p(stream))


@pytest.mark.parametrize("cfg", [
    dict(B=3, C=4, H=256, W=256, k=7, s=1, p=6, mode="circular", eps=1e-5),    # 268 x 268: large-prime stages
    dict(B=2, C=6, H=64, W=96, k=5, s=2, p=2, mode="replicate", eps=1e-5),     # upsampling epilogue
])
def test_static_scratch_entry_matches_regular_entry(cfg):
    from conversenet_b200 import _cabi
    from conversenet_b200 import functional as CF
    lib = _cabi.load()
    x, w, b, xd, table, wf = _buffers(cfg, 31)
    ref = CF.converse2d_forward(xd, table, wf, cfg["k"], cfg["s"], cfg["p"], cfg["mode"])
    shape = (cfg["B"], cfg["C"], cfg["H"] * cfg["s"], cfg["W"] * cfg["s"])
    # second input so that the second call does not just find the first call's scratch contents
    xd2 = torch.flip(xd, dims=(0, 3)).contiguous() * 1.5
    ref2 = CF.converse2d_forward(xd2, table, wf, cfg["k"], cfg["s"], cfg["p"], cfg["mode"])
    out1 = torch.full(shape, float("nan"), device="cuda")
    out2 = torch.full(shape, float("nan"), device="cuda")
    torch.cuda.synchronize()
    assert _call_static(lib, cfg, xd, table, wf, out1) == 0
    assert _call_static(lib, cfg, xd2, table, wf, out2) == 0
    torch.cuda.synchronize()
    assert lib.cvb_last_device_status(1) == 0   # no bounded wait gave up inside the kernels
    assert orc.rel_l2(out1.cpu().numpy(), ref.cpu().numpy()) <= TOL
    assert orc.rel_l2(out2.cpu().numpy(), ref2.cpu().numpy()) <= TOL
    oracle = orc.converse2d_forward(x, w, b, cfg["s"], cfg["p"], cfg["mode"], cfg["eps"], dtype=np.float64)
    assert orc.rel_l2(out1.cpu().numpy(), oracle) <= TOL


def test_static_scratch_entry_refuses_oversized_plane():
    from conversenet_b200 import _cabi
    lib = _cabi.load()
    one = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    # 2048 x 2048 padded plane pair = 32 MiB > the 16 MiB array
    rc = lib.cvb_converse2d_fwd_static_scratch(one, one, one, one, 1, 1, 2048, 2048, 3, 1, 0, 0, 0, 0, None)
    assert rc == -7
    assert b"scratch" in lib.cvb_strerror(rc)
