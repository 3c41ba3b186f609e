#!/usr/bin/env python3
"""Generate `model_fullsize_cases.npz`: the UNMODIFIED reference networks at the resolutions of
the benchmark configurations, batch 1.

Needs the reference checkout (its place: the environment variable CONVERSE_REFERENCE_ROOT).
For every network -- ConverseDnCNN 1x1x256x256, ConverseMSRResNet 1x3x128x128 (-> 512x512),
ConverseUSRNet 1x3x512x512 at sf 1 and 1x3x128x128 at sf 4, ConverseNet 1x3x256x256 -- and for
both parameter sets -- seeded random init (`rand`) and the reference's trained checkpoint
(`ckpt`, `model_zoo/*.pth`, copied next to this file so that the tests can load the same
weights) -- the reference runs in fp32 and fp64 on the seeded input of `bench.synthetic_batch`.
Stored per case:
    <case>_sub    fp64 output, every third pixel of every third row, as float32
    <case>_drift  rel. L2 of the reference's fp32 output against its fp64 output (full size)
    <case>_norm   L2 norm of the fp64 output (full size)
    <case>_insum  sum of the input (guards the input recipe)
    <case>_psum   sum of |parameters|
and for ConverseDnCNN with the checkpoint the bf16 run (`dncnn_ckpt_bf16_sub`): the fp32
reference on the bf16-rounded input, its output rounded to bf16 (torch.fft has no bf16).
Sub-sampling keeps the fixture at a few MB; stride 3 meets every residue of the scale-2 and
scale-4 up-sampling phases.
"""
import os
import shutil
import sys

import numpy as np
import torch

sys.dont_write_bytecode = True
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("CONVERSE_REFERENCE_ROOT")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set CONVERSE_REFERENCE_ROOT to the reference checkout")
sys.path.insert(0, REF)
sys.path.insert(1, ROOT)
from models.converse_dncnn import ConverseDnCNN  # noqa: E402
from models.converse_srresnet import ConverseMSRResNet  # noqa: E402
from models.converse_usrnet import ConverseUSRNet, ConverseNet  # noqa: E402
from models import converse_usrnet as cu  # noqa: E402
import bench  # noqa: E402

STRIDE = 3
CASES = [  # name, workload of bench.synthetic_batch, constructor, checkpoint file, construction seed
    ("dncnn", "dncnn", ConverseDnCNN, "converse_dncnn.pth", 201),
    ("srresnet", "srresnet", ConverseMSRResNet, "converse_srresnet.pth", 202),
    ("usrnet_sf1", "usrnet_sf1", ConverseUSRNet, "converse_usrnet.pth", 203),
    ("usrnet_sf4", "usrnet_sf4", ConverseUSRNet, "converse_usrnet.pth", 203),
    ("conversenet", "conversenet", ConverseNet, "conversenet.pth", 204),
]


def seed_alphas(model, seed):
    """The alpha-variant blocks and the data step start at zero (`models/util_converse.py:303-304`,
    `models/converse_usrnet.py:40`): re-draw them so that a random-init network uses its blocks."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith("alpha1") or n.endswith("alpha2"):
                p.copy_(0.1 * torch.randn(p.shape, generator=g))
            elif n.endswith("d.alpha"):
                p.copy_(9.0 + torch.randn(p.shape, generator=g))


def kernelnet_follow_dtype():
    # KernelNet.forward casts k to float32 (`models/converse_usrnet.py:134`); follow the weights' dtype
    def fwd(self, k):
        k = k.to(self.fc1.weight.dtype)
        b = k.shape[0]
        k = k.view(b, -1)
        k = self.gelu(self.fc1(k)); k = self.gelu(self.fc2(k)); k = self.fc3(k)
        return k.view(b, 16, self.kernel_size, self.kernel_size)
    cu.KernelNet.forward = fwd


def run(model, x, extra, dtype):
    m = model.to(dtype)
    args = [torch.from_numpy(x).to(dtype)]
    if extra:
        args += [torch.from_numpy(extra[0]).to(dtype), extra[1]]
    with torch.no_grad():
        return m(*args).double().numpy()


def main():
    torch.set_num_threads(os.cpu_count() or 1)
    kernelnet_follow_dtype()
    zoo = os.path.join(HERE, "model_zoo")
    os.makedirs(zoo, exist_ok=True)
    out = {"stride": STRIDE}
    for name, wl, ctor, ckpt, seed in CASES:
        x, extra = bench.synthetic_batch(wl, 1, 700 + seed)
        for pset in ("rand", "ckpt"):
            torch.manual_seed(seed)
            m = ctor().eval()
            if pset == "rand":
                seed_alphas(m, 5)
            else:
                src = os.path.join(REF, "model_zoo", ckpt)
                shutil.copyfile(src, os.path.join(zoo, ckpt))
                m.load_state_dict(torch.load(src, map_location="cpu"), strict=True)
            key = "%s_%s" % (name, pset)
            r32 = run(m, x, extra, torch.float32)
            r64 = run(m, x, extra, torch.float64)
            out[key + "_sub"] = r64[..., ::STRIDE, ::STRIDE].astype(np.float32)
            out[key + "_drift"] = np.linalg.norm(r32 - r64) / np.linalg.norm(r64)
            out[key + "_norm"] = np.linalg.norm(r64)
            out[key + "_insum"] = float(x.astype(np.float64).sum())
            out[key + "_psum"] = float(sum(p.detach().double().abs().sum() for p in m.parameters()))
            print(key, r64.shape, "ref32 vs ref64 %.2e" % out[key + "_drift"], flush=True)
            if name == "dncnn" and pset == "ckpt":
                xb = torch.from_numpy(x).bfloat16().float().numpy()
                rb = torch.from_numpy(run(m, xb, extra, torch.float32)).bfloat16().float().numpy()
                out[key + "_bf16_sub"] = rb[..., ::STRIDE, ::STRIDE].astype(np.float32)
                print(key, "bf16-rounded run vs ref64 %.2e" % (np.linalg.norm(rb - r64) / np.linalg.norm(r64)))
    path = os.path.join(HERE, "model_fullsize_cases.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, "%.2f MB" % (os.path.getsize(path) / 1e6))


if __name__ == "__main__":
    main()
