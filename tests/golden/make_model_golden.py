#!/usr/bin/env python3
"""Generate `model_ref_cases.npz`: outputs of the UNMODIFIED reference networks.

Imports the reference's model files (checkout named by CONVERSE_REFERENCE_ROOT), builds each network
under `torch.manual_seed(seed)` (random init as the reference's constructors do it),
runs it in fp32 and fp64 on small seeded inputs and stores inputs, outputs and a
parameter checksum.  The tests rebuild the same parameters from the same seed with
this repo's mirrors (identical construction order), so no weights are stored.
ConverseUSRNet / ConverseNet blocks are multiplied by `alpha = 0` at init
(`models/util_converse.py:303-304`); the alphas are therefore re-drawn after
construction so that the blocks take part.
"""
import os, sys
import numpy as np
import torch

sys.dont_write_bytecode = True
REF = os.environ.get("CONVERSE_REFERENCE_ROOT")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set CONVERSE_REFERENCE_ROOT to the reference checkout")
sys.path.insert(0, REF)
from models.converse_dncnn import ConverseDnCNN  # noqa: E402
from models.converse_srresnet import ConverseMSRResNet  # noqa: E402
from models.converse_usrnet import ConverseUSRNet, ConverseNet  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def seed_alphas(model, seed):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith("alpha1") or n.endswith("alpha2"):
                p.copy_(0.1 * torch.randn(p.shape, generator=g))
            elif n.endswith("d.alpha"):
                p.copy_(9.0 + torch.randn(p.shape, generator=g))


def checksum(model):
    return float(sum(p.detach().double().abs().sum() for p in model.parameters()))


def run(model, args, dtype):
    m = model.to(dtype)
    with torch.no_grad():
        a = [t.to(dtype) if torch.is_tensor(t) and t.is_floating_point() else t for t in args]
        return m(*a).contiguous().numpy()


def usr_forward_fp64_patch():
    # KernelNet.forward casts k to float32 (`models/converse_usrnet.py:134`); follow the weights' dtype instead
    from models import converse_usrnet as cu
    def fwd(self, k):
        k = k.to(self.fc1.weight.dtype)
        b = k.shape[0]
        k = k.view(b, -1)
        k = self.gelu(self.fc1(k)); k = self.gelu(self.fc2(k)); k = self.fc3(k)
        return k.view(b, 16, self.kernel_size, self.kernel_size)
    cu.KernelNet.forward = fwd


def main():
    out = {}
    g = torch.Generator().manual_seed(7)
    # DnCNN: 2 x 1 x 32 x 32
    torch.manual_seed(101); m = ConverseDnCNN().eval()
    x = torch.rand(2, 1, 32, 32, generator=g)
    out["dncnn_x"] = x.numpy(); out["dncnn_sum"] = checksum(m)
    out["dncnn_ref32"] = run(m, (x,), torch.float32); out["dncnn_ref64"] = run(m, (x,), torch.float64)
    # SRResNet: 1 x 3 x 16 x 16 -> 64 x 64
    torch.manual_seed(102); m = ConverseMSRResNet().eval()
    x = torch.rand(1, 3, 16, 16, generator=g)
    out["srres_x"] = x.numpy(); out["srres_sum"] = checksum(m)
    out["srres_ref32"] = run(m, (x,), torch.float32); out["srres_ref64"] = run(m, (x,), torch.float64)
    # USRNet: 2 x 3 x 24 x 24 with 7x7 kernels, sf 1 and sf 2 (input 12 x 12)
    usr_forward_fp64_patch()
    k = torch.rand(2, 1, 7, 7, generator=g); k = k / k.sum(dim=(-2, -1), keepdim=True)
    out["usr_k"] = k.numpy()
    for sf, hw in [(1, 24), (2, 12)]:
        torch.manual_seed(103); m = ConverseUSRNet().eval(); seed_alphas(m, 5)
        x = torch.rand(2, 3, hw, hw, generator=g)
        out[f"usr{sf}_x"] = x.numpy(); out["usr_sum"] = checksum(m)
        out[f"usr{sf}_ref32"] = run(m, (x, k, sf), torch.float32)
        out[f"usr{sf}_ref64"] = run(m, (x, k, sf), torch.float64)
    # ConverseNet: 1 x 3 x 20 x 28
    torch.manual_seed(104); m = ConverseNet().eval()
    x = torch.rand(1, 3, 20, 28, generator=g)
    out["cnet_x"] = x.numpy(); out["cnet_sum"] = checksum(m)
    out["cnet_ref32"] = run(m, (x,), torch.float32); out["cnet_ref64"] = run(m, (x,), torch.float64)
    path = os.path.join(HERE, "model_ref_cases.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path) / 1e3, "KB")
    for k_ in out:
        if k_.endswith("ref32"):
            r64 = out[k_[:-2] + "64"]
            print(k_, "ref32 vs ref64 rel L2 = %.2e" % (np.linalg.norm(out[k_] - r64) / np.linalg.norm(r64)))


if __name__ == "__main__":
    main()
