#!/usr/bin/env python3
"""Generate `converse2d_ref_cases.npz` from the UNMODIFIED reference.

Run where the reference checkout is available (its place: CONVERSE_REFERENCE_ROOT).  Imports the reference's
`models.util_converse.Converse2D` (`backend='pytorch'`), runs it in fp32 and
fp64 on seeded inputs and stores inputs, parameters and both outputs (`--grads-only` skips this file and writes
only `converse2d_ref_grads.npz`: fp64 gradients of the reference for a subset).  The
case grid follows the reference's `test/test_error.py:92-98` (B, C, H, W, k, s
with padding=k//2, circular) thinned to keep the fixture small, plus the
padding modes, eps values, non-zero biases and even kernel sizes the models
use (`models/converse_srresnet.py:66-70`, `models/converse_usrnet.py:33-68`).
"""
import os, sys, itertools
import numpy as np
import torch

sys.dont_write_bytecode = True
REF = os.environ.get("CONVERSE_REFERENCE_ROOT")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set CONVERSE_REFERENCE_ROOT to the reference checkout")
sys.path.insert(0, REF)
from models.util_converse import Converse2D  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def run_ref(mod, x, dtype):
    m = Converse2D(mod.in_channels, mod.out_channels, mod.kernel_size, scale=mod.scale,
                   padding=mod.padding, padding_mode=mod.padding_mode, eps=mod.eps,
                   backend="pytorch").to(dtype)
    m.load_state_dict({k: v.to(dtype) for k, v in mod.state_dict().items()})
    with torch.no_grad():
        return m(x.to(dtype)).contiguous().numpy()


def cases():
    # thinned test_error.py grid: every (k, s) twice, cycling through the four
    # (H, W) pairs and the B / C values
    sizes = list(itertools.product([16, 32], [18, 40]))
    grid = list(itertools.product([3, 5], [1, 2, 3], [0, 1]))
    for i, (k, s, j) in enumerate(grid):
        H, W = sizes[(i + j) % 4]
        yield dict(B=1 + i % 2, C=2 + (i // 2) % 2, H=H, W=W, k=k, s=s, p=k // 2,
                   mode="circular", eps=1e-5, bias_std=0.0)
    # model-style layers
    yield dict(B=2, C=4, H=24, W=24, k=5, s=1, p=4, mode="replicate", eps=1e-5, bias_std=0.0)
    yield dict(B=2, C=4, H=20, W=28, k=2, s=2, p=2, mode="replicate", eps=1e-3, bias_std=0.0)
    yield dict(B=1, C=4, H=30, W=26, k=7, s=1, p=6, mode="circular", eps=1e-5, bias_std=0.0)
    yield dict(B=2, C=3, H=32, W=32, k=7, s=4, p=0, mode="circular", eps=1e-3, bias_std=2.0)
    yield dict(B=1, C=3, H=17, W=23, k=3, s=1, p=2, mode="reflect", eps=1e-5, bias_std=3.0)
    yield dict(B=3, C=2, H=19, W=21, k=4, s=2, p=3, mode="constant", eps=1e-4, bias_std=5.0)
    yield dict(B=1, C=2, H=64, W=64, k=5, s=2, p=2, mode="circular", eps=1e-5, bias_std=0.0)
    yield dict(B=1, C=2, H=13, W=13, k=3, s=1, p=0, mode="circular", eps=1e-5, bias_std=1.0)


GRAD_CASES = [1, 4, 9, 12, 13, 15, 17]   # indices into cases(): scales 1-3, every padding mode the models use


def reference_grads(c, seed):
    """Gradients of the unmodified reference in fp64 under the protocol of `test/test_error.py:50-54`
    (loss = y^2 mean): dL/dx, dL/dweight, dL/dbias, and the forward output."""
    torch.manual_seed(seed)
    mod = Converse2D(c["C"], c["C"], c["k"], scale=c["s"], padding=c["p"], padding_mode=c["mode"],
                     eps=c["eps"], backend="pytorch")
    if c["bias_std"] > 0:
        with torch.no_grad():
            mod.bias.copy_(9.0 + c["bias_std"] * torch.randn_like(mod.bias))
    x = torch.randn(c["B"], c["C"], c["H"], c["W"])
    mod = mod.double()
    x64 = x.double().requires_grad_(True)
    y = mod(x64)
    gx, gw, gb = torch.autograd.grad(y.square().mean(), (x64, mod.weight, mod.bias))
    return dict(x=x.numpy(), w=mod.weight.detach().float().numpy(), b=mod.bias.detach().float().numpy(),
                y=y.detach().numpy(), gx=gx.numpy(), gw=gw.numpy(), gb=gb.numpy())


def write_grads():
    out, meta = {}, []
    all_cases = list(cases())
    # the reference's own fp64 gradcheck case (`test/test_error.py:140-153`): 1 x 2 x 8 x 9, k 5, scale 2
    extra = dict(B=1, C=2, H=8, W=9, k=5, s=2, p=2, mode="circular", eps=1e-5, bias_std=0.0)
    for j, (c, seed) in enumerate([(all_cases[i], 1000 + i) for i in GRAD_CASES] + [(extra, 4242)]):
        for key, v in reference_grads(c, seed).items():
            out[f"{key}{j}"] = v
        meta.append(c)
    out["meta"] = np.array(repr(meta))
    path = os.path.join(HERE, "converse2d_ref_grads.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(meta)} cases, {os.path.getsize(path) / 1e6:.2f} MB")


def main():
    if "--grads-only" not in sys.argv:
        write_cases()
    write_grads()


def write_cases():
    out = {}
    meta = []
    for i, c in enumerate(cases()):
        torch.manual_seed(1000 + i)
        mod = Converse2D(c["C"], c["C"], c["k"], scale=c["s"], padding=c["p"],
                         padding_mode=c["mode"], eps=c["eps"], backend="pytorch")
        if c["bias_std"] > 0:
            with torch.no_grad():
                mod.bias.copy_(9.0 + c["bias_std"] * torch.randn_like(mod.bias))
        x = torch.randn(c["B"], c["C"], c["H"], c["W"])
        out[f"x{i}"] = x.numpy()
        out[f"w{i}"] = mod.weight.detach().numpy()
        out[f"b{i}"] = mod.bias.detach().numpy()
        out[f"ref32_{i}"] = run_ref(mod, x, torch.float32)
        out[f"ref64_{i}"] = run_ref(mod, x, torch.float64).astype(np.float64)
        meta.append(c)
    out["meta"] = np.array(repr(meta))
    path = os.path.join(HERE, "converse2d_ref_cases.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(meta)} cases, {os.path.getsize(path) / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
