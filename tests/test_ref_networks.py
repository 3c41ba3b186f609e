"""The network restatement in oracle/ref_networks.py (the checker and CPU baseline of the network
workloads) against the unmodified reference.

Where the reference checkout is present (environment variable CONVERSE_REFERENCE_ROOT, else a
directory `reference` beside this repository) every
restated network must give the reference network's output on CPU with the same state dict (fp64:
1e-10; fp32: within the reference's own rounding noise).  Everywhere, the restatement must load the reference's trained checkpoints strictly (copies
under tests/golden/model_zoo) and so must this package's mirrors; and it must reproduce the stored
small-size outputs of the reference (tests/golden/model_ref_cases.npz)."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import converse2d_oracle as orc
from oracle import ref_networks as rn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ZOO = os.path.join(ROOT, "tests", "golden", "model_zoo")
CKPT = {"dncnn": "converse_dncnn.pth", "srresnet": "converse_srresnet.pth", "usrnet": "converse_usrnet.pth",
        "conversenet": "conversenet.pth"}


def _mirror(name):
    from conversenet_b200 import models
    return {"dncnn": models.ConverseDnCNN, "srresnet": models.ConverseMSRResNet, "usrnet": models.ConverseUSRNet,
            "conversenet": models.ConverseNet}[name]()


@pytest.mark.parametrize("name", sorted(CKPT))
def test_trained_checkpoints_load_strictly(name):
    sd = torch.load(os.path.join(ZOO, CKPT[name]), map_location="cpu")
    rn.NETWORKS[name]().load_state_dict(sd, strict=True)
    _mirror(name).load_state_dict(sd, strict=True)


def _small_inputs(name):
    g = torch.Generator().manual_seed(3)
    if name == "dncnn":
        return (torch.rand(1, 1, 20, 24, generator=g),)
    if name == "usrnet":
        k = torch.rand(1, 1, 7, 7, generator=g)
        return (torch.rand(1, 3, 12, 16, generator=g), k / k.sum(), 2)
    return (torch.rand(1, 3, 12, 16, generator=g),)


@pytest.mark.parametrize("name", sorted(CKPT))
def test_restatement_matches_imported_reference(name):
    from oracle.build_ref import default_reference_root
    ref_root = default_reference_root()
    if not os.path.isdir(os.path.join(ref_root, "models")):
        pytest.skip("reference checkout not present")
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_root)
    try:
        from models.converse_dncnn import ConverseDnCNN
        from models.converse_srresnet import ConverseMSRResNet
        from models.converse_usrnet import ConverseUSRNet, ConverseNet
    finally:
        sys.path.remove(ref_root)
    ctor = {"dncnn": ConverseDnCNN, "srresnet": ConverseMSRResNet, "usrnet": ConverseUSRNet,
            "conversenet": ConverseNet}[name]
    sd = torch.load(os.path.join(ZOO, CKPT[name]), map_location="cpu")
    ref = ctor().eval()
    ref.load_state_dict(sd, strict=True)
    mine = rn.NETWORKS[name]().eval()
    mine.load_state_dict(sd, strict=True)
    rn.use_reference_op(False)
    args = _small_inputs(name)
    with torch.no_grad():
        a, b = ref(*args), mine(*args)
    # fp32: the reference's own rounding noise (its division by lambda amplifies summation-order
    # differences to ~3e-5 per layer); the fp64 run below is the pin
    assert orc.rel_l2(b.numpy(), a.numpy()) <= 3e-4
    if name != "usrnet":  # the reference's KernelNet casts to fp32 (`models/converse_usrnet.py:134`)
        with torch.no_grad():
            a64 = ref.double()(*[t.double() for t in args])
            b64 = mine.double()(*[t.double() for t in args])
        assert orc.rel_l2(b64.numpy(), a64.numpy()) <= 1e-10


def test_restatement_matches_stored_reference_outputs():
    fx = np.load(os.path.join(ROOT, "tests", "golden", "model_ref_cases.npz"))
    from conversenet_b200 import models
    rn.use_reference_op(False)
    # parameters as the fixture's generator made them: the mirror built under the same seed
    torch.manual_seed(101)
    sd = models.ConverseDnCNN().state_dict()
    net = rn.RefDnCNN().double().eval()
    net.load_state_dict({k: v.double() for k, v in sd.items()}, strict=True)
    with torch.no_grad():
        out = net(torch.from_numpy(fx["dncnn_x"]).double()).numpy()
    assert orc.rel_l2(out, fx["dncnn_ref64"]) <= 1e-9
    torch.manual_seed(102)
    sd = models.ConverseMSRResNet().state_dict()
    net = rn.RefSRResNet().double().eval()
    net.load_state_dict({k: v.double() for k, v in sd.items()}, strict=True)
    with torch.no_grad():
        out = net(torch.from_numpy(fx["srres_x"]).double()).numpy()
    assert orc.rel_l2(out, fx["srres_ref64"]) <= 1e-9
