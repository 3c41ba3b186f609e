#!/usr/bin/env python3
"""Compile the reference's own C++ operator into oracle/_ref/ -- TEST INFRASTRUCTURE ONLY.

Source: `Converse2D/torch_converse2d/converse2d.cpp` of the reference checkout, compiled
where it lies with g++ against the installed torch headers (no copy of the source is
made, nothing of the reference's build system is run).  Output:
`oracle/_ref/converse2d_ref.so`, which registers `torch.ops.converse2d.forward` and
`clear_cache` exactly as the reference's extension does (`converse2d.cpp:218-227`).

The result is used as a checker in tests and as the timed CPU baseline; the product
library never loads it.  Skips quietly when the reference checkout is absent (the GPU
box only carries the prebuilt file).
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "converse2d_ref.so")


def default_reference_root():
    """The reference checkout: CONVERSE_REFERENCE_ROOT, else a directory `reference` beside this repository."""
    return os.environ.get("CONVERSE_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build_ref(reference_root=None, force=False):
    root = reference_root or default_reference_root()
    src = os.path.join(root, "Converse2D", "torch_converse2d", "converse2d.cpp")
    if not os.path.exists(src):
        return OUT if os.path.exists(OUT) else None
    if os.path.exists(OUT) and not force and os.path.getmtime(OUT) >= os.path.getmtime(src):
        return OUT
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-w", "-DTORCH_EXTENSION_NAME=converse2d_ref",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    for inc in ce.include_paths() + [sysconfig.get_paths()["include"]]:
        cmd += ["-isystem", inc]
    libdir = ce.library_paths()[0]
    cmd += [src, "-o", OUT, "-L" + libdir, "-Wl,-rpath," + libdir, "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    subprocess.run(cmd, check=True)
    return OUT


def load_ref():
    """Register the reference op in THIS process (do not combine with the product's own
    `torch.ops.converse2d` registration: the schema can only be defined once)."""
    import torch
    path = build_ref()
    if path is None:
        return False
    torch.ops.load_library(path)
    return hasattr(torch.ops.converse2d, "forward")


if __name__ == "__main__":
    print(build_ref(force="--force" in sys.argv))
