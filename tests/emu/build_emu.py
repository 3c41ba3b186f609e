"""Build the host-emulation library (test infrastructure; g++ only, no GPU, no nvcc)."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
LIB = os.path.join(HERE, "libcvb_emu.so")


def build_emu():
    csrc = os.path.join(ROOT, "conversenet_b200", "csrc")
    srcs = [os.path.join(HERE, "emu.cpp")] + [os.path.join(csrc, f) for f in os.listdir(csrc)
                                               if f.endswith((".cuh", ".h"))]
    if os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(s) for s in srcs):
        return LIB
    if not os.path.exists(os.path.join(csrc, "fft_codelets.cuh")):
        from conversenet_b200.build import generate_sources
        generate_sources()
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-w", "-ffp-contract=off", "-x", "c++",
           "-I" + cuda_inc, "-o", LIB, os.path.join(HERE, "emu.cpp")]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build_emu())
