"""Fixtures for the caller-side data path: PSNR / SSIM / conversions / blur of the UNMODIFIED
reference helpers (`utils/utils_image.py`) on seeded random images.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_image_golden.py

Needs the reference checkout (its place: $CONVERSE_REFERENCE_ROOT) with numpy, scipy and
OpenCV; writes tests/golden/image_ref_cases.npz (a few KB)."""
import os
import sys
import types

import numpy as np

REF = os.environ.get("CONVERSE_REFERENCE_ROOT")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set CONVERSE_REFERENCE_ROOT to the reference checkout")
HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    sys.dont_write_bytecode = True
    for name in ("matplotlib", "matplotlib.pyplot", "mpl_toolkits", "mpl_toolkits.mplot3d"):
        try:
            __import__(name)
        except Exception:   # plotting is not used by the helpers recorded here
            mod = types.ModuleType(name)
            mod.Axes3D = object
            sys.modules[name] = mod
    sys.path.insert(0, REF)
    from utils import utils_image as util
    from scipy import ndimage
    rng = np.random.default_rng(2024)
    out = {}
    shapes = [(23, 27), (21, 25, 3), (28, 22, 1)]
    for i, shp in enumerate(shapes):
        a = rng.integers(0, 256, size=shp, dtype=np.uint8)
        noise = rng.normal(0, 12.0, size=shp)
        b = np.uint8(np.clip(a.astype(np.float64) + noise, 0, 255).round())
        out["a%d" % i], out["b%d" % i] = a, b
        for border in (0, 4):
            out["psnr%d_%d" % (i, border)] = np.float64(util.calculate_psnr(a, b, border=border))
            out["ssim%d_%d" % (i, border)] = np.float64(util.calculate_ssim(a, b, border=border))
        t = util.uint2tensor4(a)
        out["t4_%d" % i] = t.numpy()
        f = rng.random(size=t.shape).astype(np.float32) * 1.2 - 0.1
        import torch
        out["f%d" % i] = f
        out["u8_%d" % i] = util.tensor2uint(torch.from_numpy(f))
    # wrap-around blur of the USRNet script (main_test_converse_usrnet.py:141)
    img = rng.random(size=(18, 16, 3))
    k = rng.random(size=(7, 7)); k /= k.sum()
    out["blur_in"], out["blur_k"] = img, k
    out["blur_out"] = ndimage.convolve(img, np.expand_dims(k, axis=2), mode="wrap")
    k2 = rng.random(size=(4, 5)); k2 /= k2.sum()
    out["blur_k2"] = k2
    out["blur_out2"] = ndimage.convolve(img, np.expand_dims(k2, axis=2), mode="wrap")
    np.savez_compressed(os.path.join(HERE, "image_ref_cases.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
