"""Test-time drivers around a restoration network: plain call, pad-to-multiple, quadrant
splitting with overlap, and the x8 geometric self-ensemble.

Same entry points and argument meaning as the reference's `utils/utils_model.py:51-229`
(`test_mode`, `test`, `test_pad`, `test_split`, `test_x8`, `test_split_x8`) and
`utils/utils_image.py:405-423` (`augment_img_tensor4`), so that its `main_test_*.py`
scripts can switch backends by changing one import.  The x8 modes transpose the image,
which is what exercises H != W planes in the Converse2D kernels.
"""
import math

import torch
import torch.nn.functional as F

# The eight symmetries of the square as (transpose first, flip rows, flip columns), in the
# reference's mode order (0 identity, 1 rot90+flipud, 2 flipud, 3 rot270, 4 rot180+flipud,
# 5 rot90, 6 rot180, 7 rot270+flipud).
_SYMMETRIES = (
    (False, False, False),
    (True, False, False),
    (False, True, False),
    (True, False, True),
    (False, False, True),
    (True, True, False),
    (False, True, True),
    (True, True, True),
)


def augment_img_tensor4(img, mode=0):
    """Apply symmetry `mode` (0..7) to the last two axes of a (B,C,H,W) tensor."""
    transpose, flip_rows, flip_cols = _SYMMETRIES[mode]
    out = img.transpose(2, 3) if transpose else img
    dims = [d for d, on in ((2, flip_rows), (3, flip_cols)) if on]
    return out.flip(dims) if dims else out


def _inverse_mode(mode):
    """Mode whose symmetry undoes `mode`: every mode is an involution except the two
    quarter turns, which undo each other."""
    return {3: 5, 5: 3}.get(mode, mode)


def _pad_to_multiple(L, modulo):
    h, w = L.shape[-2:]
    pad_b = int(math.ceil(h / modulo) * modulo - h)
    pad_r = int(math.ceil(w / modulo) * modulo - w)
    if pad_b == 0 and pad_r == 0:
        return L
    return F.pad(L, (0, pad_r, 0, pad_b), mode="replicate")


def test(model, L):
    """Mode 0: the network as it is."""
    return model(L)


def test_pad(model, L, modulo=16, sf=1):
    """Mode 1: replicate-pad bottom/right to a multiple of `modulo`, run, crop to sf*(h, w)."""
    h, w = L.shape[-2:]
    E = model(_pad_to_multiple(L, modulo))
    return E[..., : h * sf, : w * sf]


def test_split_fn(model, L, refield=32, min_size=256, sf=1, modulo=1):
    """Run `model` on four overlapping quadrants (recursively while a quadrant has more than
    `min_size`^2 pixels) and keep from each the part that lies inside its own quarter."""
    h, w = L.shape[-2:]
    if h * w <= min_size ** 2:
        E = model(_pad_to_multiple(L, modulo))
        return E[..., : h * sf, : w * sf]
    qh = (h // 2 // refield + 1) * refield   # quadrant extents: half the image plus overlap,
    qw = (w // 2 // refield + 1) * refield   # rounded up to the receptive-field step
    rows = (slice(0, qh), slice(h - qh, h))
    cols = (slice(0, qw), slice(w - qw, w))
    parts = [L[..., r, c] for r in rows for c in cols]
    if h * w <= 4 * (min_size ** 2):
        outs = [model(p) for p in parts]
    else:
        outs = [test_split_fn(model, p, refield=refield, min_size=min_size, sf=sf, modulo=modulo) for p in parts]
    b, ch = outs[0].shape[:2]
    E = torch.zeros(b, ch, sf * h, sf * w, dtype=L.dtype, device=L.device)
    top, left = (h // 2) * sf, (w // 2) * sf
    bot, right = (h - h // 2) * sf, (w - w // 2) * sf   # rows / columns taken from the far quadrants
    E[..., :top, :left] = outs[0][..., :top, :left]
    E[..., :top, left:] = outs[1][..., :top, -right:]
    E[..., top:, :left] = outs[2][..., -bot:, :left]
    E[..., top:, left:] = outs[3][..., -bot:, -right:]
    return E


def test_split(model, L, refield=32, min_size=256, sf=1, modulo=1):
    """Mode 2."""
    return test_split_fn(model, L, refield=refield, min_size=min_size, sf=sf, modulo=modulo)


def _ensemble(run, L):
    total = None
    for mode in range(8):
        E = augment_img_tensor4(run(augment_img_tensor4(L, mode)), _inverse_mode(mode))
        total = E if total is None else total + E
    return total / 8.0


def test_x8(model, L, modulo=1, sf=1):
    """Mode 3: mean over the eight symmetries of `test_pad`."""
    return _ensemble(lambda t: test_pad(model, t, modulo=modulo, sf=sf), L)


def test_split_x8(model, L, refield=32, min_size=256, sf=1, modulo=1):
    """Mode 4: mean over the eight symmetries of `test_split_fn`."""
    return _ensemble(lambda t: test_split_fn(model, t, refield=refield, min_size=min_size, sf=sf, modulo=modulo), L)


def test_mode(model, L, mode=0, refield=32, min_size=256, sf=1, modulo=1):
    """Dispatch on `mode` (0 plain, 1 pad, 2 split, 3 x8, 4 split + x8)."""
    if mode == 0:
        return test(model, L)
    if mode == 1:
        return test_pad(model, L, modulo, sf)
    if mode == 2:
        return test_split(model, L, refield, min_size, sf, modulo)
    if mode == 3:
        return test_x8(model, L, modulo, sf)
    if mode == 4:
        return test_split_x8(model, L, refield, min_size, sf, modulo)
    raise ValueError("mode must be 0..4, got %r" % (mode,))
