"""ctypes binding of libconverse_b200.so (the C ABI declared in include/converse_b200.h).

The library is the only compute path: if it is missing the import of the
package succeeds (so that CPU-only tooling can build it) but every operator
call raises.  There is no fallback.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("CVB_LIBRARY") or os.path.join(_HERE, "libconverse_b200.so")

PAD_MODES = {"circular": 0, "replicate": 1, "reflect": 2, "constant": 3}
CVB_F32, CVB_BF16 = 0, 1
OPT_RUNTIME_PLAN, OPT_MULTIPASS, OPT_PERSISTENT, OPT_BLOCK_KERNELS = 0, 1, 2, 3

# name -> (restype, argtypes); one line per declaration in include/converse_b200.h
_c = ctypes
SIGNATURES = {
    "cvb_version": (_c.c_int, []),
    "cvb_strerror": (_c.c_char_p, [_c.c_int]),
    "cvb_last_cuda_error": (_c.c_int, []),
    "cvb_set_option": (_c.c_int, [_c.c_int, _c.c_int]),
    "cvb_get_option": (_c.c_int, [_c.c_int]),
    "cvb_last_device_status": (_c.c_int, [_c.c_int]),
    "cvb_transfer_bytes": (_c.c_size_t, [_c.c_int, _c.c_int, _c.c_int]),
    "cvb_build_transfer": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                      _c.c_int, _c.c_float, _c.c_void_p, _c.c_void_p]),
    "cvb_build_x0_table": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                      _c.c_int, _c.c_float, _c.c_void_p, _c.c_void_p]),
    "cvb_converse2d_workspace_bytes": (_c.c_size_t, [_c.c_int] * 7),
    "cvb_converse2d_fwd": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p] + [_c.c_int] * 10 +
                           [_c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "cvb_converse2d_fwd_static_scratch": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p] +
                                          [_c.c_int] * 10 + [_c.c_void_p]),
    "cvb_ln_pw_gelu_fwd": (_c.c_int, [_c.c_void_p] * 4 + [_c.c_float] + [_c.c_void_p] * 2 + [_c.c_int] * 4 + [_c.c_void_p]),
    "cvb_pw_res_mlp_fwd": (_c.c_int, [_c.c_void_p] * 8 + [_c.c_float] + [_c.c_void_p] * 5 + [_c.c_int] * 4 + [_c.c_void_p]),
    "cvb_pw_res_fwd": (_c.c_int, [_c.c_void_p] * 6 + [_c.c_int] * 4 + [_c.c_void_p]),
    "cvb_plan_radices": (_c.c_int, [_c.c_int, _c.POINTER(_c.c_int), _c.c_int]),
    "cvb_fits_shared": (_c.c_int, [_c.c_int, _c.c_int]),
    "cvb_cross_spectrum": (_c.c_int, [_c.c_void_p] * 4 + [_c.c_int] * 7 + [_c.c_void_p]),
    "cvb_cross_spectrum_supported": (_c.c_int, [_c.c_int, _c.c_int]),
    "cvb_tap_gradient": (_c.c_int, [_c.c_void_p] * 3 + [_c.c_int] * 7 + [_c.c_void_p]),
}

_lib = None


class ConverseLibraryError(RuntimeError):
    pass


def load():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ConverseLibraryError(
            "libconverse_b200.so is not built (run `python -m conversenet_b200.build`); "
            "this package has no other compute path")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the ABI and the header drift apart
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status, what):
    if status != 0:
        lib = load()
        msg = lib.cvb_strerror(status).decode()
        extra = ""
        if status == -5:
            extra = " (cudaError %d)" % lib.cvb_last_cuda_error()
        raise RuntimeError("%s failed: %s%s" % (what, msg, extra))


class option:
    """`with option(OPT_MULTIPASS, 1): ...` -- set a routing option of the library for a block of code."""

    def __init__(self, which, value):
        self.which, self.value = which, value

    def __enter__(self):
        lib = load()
        self.old = lib.cvb_get_option(self.which)
        check(lib.cvb_set_option(self.which, self.value), "cvb_set_option")
        return self

    def __exit__(self, *exc):
        load().cvb_set_option(self.which, self.old)
        return False
