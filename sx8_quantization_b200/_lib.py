"""Bindings of libsx8b200.so (the C ABI declared in include/sx8_b200.h): ctypes for every
entry point, and -- for the calls a decode loop makes hundreds of times per token -- the thin
torch extension _sx8_torch.so (csrc/sx8_torch_binding.cpp), which resolves device, stream and
data pointers in C++.

There is no fallback: if the shared library is missing the import of any kernel
wrapper raises, and every non-zero status from the library becomes an exception."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# SX8_LIB_PATH selects another build of the same library (e.g. one compiled with extra flags)
LIB_PATH = os.environ.get("SX8_LIB_PATH") or os.path.join(_HERE, "libsx8b200.so")

_vp, _i, _l, _sz, _u = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_size_t, ctypes.c_uint

# name -> (restype, argtypes); mirrors include/sx8_b200.h one to one
SIGNATURES = {
    "sx8_version": (_i, []),
    "sx8_last_error": (ctypes.c_char_p, []),
    "sx8_gemv_workspace_bytes": (_sz, [_i, _i]),
    "sx8_gemv": (_i, [_vp, _i, _i, _l, _vp, _vp, _vp, _i, _i, _vp, _vp, _sz, _u, _vp]),
    "sx8_gemv_multi": (_i, [_vp, _i, _i, _l, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp, _sz, _u, _vp]),
    "sx8_gemv_allreduce": (_i, [_vp, _i, _i, _l, _vp, _vp, _vp, _i, _i, _vp, _vp, _sz, _u, _vp, _vp]),
    "sx8_gemm_workspace_bytes": (_sz, [_i, _i, _i]),
    "sx8_gemm": (_i, [_vp, _i, _i, _l, _vp, _vp, _vp, _i, _i, _vp, _i, _vp, _sz, _vp]),
    "sx8_gemm_multi_workspace_bytes": (_sz, [_i, _i, _vp, _i]),
    "sx8_gemm_multi": (_i, [_vp, _i, _i, _l, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _sz, _vp]),
    "sx8_gemm_static_max_ncb": (_sz, []),
    "sx8_gemm_static": (_i, [_vp, _i, _i, _l, _vp, _vp, _vp, _i, _i, _vp, _i, _vp]),
    "sx8_embed": (_i, [_vp, _l, _vp, _vp, _vp, _i, _i, _i, _vp, _vp]),
    "sx8_dequant_planes": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _l, _l, _i, _i, _vp, _vp]),
    "sx8_dequant_t16": (_i, [_vp, _vp, _vp, _l, _l, _i, _i, _vp, _vp]),
    "sx8_quantize_blocks": (_i, [_vp, _i, _l, _l, _l, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "sx8_pca_gram_scratch_bytes": (_sz, [_l, _l]),
    "sx8_pca_gram": (_i, [_vp, _i, _l, _l, _l, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "sx8_pca_project": (_i, [_vp, _i, _l, _l, _l, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "sx8_pca_pack": (_i, [_vp, _vp, _l, _i, _vp, _vp]),
    "sx8_t16_bytes": (_sz, [_l, _i]),
    "sx8_repack_t16": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _l, _i, _vp, _vp]),
    "sx8_repack_v44": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _l, _i, _i, _vp, _vp, _vp]),
    "sx8_repack_t16_blocks": (_i, [_vp, _l, _i, _vp, _vp]),
    "sx8_blocks_from_planes": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _l, _vp, _vp]),
    "sx8_planes_from_blocks": (_i, [_vp, _l, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "sx8_glue_add_rmsnorm": (_i, [_vp, _vp, _vp, _i, _i, ctypes.c_float, _vp, _vp]),
    "sx8_glue_allreduce_add_rmsnorm": (_i, [_vp, _i, _i, _vp, _vp, ctypes.c_float, _vp, _vp]),
    "sx8_glue_rope_cache": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "sx8_glue_attn_scratch_bytes": (_sz, [_i, _i, _i, _i]),
    "sx8_glue_attn_decode": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, ctypes.c_float, _vp, _vp, _sz, _vp]),
    "sx8_glue_silu_mul": (_i, [_vp, _vp, _l, _vp, _vp]),
    "sx8_device_error_flag": (_i, [ctypes.POINTER(ctypes.c_uint)]),
}

# include/sx8_b200_test.h: hooks for the test suite, not part of the library's contract
TEST_SIGNATURES = {
    "sx8_gemv_tune": (None, [_i, _i, _i]),
}

SX8_F_PDL = 1


class Peers(ctypes.Structure):
    """sx8_peers_t of include/sx8_b200.h."""
    _fields_ = [("data", ctypes.c_void_p * 8), ("flags", ctypes.c_void_p * 8), ("slot_elems", ctypes.c_long),
                ("rank", ctypes.c_int), ("world", ctypes.c_int), ("parity", ctypes.c_int)]


class SX8Error(RuntimeError):
    pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise SX8Error("libsx8b200.so is not built (run `python -m sx8_quantization_b200.build`); "
                           "there is no CPU or PyTorch fallback for the S-X8 kernels")
        l = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in list(SIGNATURES.items()) + list(TEST_SIGNATURES.items()):
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


_ext = None
_ext_tried = False


def ext():
    """The torch binding module, or None when it is not built or when SX8_LIB_PATH points the
    ctypes binding at another build of the library (the extension is linked to the in-tree one)."""
    global _ext, _ext_tried
    if not _ext_tried:
        _ext_tried = True
        path = os.path.join(_HERE, "_sx8_torch.so")
        if os.path.exists(path) and not os.environ.get("SX8_LIB_PATH") and os.environ.get("SX8_NO_TORCH_EXT") != "1":
            import importlib.util
            import torch  # noqa: F401  (libtorch must be loaded first)
            lib()
            spec = importlib.util.spec_from_file_location("_sx8_torch", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            _ext = mod
    return _ext


def check(rc, what):
    if rc != 0:
        msg = lib().sx8_last_error().decode(errors="replace")
        raise SX8Error("%s failed (%d): %s" % (what, rc, msg))


def device_error_flag():
    v = ctypes.c_uint(0)
    check(lib().sx8_device_error_flag(ctypes.byref(v)), "sx8_device_error_flag")
    return v.value
