"""CPU-side checks: the C-ABI library loads and exports every symbol the public header
declares (no compute without a GPU), and the drop-in Python modules expose the
reference's public names with the reference's parameter lists."""
import ctypes
import inspect
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    txt = open(os.path.join(ROOT, "include", "sx8_b200.h")).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    return sorted(set(re.findall(r"\b(sx8_[a-z0-9_]+)\s*\(", txt)))


def test_library_exports_every_declared_symbol():
    from sx8_quantization_b200 import _lib
    assert os.path.exists(_lib.LIB_PATH), "libsx8b200.so not built"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = _header_functions()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), "missing export " + n
    assert set(_lib.SIGNATURES) == set(names), "ctypes table and header disagree"


def test_version_and_error_string_without_gpu():
    from sx8_quantization_b200 import _lib
    L = _lib.lib()
    assert L.sx8_version() >= 100
    assert L.sx8_last_error() == b"" or isinstance(L.sx8_last_error(), bytes)
    assert L.sx8_gemv_workspace_bytes(80, 8) == 80 * 8 * 64
    assert L.sx8_t16_bytes(2560, 80) == 160 * 80 * 480
    assert L.sx8_t16_bytes(10, 1) == 480


def test_host_validation_rejects_before_any_launch():
    """Argument checks run on the host: null pointers are refused without touching a device."""
    from sx8_quantization_b200 import _lib
    L = _lib.lib()
    rc = L.sx8_gemv(None, 1, 32, 32, None, None, None, 8, 1, None, None, 0, 0, None)
    assert rc == -1 and b"null pointer" in L.sx8_last_error()
    rc = L.sx8_embed(None, 4, None, None, None, 32, 8, 1, None, None)
    assert rc == -1
    rc = L.sx8_quantize_blocks(None, 1, 8, 32, 32, None, None, None, None, None, None, 0, None)
    assert rc == -1
    rc = L.sx8_pca_gram(None, 1, 8, 32, 32, None, None, None, None, None, None, None, 0, None)
    assert rc == -1 and b"sx8_pca_gram" in L.sx8_last_error()
    rc = L.sx8_pca_project(None, 1, 8, 32, 32, None, None, None, None, None, None, None, None)
    assert rc == -1 and b"sx8_pca_project" in L.sx8_last_error()
    rc = L.sx8_pca_pack(None, None, 8, 1, None, None)
    assert rc == -1 and b"sx8_pca_pack" in L.sx8_last_error()
    rc = L.sx8_gemm_multi(None, 32, 32, 32, 0, None, None, None, None, None, 0, 1, None, 0, None)
    assert rc == -1 and b"count" in L.sx8_last_error()
    rc = L.sx8_gemm_multi(None, 32, 32, 32, 2, None, None, None, None, None, 0, 1, None, 0, None)
    assert rc == -1 and b"null" in L.sx8_last_error()
    assert L.sx8_gemm_multi_workspace_bytes(32, 0, None, 1) == 0
    assert L.sx8_pca_gram_scratch_bytes(0, 32) == 0 and L.sx8_pca_gram_scratch_bytes(1000, 64) > 0


# (module, function) -> parameter names of the reference's public wrapper API
#   ref scripts/sx8_decode1_v3.py:57,69,91 ; scripts/sx8_gemm_compact.py:42 ;
#   scripts/sx8_fused_wmma.py:60,69,90,97 ; scripts/sx8_embed_v44.py:40-62 ;
#   scripts/kernel_sx8_v43.py:54,109
REFERENCE_API = {
    ("sx8_decode1_v3", "make_tensors_v44"): ["qt", "bases_info", "hdr_aligned"],
    ("sx8_decode1_v3", "best_split_k"): ["N", "n_cb"],
    ("sx8_decode1_v3", "decode1_v44"): ["X", "qt", "bases_info", "hdr_t", "lvl_t", "bas_t", "sca_t", "hdr_bytes",
                                        "split_k"],
    ("sx8_gemm_compact", "gemm_sx8_compact"): ["X", "qt", "bases_info", "hdr_t", "lvl_t", "bas_t", "sca_t",
                                               "hdr_bytes", "in_f", "n_cb"],
    ("sx8_fused_wmma", "gemm_sx8_wmma_cached"): ["X", "tensors", "n_cb"],
    ("sx8_fused_wmma", "make_tensors"): ["qt_kbmajor", "bases_info", "device"],
    ("sx8_fused_wmma", "gemm_sx8_wmma"): ["X", "qt_kbmajor", "bases_info", "n_cb"],
    ("sx8_fused_wmma", "decode1_sx8_cached"): ["X", "tensors", "n_cb"],
    ("kernel_sx8_v43", "decode_tensor_gpu_fast"): ["qt", "bases_info", "out"],
    ("kernel_sx8_v43", "decode_tensor_gpu"): ["qt", "bases_info"],
}


@pytest.mark.parametrize("key", list(REFERENCE_API))
def test_drop_in_signatures(key):
    import importlib
    mod = importlib.import_module("sx8_quantization_b200." + key[0])
    fn = getattr(mod, key[1])
    params = list(inspect.signature(fn).parameters)
    want = REFERENCE_API[key]
    assert params[:len(want)] == want, (key, params)
    for extra in params[len(want):]:   # additions must be optional
        assert inspect.signature(fn).parameters[extra].default is not inspect.Parameter.empty


def test_embedding_module_interface():
    from sx8_quantization_b200.sx8_embed_v44 import SX8EmbeddingV44
    params = list(inspect.signature(SX8EmbeddingV44.__init__).parameters)
    assert params == ["self", "qt", "bases_info", "hdr_bytes"]
    assert hasattr(SX8EmbeddingV44, "forward")


def test_launcher_registers_reference_module_names():
    import sys
    from sx8_quantization_b200 import launch
    mods = launch.register()
    for name in launch.DROP_IN:
        assert sys.modules[name].__name__ == "sx8_quantization_b200." + name
    assert len(mods) == len(launch.DROP_IN)


def test_reference_signatures_match_checkout_if_present():
    """When a reference checkout is available, compare against its source directly."""
    import ast
    from oracle import build as ob
    ref = ob.ref_root()   # $SX8_REF, else the path BASELINE.json records
    if not ref or not os.path.isdir(os.path.join(ref, "scripts")):
        pytest.skip("no reference checkout")
    for (mod, fn), want in REFERENCE_API.items():
        tree = ast.parse(open(os.path.join(ref, "scripts", mod + ".py")).read())
        node = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == fn)
        assert [a.arg for a in node.args.args] == want, (mod, fn)


def test_torch_binding_is_built_and_forwards_to_the_c_abi():
    """The thin torch extension over the C ABI loads without a GPU and answers the size queries
    with the library's own numbers."""
    from sx8_quantization_b200 import _lib
    E = _lib.ext()
    assert E is not None, "_sx8_torch.so not built (python -m sx8_quantization_b200.build)"
    L = _lib.lib()
    assert E.gemv_workspace_bytes(80, 8) == L.sx8_gemv_workspace_bytes(80, 8)
    assert E.gemm_workspace_bytes(128, 1024, 80) == L.sx8_gemm_workspace_bytes(128, 1024, 80)
    assert isinstance(E.last_error(), str)
    for fn in ("gemv", "gemm", "embed"):
        assert callable(getattr(E, fn))
