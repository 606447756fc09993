"""Build recipe for the checker: the C restatement (oracle/sx8_oracle.c ->
oracle/libsx8oracle.so) and, when a checkout of the reference is present, the
reference's own CUDA kernels compiled from where they lie into oracle/_ref/.

TEST INFRASTRUCTURE ONLY -- nothing in the product package imports this.

    python oracle/build.py            # C oracle only
    python oracle/build.py --ref      # also oracle/_ref (needs a reference checkout, see ref_root)

oracle/_ref/ receives compiled artefacts only, never source text:
  <name>/<name>.so   the reference's four CUDA files built as torch extensions;
  pyc/<module>.bin   byte-compiled copies of the reference's Python callers and of its
                     numba decoder (sourceless modules: importable, not readable), so that a
                     GPU machine without the checkout can still run the reference's own
                     SX8LinearV44 / decode_tensor_gpu_fast against this library;
  pyc/ref_quantizer_funcs.bin   the four pure functions of the reference's quantizer script
                     (taken out of its syntax tree, because the script itself opens a model
                     at import).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libsx8oracle.so")
SRC = os.path.join(HERE, "sx8_oracle.c")
REF_DIR = os.path.join(HERE, "_ref")


def build_oracle(force=False):
    if (not force and os.path.exists(LIB)
            and os.path.getmtime(LIB) >= os.path.getmtime(SRC)):
        return LIB
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-shared",
           "-fPIC", "-o", LIB, SRC, "-lm"]
    subprocess.check_call(cmd)
    return LIB


def ref_root():
    """Path of the reference checkout: $SX8_REF, else the `reference_path` that
    BASELINE.json at the repository root records; None when neither exists."""
    root = os.environ.get("SX8_REF")
    if not root:
        try:
            import json
            root = json.load(open(os.path.join(os.path.dirname(HERE), "BASELINE.json"))).get("reference_path")
        except Exception:
            root = None
    return root if root and os.path.isdir(os.path.join(root, "cuda")) else None


# name -> (cu file, C++ prototypes the reference's own wrapper declares, functions)
_REF_EXT = {
    "ref_sx8_decode1_v3": ("sx8_decode1_v3.cu", """
torch::Tensor compute_z44(torch::Tensor X, torch::Tensor basis, torch::Tensor scales,
                          int64_t n_cb, torch::Tensor out);
torch::Tensor decode1_v44(torch::Tensor X, torch::Tensor hdr, torch::Tensor levels,
                          torch::Tensor Z, int64_t n_cb, int64_t hdr_bytes,
                          int64_t split_k, torch::Tensor out);
torch::Tensor decode1_v44_combined(torch::Tensor X, torch::Tensor hdr, torch::Tensor levels,
                                   torch::Tensor basis, torch::Tensor scales,
                                   int64_t n_cb, int64_t hdr_bytes,
                                   torch::Tensor Z, torch::Tensor out);
""", ["compute_z44", "decode1_v44", "decode1_v44_combined"]),
    "ref_sx8_gemm_compact": ("sx8_gemm_compact.cu", """
torch::Tensor compute_z44_batch(torch::Tensor X, torch::Tensor basis, torch::Tensor scales, int64_t n_cb);
torch::Tensor gemm_compact(torch::Tensor X, torch::Tensor hdr, torch::Tensor levels,
                           torch::Tensor Z, int64_t n_cb, int64_t hdr_bytes);
""", ["compute_z44_batch", "gemm_compact"]),
    "ref_sx8_fused_wmma": ("sx8_fused_wmma.cu",
                           "torch::Tensor fused_forward(torch::Tensor, torch::Tensor, torch::Tensor, "
                           "torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, "
                           "torch::Tensor, int64_t);", ["fused_forward"]),
    "ref_sx8_embed_v44": ("sx8_embed_v44.cu", """
torch::Tensor sx8_embed_v44(torch::Tensor ids, torch::Tensor hdr, torch::Tensor levels,
                            torch::Tensor basis, torch::Tensor scales,
                            int64_t K, int64_t N, int64_t n_cb, torch::Tensor out);
""", ["sx8_embed_v44"]),
}


def build_ref(verbose=False):
    """Compile the reference's four hot-path .cu files, unmodified and read from
    the reference checkout, the way its own wrappers do (load_inline, -O3), but
    for sm_100 and with the build directory set to oracle/_ref/<name>/.  The
    resulting .so files are what `load_ref` imports on a GPU box."""
    root = ref_root()
    if root is None:
        raise RuntimeError("no reference checkout (set SX8_REF)")
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    from torch.utils.cpp_extension import load_inline
    built = []
    for name, (cu, cpp, funcs) in _REF_EXT.items():
        bdir = os.path.join(REF_DIR, name)
        os.makedirs(bdir, exist_ok=True)
        if os.path.exists(os.path.join(bdir, name + ".so")):
            built.append(name)
            continue
        src = open(os.path.join(root, "cuda", cu)).read()
        # is_python_module=False: compile and link only; importing would need a GPU
        load_inline(name=name, cpp_sources=cpp, cuda_sources=src, functions=funcs,
                    extra_cuda_cflags=["-O3"], build_directory=bdir, verbose=verbose,
                    is_python_module=False)
        # keep the shared object only: generated sources embed the reference text
        for f in os.listdir(bdir):
            if not f.endswith(".so"):
                os.remove(os.path.join(bdir, f))
        built.append(name)
    return built


# Python modules of the reference that the caller-level parity tests import on the GPU box.
_REF_PY = ["kernel_sx8_v43", "kernel_sx8_v4", "kernel_sx8_fused", "eval_common", "integrate_fused",
           "integrate_fused_v44", "prepare_v44"]
_REF_QUANT = "quantize_qwen35_4b_sx8_v43_gpu"
_REF_QUANT_FUNCS = ("v6_encode_6bit_gpu", "chunked_v6_encode", "pca_correct_gpu", "pack_levels_6bit")
PYC_DIR = os.path.join(REF_DIR, "pyc")


def build_ref_py():
    """Byte-compile the reference's caller modules from where they lie into oracle/_ref/pyc/
    (sourceless byte code, stored as .bin: snapshot tools tend to drop *.pyc).  The quantizer script runs a model conversion at import, so only
    its four pure functions are compiled, from its syntax tree, into ref_quantizer_funcs.bin;
    the importer supplies the module constants (DEV, B, L63, N_BASES, MAX_BLOCKS_PER_CHUNK)."""
    import ast
    import importlib.util
    import marshal
    import py_compile
    root = ref_root()
    if root is None:
        raise RuntimeError("no reference checkout (set SX8_REF)")
    os.makedirs(PYC_DIR, exist_ok=True)
    done = []
    for mod in _REF_PY:
        src = os.path.join(root, "scripts", mod + ".py")
        # dfile: the name recorded inside the code object (tracebacks), not a path of this machine
        py_compile.compile(src, cfile=os.path.join(PYC_DIR, mod + ".bin"), dfile="ref/scripts/" + mod + ".py",
                           doraise=True)
        done.append(mod)
    tree = ast.parse(open(os.path.join(root, "scripts", _REF_QUANT + ".py")).read())
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in _REF_QUANT_FUNCS]
    if len(body) != len(_REF_QUANT_FUNCS):
        raise RuntimeError("the reference quantizer no longer defines " + ", ".join(_REF_QUANT_FUNCS))
    code = compile(ast.Module(body=body, type_ignores=[]), "ref/scripts/" + _REF_QUANT + ".py", "exec")
    with open(os.path.join(PYC_DIR, "ref_quantizer_funcs.bin"), "wb") as f:
        f.write(importlib.util.MAGIC_NUMBER + b"\0" * 12)   # unchecked, no source: flags 0, mtime 0, size 0
        f.write(marshal.dumps(code))
    done.append("ref_quantizer_funcs")
    return done


class RefFinder:
    """sys.meta_path entry that resolves the reference's bare module names (`import
    integrate_fused`, `from eval_common import ...`) to the byte code staged in
    oracle/_ref/pyc/.  Names already in sys.modules (the drop-in modules registered by
    sx8_quantization_b200.launch) never reach a finder, so they keep precedence."""

    def find_spec(self, name, path=None, target=None):
        import importlib.machinery
        import importlib.util
        if name not in _REF_PY:
            return None
        f = os.path.join(PYC_DIR, name + ".bin")
        if not os.path.exists(f):
            return None
        return importlib.util.spec_from_loader(name, importlib.machinery.SourcelessFileLoader(name, f))


def install_ref_finder():
    """Make the staged reference modules importable by bare name; False when none are staged."""
    if not os.path.exists(os.path.join(PYC_DIR, "integrate_fused_v44.bin")):
        return False
    if not any(isinstance(f, RefFinder) for f in sys.meta_path):
        sys.meta_path.append(RefFinder())
    return True


def load_ref_py(module, alias=None):
    """Import oracle/_ref/pyc/<module>.bin under the name `alias` (default: module) without
    touching sys.modules[module]; None when it was not staged."""
    import importlib.machinery
    import importlib.util
    path = os.path.join(PYC_DIR, module + ".bin")
    if not os.path.exists(path):
        return None
    name = alias or module
    loader = importlib.machinery.SourcelessFileLoader(name, path)
    spec = importlib.util.spec_from_loader(name, loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


def load_ref_quantizer(device):
    """The reference quantizer's four functions bound to `device` (a torch.device), with the
    module constants the script defines beside them; None when not staged."""
    import marshal
    path = os.path.join(PYC_DIR, "ref_quantizer_funcs.bin")
    if not os.path.exists(path):
        return None
    import numpy as np
    import torch
    ns = dict(torch=torch, np=np, DEV=device, B=32, L63=63, N_BASES=4, MAX_BLOCKS_PER_CHUNK=3_000_000)
    with open(path, "rb") as f:
        f.read(16)
        exec(marshal.loads(f.read()), ns)
    return ns


def load_ref(name):
    """Import a prebuilt reference extension from oracle/_ref (GPU box). Returns
    None when it was not built."""
    so = os.path.join(REF_DIR, name, name + ".so")
    if not os.path.exists(so):
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch symbols must be loaded first)
    spec = importlib.util.spec_from_file_location(name, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    if "--ref" in sys.argv:
        print(build_ref(verbose="-v" in sys.argv))
        print(build_ref_py())
