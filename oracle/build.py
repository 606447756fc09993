"""Build recipe for the checker: the C restatement (oracle/sx8_oracle.c ->
oracle/libsx8oracle.so) and, when a checkout of the reference is present, the
reference's own CUDA kernels compiled from where they lie into oracle/_ref/.

TEST INFRASTRUCTURE ONLY -- nothing in the product package imports this.

    python oracle/build.py            # C oracle only
    python oracle/build.py --ref      # also oracle/_ref (needs a reference checkout, see ref_root)
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
    root = os.environ.get("SX8_REF", "/root/reference")
    return root if os.path.isdir(os.path.join(root, "cuda")) else None


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
