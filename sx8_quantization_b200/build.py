"""Build, in-tree: libsx8b200.so (the C-ABI CUDA library, nvcc for sm_100a) and
_sx8_torch.so (the thin torch binding over that C ABI, g++).

    python -m sx8_quantization_b200.build [--force] [-v]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libsx8b200.so")
SOURCES = ["sx8_api.cu", "sx8_codec.cu", "sx8_gemv.cu", "sx8_gemm.cu", "sx8_gemm_tc.cu", "sx8_glue.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-rdc=true"]


EXT = os.path.join(HERE, "_sx8_torch.so")
EXT_SRC = os.path.join(CSRC, "sx8_torch_binding.cpp")


def build_ext(force=False, verbose=False):
    """The torch binding: one host-only translation unit linked against libsx8b200.so (found
    at run time beside it, rpath $ORIGIN) and torch's own libraries."""
    inc = os.path.join(os.path.dirname(HERE), "include", "sx8_b200.h")
    if (not force and os.path.exists(EXT)
            and os.path.getmtime(EXT) >= max(os.path.getmtime(EXT_SRC), os.path.getmtime(inc), os.path.getmtime(LIB))):
        return EXT
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-w",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch.compiled_with_cxx11_abi()),
           "-DTORCH_EXTENSION_NAME=_sx8_torch", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    for d in ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include"),
                                   os.path.join(os.path.dirname(HERE), "include")]:
        cmd += ["-I", d]
    cmd += [EXT_SRC, "-o", EXT, "-L", tlib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch", "-ltorch_python",
            "-L", HERE, "-l:libsx8b200.so", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib,
            "-L", os.path.join(cuda_home, "lib64"), "-lcudart"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return EXT


def _newest_source():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if not f.endswith(".cpp")]
    files.append(os.path.join(os.path.dirname(HERE), "include", "sx8_b200.h"))
    return max(os.path.getmtime(f) for f in files)


def build(force=False, verbose=False):
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_source():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    extra = os.environ.get("SX8_NVCC_EXTRA", "").split()
    objs = []
    procs = []
    for s in SOURCES:
        o = os.path.join(CSRC, s.replace(".cu", ".o"))
        cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, s), "-o", o]
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(o)
    for s, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            print(out)
        if p.returncode:
            raise RuntimeError("nvcc failed on %s" % s)
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", "-o", LIB] + objs + \
          ["-lcudart"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_ext(force="--force" in sys.argv, verbose="-v" in sys.argv))
