"""Builds libblr_b200.so in-tree with nvcc for sm_100a (no JIT cache, no torch headers needed), and the thin PyTorch
C++ extension _blr_torch.so over its C ABI (g++ against the torch headers, also in-tree)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libblr_b200.so")
SOURCES = ["tmap.cu", "stream_kernel.cu", "blast_cluster.cu", "blast_split.cu", "umma_gemm.cu", "pipeline.cu", "ref32.cu", "decoder_kernels.cu", "c_api.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the library cannot be built")
    return cand


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "blr_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every .cu file to an object (in parallel) and links the shared library."""
    if not force and not needs_build():
        return LIB
    nvcc = _nvcc()
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    log = []
    for src, obj, p in procs:
        out, _ = p.communicate()
        log.append(f"== {src}\n{out}")
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        objs.append(obj)
    # the soname lets the torch extension's DT_NEEDED entry resolve to the copy the Python layer has already loaded
    link = [nvcc, "-shared", "-o", LIB, *objs, "-lcudart", "-Xlinker", "-soname=libblr_b200.so"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    with open(os.path.join(objdir, "build.log"), "w") as f:
        f.write("\n".join(log))
    if verbose:
        print("\n".join(log))
    return LIB


EXT = os.path.join(HERE, "_blr_torch.so")


def ext_needs_build() -> bool:
    if not os.path.exists(EXT):
        return True
    t = os.path.getmtime(EXT)
    deps = [os.path.join(CSRC, "torch_ext.cpp"), os.path.join(HERE, "..", "include", "blr_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build_torch_ext(force: bool = False, verbose: bool = False) -> str:
    """Compiles csrc/torch_ext.cpp (TORCH_LIBRARY ops over the C ABI) against the installed torch and links it to
    libblr_b200.so; the result is copied next to it.  Needs libblr_b200.so built first."""
    if not force and not ext_needs_build():
        return EXT
    import ctypes
    from torch.utils import cpp_extension as ce
    ctypes.CDLL(LIB, mode=ctypes.RTLD_GLOBAL)  # the extension is loaded right after it is built and links against this library
    bdir = os.path.join(HERE, "build", "torch_ext")
    os.makedirs(bdir, exist_ok=True)
    ce.load(name="_blr_torch", sources=[os.path.join(CSRC, "torch_ext.cpp")], extra_cflags=["-O2", "-std=c++17"],
            extra_include_paths=[os.path.join(HERE, "..", "include")], extra_ldflags=[f"-L{HERE}", "-lblr_b200"],
            build_directory=bdir, with_cuda=True, is_python_module=False, verbose=verbose)
    shutil.copyfile(os.path.join(bdir, "_blr_torch.so"), EXT)
    return EXT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_torch_ext(force="--force" in sys.argv, verbose="-v" in sys.argv))
