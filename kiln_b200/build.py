"""Builds the CUDA library in-tree for sm_100a: kiln_b200/lib/libkiln_b200.so.

    python -m kiln_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. The library links the CUDA runtime statically and resolves the
one driver entry point it needs (cuTensorMapEncodeTiled) at run time, so it loads on a machine
without a driver; every launch entry point then fails with KB_ERR_DEVICE.
"""
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIB_DIR, "libkiln_b200.so")
HOST_LIB = os.path.join(LIB_DIR, "libkiln_engine_ops.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-shared", "-I" + INCLUDE]


def _sources(dirs, exts):
    out = []
    for d in dirs:
        for root, _, files in os.walk(d):
            out += [os.path.join(root, f) for f in files if f.endswith(exts)]
    return out


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, defines=(), out=None):
    """Compile csrc/abi.cu (which includes every kernel) into the shared library; returns its path."""
    out = out or LIB
    os.makedirs(os.path.dirname(out), exist_ok=True)
    deps = _sources([CSRC, INCLUDE], (".cu", ".cuh", ".h"))
    if not force and not _stale(out, deps):
        return out
    cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-D" + d for d in defines] + \
          ["-o", out, os.path.join(CSRC, "abi.cu")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + r.stderr[-6000:])
    return out


def build_host(force=False):
    """Compile the C++ host shim (the engine-facing op set) against the C ABI; returns its path."""
    src = os.path.join(PKG, "host", "gpu_ops.cpp")
    deps = _sources([os.path.join(PKG, "host"), INCLUDE], (".cpp", ".h"))
    if not force and not _stale(HOST_LIB, deps + [LIB]):
        return HOST_LIB
    cmd = ["nvcc", "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-I" + INCLUDE, "-o", HOST_LIB, src,
           "-L" + LIB_DIR, "-lkiln_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("host shim build failed:\n" + r.stderr[-6000:])
    return HOST_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if os.path.exists(os.path.join(PKG, "host", "gpu_ops.cpp")):
        print(build_host(force="--force" in sys.argv))
