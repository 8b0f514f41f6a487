"""Build recipe for the test oracle (TEST INFRASTRUCTURE; the shipped library never uses it).

    python oracle/build.py            # oracle/libkiln_oracle.so  (CPU restatement, gcc + OpenMP)
    python oracle/build.py --ref DIR  # oracle/_ref/libkiln_ref.so (the reference's own CUDA kernels,
                                      # compiled for sm_100a from the sources where they lie under DIR)

Nothing from the reference tree is copied: ref_wrap.cu only #includes its files by path, and the
output goes to oracle/_ref/, which is kept out of version control.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libkiln_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libkiln_ref.so")
REF_SHIM_SO = os.path.join(REF_DIR, "libkiln_ref_shim.so")


def _gomp_dir():
    """Directory of libgomp.spec as gcc itself reports it, for images whose gcc wrapper does not find it for -fopenmp."""
    try:
        path = subprocess.run(["gcc", "-print-file-name=libgomp.spec"], capture_output=True, text=True).stdout.strip()
    except OSError:
        return None
    return os.path.dirname(path) + os.sep if os.path.isabs(path) and os.path.exists(path) else None


def _newer(target, *deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build_oracle(force=False):
    src = os.path.join(HERE, "kiln_oracle.c")
    if not force and _newer(ORACLE_SO, src):
        return ORACLE_SO
    base = ["gcc", "-O3", "-fopenmp", "-fPIC", "-mavx2", "-mfma", "-fno-math-errno", "-shared", "-o", ORACLE_SO, src, "-lm"]
    r = subprocess.run(base, capture_output=True, text=True)
    gomp = _gomp_dir()
    if r.returncode != 0 and gomp:
        r = subprocess.run(base[:1] + ["-B" + gomp] + base[1:], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + r.stderr)
    return ORACLE_SO


def build_ref(ref_root, force=False):
    """Compile the reference's attention / norm / rope / NAG kernels for sm_100a (GPU-side oracle)."""
    src = os.path.join(HERE, "ref_wrap.cu")
    if not os.path.isdir(os.path.join(ref_root, "engine", "src")):
        raise FileNotFoundError(ref_root)
    if not force and _newer(REF_SO, src):
        return REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = ["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-Xcompiler", "-fPIC", "-shared", "-I" + os.path.join(ref_root, "engine", "src"),
           "-I" + os.path.join(ref_root, "bench"), "-o", REF_SO, src, "-lcublas", "-Xlinker", "--no-undefined"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference kernel build failed:\n" + r.stderr[-4000:])
    return REF_SO


def build_ref_shim(ref_root, force=False):
    """The same translation unit with the attention-path ops bound to the library (kiln_b200/host/gpu_ops.h): the
    reference's own DiT driver over this repository's kernels. Needs the product libraries built (kiln_b200/lib)."""
    src = os.path.join(HERE, "ref_wrap.cu")
    root = os.path.dirname(HERE)
    lib = os.path.join(root, "kiln_b200", "lib")
    deps = [os.path.join(lib, "libkiln_engine_ops.so"), os.path.join(lib, "libkiln_b200.so")]
    for d in deps:
        if not os.path.exists(d):
            raise FileNotFoundError(d)
    if not os.path.isdir(os.path.join(ref_root, "engine", "src")):
        raise FileNotFoundError(ref_root)
    if not force and _newer(REF_SHIM_SO, src, os.path.join(root, "kiln_b200", "host", "gpu_ops.h"), os.path.join(root, "include", "kiln_b200.h")):
        return REF_SHIM_SO
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = ["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-DKILN_OPS_FROM_SHIM",
           "-Xcompiler", "-fPIC", "-shared", "-I" + os.path.join(ref_root, "engine", "src"),
           "-I" + os.path.join(ref_root, "bench"), "-I" + os.path.join(root, "kiln_b200", "host"), "-I" + os.path.join(root, "include"),
           "-o", REF_SHIM_SO, src, "-L" + lib, "-lkiln_engine_ops", "-lkiln_b200", "-lcublas",
           "-Xlinker", "-rpath=$ORIGIN/../../kiln_b200/lib", "-Xlinker", "-Bsymbolic", "-Xlinker", "--no-undefined"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference driver over the library: build failed:\n" + r.stderr[-4000:])
    return REF_SHIM_SO


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    if "--ref" in sys.argv:
        print(build_ref(sys.argv[sys.argv.index("--ref") + 1], force=True))
        print(build_ref_shim(sys.argv[sys.argv.index("--ref") + 1], force=True))
