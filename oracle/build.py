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
REF_ENGINE = os.path.join(REF_DIR, "kiln-engine-ref")            # the reference's engine, its own kernels
REF_ENGINE_SHIM = os.path.join(REF_DIR, "kiln-engine-shim")      # the same engine over this repository's library
# engine/build.bat's source list without its two Win32-only files (safetensors.cpp, image_io.cpp: oracle/posix/ has
# POSIX ones behind the same headers) and without the optional face-detector / upscaler modules
ENGINE_UNITS = ["main.cpp", "graph.cpp", "kernels.cu", "te.cu", "dit.cu", "train.cu", "tagger.cu", "vae.cu", "pipeline.cu",
                "sdops.cu", "sdxl.cu", "clip.cu", "sdvae.cu", "sdpipe.cu"]
OP_RENAMES = ["-D%s=ref_own_%s" % (n, n) for n in ("attention", "attention16", "rmsnorm", "rope_half", "linear16", "gpu_alloc_scratch")]


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


def build_ref_engine(ref_root, force=False):
    """The reference's engine executable (engine/build.bat's recipe) for Linux and sm_100a, twice: over its own kernels and
    over this repository's library. Its sources are compiled where they lie; the three stand-ins under oracle/posix/
    (windows.h, io.h and the POSIX halves of the safetensors and image readers) are all that is added."""
    from concurrent.futures import ThreadPoolExecutor
    src_dir = os.path.join(ref_root, "engine", "src")
    if not os.path.isdir(src_dir):
        raise FileNotFoundError(ref_root)
    root = os.path.dirname(HERE)
    posix = os.path.join(HERE, "posix")
    lib = os.path.join(root, "kiln_b200", "lib")
    own = [os.path.join(posix, f) for f in ("windows.h", "io.h", "safetensors_posix.cpp", "image_io_posix.cpp")] + \
          [os.path.join(HERE, f) for f in ("ref_engine_bind.cu", "ref_engine_train_bind.cu", "ref_ops_binding.h")] + \
          [os.path.join(root, "kiln_b200", "host", "gpu_ops.h"), os.path.join(root, "include", "kiln_b200.h")]
    if not force and _newer(REF_ENGINE, *own) and _newer(REF_ENGINE_SHIM, *own):
        return REF_ENGINE, REF_ENGINE_SHIM
    obj = os.path.join(REF_DIR, "engine_obj")
    os.makedirs(obj, exist_ok=True)
    nvcc = ["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-I" + posix, "-I" + src_dir]
    jobs = [(os.path.join(src_dir, u), os.path.join(obj, u.rsplit(".", 1)[0] + ".o"), []) for u in ENGINE_UNITS]
    jobs.append((os.path.join(src_dir, "kernels.cu"), os.path.join(obj, "kernels_renamed.o"), OP_RENAMES))
    jobs.append((os.path.join(HERE, "ref_engine_bind.cu"), os.path.join(obj, "bind.o"),
                 ["-I" + HERE, "-I" + os.path.join(root, "kiln_b200", "host"), "-I" + os.path.join(root, "include")]))
    jobs.append((os.path.join(HERE, "ref_engine_train_bind.cu"), os.path.join(obj, "train_bound.o"), []))
    jobs.append((os.path.join(posix, "safetensors_posix.cpp"), os.path.join(obj, "safetensors_posix.o"), []))
    jobs.append((os.path.join(posix, "image_io_posix.cpp"), os.path.join(obj, "image_io_posix.o"), []))

    def compile_one(job):
        src, out, extra = job
        return subprocess.run(nvcc + extra + ["-x", "cu", "-c", src, "-o", out], capture_output=True, text=True)

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        for job, r in zip(jobs, pool.map(compile_one, jobs)):
            if r.returncode != 0:
                raise RuntimeError("reference engine: %s failed to compile:\n%s" % (job[0], r.stderr[-4000:]))
    common = [os.path.join(obj, u.rsplit(".", 1)[0] + ".o") for u in ENGINE_UNITS if u not in ("kernels.cu", "train.cu")] + \
             [os.path.join(obj, "safetensors_posix.o"), os.path.join(obj, "image_io_posix.o")]
    r = subprocess.run(["nvcc", "-o", REF_ENGINE] + common + [os.path.join(obj, "kernels.o"), os.path.join(obj, "train.o"), "-lcublas"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference engine: link failed:\n" + r.stderr[-4000:])
    r = subprocess.run(["nvcc", "-o", REF_ENGINE_SHIM] + common + [os.path.join(obj, "kernels_renamed.o"), os.path.join(obj, "train_bound.o"), os.path.join(obj, "bind.o"),
                        "-L" + lib, "-lkiln_engine_ops", "-lkiln_b200", "-lcublas", "-Xlinker", "-rpath=$ORIGIN/../../kiln_b200/lib"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference engine over the library: link failed:\n" + r.stderr[-4000:])
    return REF_ENGINE, REF_ENGINE_SHIM


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    if "--ref" in sys.argv:
        print(build_ref(sys.argv[sys.argv.index("--ref") + 1], force=True))
        print(build_ref_shim(sys.argv[sys.argv.index("--ref") + 1], force=True))
        print(*build_ref_engine(sys.argv[sys.argv.index("--ref") + 1], force=True))
