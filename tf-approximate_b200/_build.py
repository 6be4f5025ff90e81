"""Builds libaxconv.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Every source is compiled to an object of its own, in parallel, then linked.  `build_library(check=True)` builds the
debug flavour libaxconv_check.so (-DAXC_BOUNDS_CHECK: every computed shared-memory address and global index is checked
before use, violations are recorded instead of trapping)."""
import concurrent.futures
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libaxconv.so")
LIB_CHECK = os.path.join(HERE, "libaxconv_check.so")
OBJDIR = os.path.join(HERE, "build")
SOURCES = ["axc_api.cu", "axc_conv.cu", "axc_sched.cu", "axc_depthwise.cu", "axc_probe.cu", "axc_qconv.cu", "axc_prologue.cu"]


def needs_build(lib=LIB):
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, "axconv.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False, check=False):
    lib = LIB_CHECK if check else LIB
    if not force and not needs_build(lib):
        return lib
    nvcc = os.environ.get("NVCC", "nvcc")
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
             "-I" + INCLUDE]
    if verbose:
        flags.append("-Xptxas=-v")
    if check:
        flags.append("-DAXC_BOUNDS_CHECK")
    os.makedirs(OBJDIR, exist_ok=True)
    tag = "check_" if check else ""

    def compile_one(src):
        obj = os.path.join(OBJDIR, tag + src.replace(".cu", ".o"))
        r = subprocess.run([nvcc] + flags + ["-c", os.path.join(CSRC, src), "-o", obj], capture_output=True, text=True)
        return src, obj, r

    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    objs = []
    for src, obj, r in results:
        if verbose or r.returncode != 0:
            print(r.stdout + r.stderr)
        if r.returncode != 0:
            raise subprocess.CalledProcessError(r.returncode, "nvcc -c " + src)
        objs.append(obj)
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", lib] + objs, check=True)
    return lib
