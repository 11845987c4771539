"""Builds the native parts of the package in-tree.

  lib/libttb.so   CUDA kernels + the C ABI declared in include/ttb.h   (nvcc, sm_100a only)
  ttnn/_ttnn*.so  C++ host layer + pybind11 surface, linked against libttb.so   (g++)

Run as a script (``python build.py``) or call ``build_all()``. Objects are rebuilt only when their
sources or the shared headers are newer.
"""
import concurrent.futures
import glob
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
HOST = os.path.join(HERE, "host")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "lib")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-I" + os.path.join(ROOT, "include"), "-I" + CSRC]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    return r.stdout + r.stderr


def build_libttb(verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(ROOT, "include", "ttb.h")]
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    jobs = []
    objs = []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if _newer(obj, [src] + headers):
            jobs.append([NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj])
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        for out in ex.map(_run, jobs):
            if verbose and out:
                print(out)
    so = os.path.join(LIB, "libttb.so")
    if _newer(so, objs):
        _run([NVCC, "-shared", "-o", so] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"])
    return so


def build_host(verbose=False):
    """C++ host layer + pybind11 module; skipped (returns None) while the host sources do not exist."""
    sources = sorted(glob.glob(os.path.join(HOST, "*.cpp")))
    if not sources:
        return None
    import pybind11
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    so = os.path.join(HERE, "ttnn", "_ttnn" + ext)
    deps = sources + glob.glob(os.path.join(HOST, "*.hpp")) + [os.path.join(ROOT, "include", "ttb.h")]
    if _newer(so, deps):
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-I" + os.path.join(ROOT, "include"),
               "-I" + HOST, "-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"]] + sources + \
              ["-o", so, "-L" + LIB, "-lttb", "-Wl,-rpath,$ORIGIN/../lib"]
        _run(cmd)
    return so


def build_all(verbose=False):
    lib = build_libttb(verbose)
    host = build_host(verbose)
    return lib, host


if __name__ == "__main__":
    print(build_all(verbose="-v" in sys.argv))
