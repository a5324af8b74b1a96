"""In-tree native build for tnn_b200.

Two shared objects are produced next to this file, under ``_lib/``:

* ``libtnnb_kernels.so`` - every CUDA kernel, compiled by ``nvcc`` for
  ``sm_100a`` only and exported through ``extern "C"`` entry points (loaded
  with ``ctypes``; it does not link against libtorch so it compiles in seconds).
* ``_host.*.so`` - the host-side C++ runtime (typed config, archiver wire
  format, TNNG checkpoints, graph IR, partitioner, CPU oracle engine, profiler,
  data loaders, allocators) as a pybind11 module.

Both are rebuilt only when a source is newer than the output.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
import sysconfig

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
LIB = os.path.join(ROOT, "_lib")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
# The system compiler is preferred over $CXX: toolchain wrappers found in some images
# cannot link OpenMP.
CXX = os.environ.get("TNNB_CXX") or ("/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "--expt-relaxed-constexpr",
]


def _newer(srcs, out):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in srcs)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd[:6]) + " ...")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr)


def kernels_path(bounds_check=False):
    return os.path.join(LIB, "dbg", "libtnnb_kernels.so") if bounds_check else os.path.join(LIB, "libtnnb_kernels.so")


def host_path(sanitize=False):
    ext = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(LIB, "san", "_host" + ext) if sanitize else os.path.join(LIB, "_host" + ext)


# AddressSanitizer + UndefinedBehaviorSanitizer build of the host runtime (the reference's ENABLE_DEBUG build uses
# -fsanitize=address,undefined for its CPU-only configuration, cmake/CompilerFlags.cmake:28-33). The interpreter is not
# instrumented, so a process that imports this variant must start with the ASan runtime preloaded: sanitizer_env().
SAN_FLAGS = ["-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"]


def sanitizer_env(base=None):
    """Environment for a child process that loads the sanitized host runtime (TNNB_HOST_SANITIZE=1)."""
    env = dict(os.environ if base is None else base)
    asan = subprocess.run([CXX, "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    # libstdc++ is preloaded too: ASan looks up the real __cxa_throw when it starts, and the interpreter itself does not
    # link the C++ runtime, so without it the first C++ exception aborts inside the interceptor
    cxxrt = subprocess.run([CXX, "-print-file-name=libstdc++.so.6"], capture_output=True, text=True).stdout.strip()
    env["LD_PRELOAD"] = " ".join(x for x in (asan, cxxrt if os.path.isabs(cxxrt) else "libstdc++.so.6", env.get("LD_PRELOAD", "")) if x)
    # the interpreter's own arenas are not leaks of the runtime; an error must end the process with a non-zero code
    env["ASAN_OPTIONS"] = "detect_leaks=0:abort_on_error=0:exitcode=97:allocator_may_return_null=1"
    env["UBSAN_OPTIONS"] = "print_stacktrace=1:halt_on_error=1:exitcode=98"
    env["TNNB_HOST_SANITIZE"] = "1"
    return env


def build_kernels(verbose=False, force=False, ptxas_info=False, bounds_check=False):
    """``bounds_check=True`` builds the checked variant (``-DTNNB_BOUNDS_CHECK``, see ptx.cuh) into ``_lib/dbg``; a process
    loads it instead of the regular library when ``TNNB_BOUNDS_CHECK=1`` is set."""
    odir = os.path.join(LIB, "dbg") if bounds_check else LIB
    os.makedirs(odir, exist_ok=True)
    kdir = os.path.join(CSRC, "kernels")
    srcs = sorted(glob.glob(os.path.join(kdir, "*.cu")))
    hdrs = glob.glob(os.path.join(kdir, "*.cuh")) + glob.glob(os.path.join(kdir, "*.h"))
    objs = []
    jobs = []
    for s in srcs:
        o = os.path.join(odir, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer([s] + hdrs, o):
            cmd = ([NVCC] + CUDA_FLAGS + (["-DTNNB_BOUNDS_CHECK"] if bounds_check else []) + (["-Xptxas", "-v"] if ptxas_info else [])
                   + ["-I", kdir, "-c", s, "-o", o])
            jobs.append(cmd)
    if jobs:
        procs = []
        for cmd in jobs:
            if verbose:
                print(" ".join(cmd), flush=True)
            procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        for cmd, pr in procs:
            out, _ = pr.communicate()
            if pr.returncode != 0:
                sys.stderr.write(out)
                raise RuntimeError("nvcc failed for " + cmd[-3])
            if (verbose or ptxas_info) and out:
                print(out)
    out = kernels_path(bounds_check)
    if force or jobs or _newer(objs, out):
        _run([NVCC, "-shared", "-o", out] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"], verbose)
    return out


def build_host(verbose=False, force=False, sanitize=False):
    import pybind11

    os.makedirs(os.path.join(LIB, "san") if sanitize else LIB, exist_ok=True)
    hdir = os.path.join(CSRC, "host")
    srcs = sorted(glob.glob(os.path.join(hdir, "*.cc")))
    hdrs = glob.glob(os.path.join(hdir, "*.h"))
    out = host_path(sanitize)
    opt = SAN_FLAGS if sanitize else ["-O2"]
    tag = "host_san_" if sanitize else "host_"
    site = os.path.dirname(os.path.dirname(pybind11.__file__))
    json_inc = os.path.join(site, "include", "cudnn_frontend", "thirdparty")
    objs = []
    procs = []
    for s in srcs:
        o = os.path.join(LIB, tag + os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer([s] + hdrs, o):
            cmd = [CXX] + opt + ["-std=c++17", "-fPIC", "-fopenmp", "-fvisibility=hidden", "-I", hdir,
                   "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
                   "-I", json_inc, "-c", s, "-o", o]
            if verbose:
                print(" ".join(cmd), flush=True)
            procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for s, pr in procs:
        o, _ = pr.communicate()
        if pr.returncode != 0:
            sys.stderr.write(o)
            raise RuntimeError("g++ failed for " + s)
    if force or procs or _newer(objs, out):
        _run([CXX, "-shared", "-fopenmp"] + (["-fsanitize=address,undefined"] if sanitize else []) + ["-o", out] + objs, verbose)
    return out


def build_all(verbose=False, force=False):
    """Every native piece: the kernel library, its bounds-checked variant, and the host runtime."""
    k = build_kernels(verbose, force)
    build_kernels(verbose, force, bounds_check=True)
    return k, build_host(verbose, force)


if __name__ == "__main__":
    build_all(verbose=True, force="--force" in sys.argv)
    print("built:", kernels_path(), host_path())
