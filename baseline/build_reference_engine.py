"""Out-of-tree build of the reference's own C++/CUDA/cuDNN engine and its stock ``trainer`` binary.

The reference's CMake project cannot be configured without a network (it fetches asio, nlohmann_json,
googletest, stb, spdlog and cudnn-frontend) and requires libibverbs and TBB. This script compiles the
UNMODIFIED reference sources directly with g++ / nvcc instead, leaving out only the ``distributed``
module (asio, ibverbs) which the single-GPU trainer does not use:

* every ``src/<module>/*.cpp|*.cu|*.S`` except ``src/distributed`` and ``src/data_loading/stb_image_impl.cpp``
  (the stb headers are not on the machine; ``ref_shims/stb_stub.cpp`` provides failing stand-ins that the
  image-folder loaders link against), plus ``examples/trainer.cpp``;
* ``USE_TBB`` against ``ref_shims/tbb/`` - a small stand-in for the few oneTBB calls the sources make (TBB is not
  installed, and the sources compile in no other threading configuration: ``ThreadWrapper`` names its task arena
  unconditionally and the OpenMP branch uses ``schedule(affinity)``, which g++ rejects); ``USE_CUDA`` + ``USE_CUDNN``, CUDA architecture sm_100 (the project caps
  auto-detection at sm_89 but accepts any ``-DCUDA_ARCH``; cmake/FindCUDA.cmake:65-83);
* third-party headers from what the Python environment ships: cudnn_frontend and its bundled nlohmann
  json, spdlog 1.14 from flashinfer's data directory and the fmt 10.2 headers bundled with it (header-only).

Result: ``<out>/bin/trainer`` (the reference's examples/trainer.cpp). Nothing of this repository's own
engine is compiled or linked into it.

``--fix-block-engine`` (default output ``baseline/_ref/tunx_build_fixed``). As checked out, the reference never hands
its engine object and backend handle to the layers INSIDE a block: ``Graph::compile`` calls ``set_engine`` /
``set_backend_handle`` on the top-level layers (src/nn/graph.cpp:59-66) and ``Block`` forwards every other setter
to its sub-layers (include/nn/block.hpp:22-84) but not these two, so the first dense layer inside an attention or
residual block dereferences a null engine (observed: SIGSEGV in ``DenseLayerImpl::forward_impl`` called from
``FlashAttentionBlockImpl::forward_impl`` on the first step of ``flash_gpt2_small``). With this flag the script
writes a copy of ``block.hpp`` with the two missing forwarders added into ``<out>/overlay/nn/`` and puts that
directory first on the include path. Nothing else differs. Numbers from such a build are labelled as such.

    python baseline/build_reference_engine.py --src <reference checkout> [--out baseline/_ref/tunx_build] [-j 8]
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shlex
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
SKIP_DIRS = {"distributed"}
SKIP_FILES = {"stb_image_impl.cpp", "tunx_lib.cpp"}
# Headers the sources use without including them (they reach them through TBB headers in the stock build).
FORCE_INC = ["-include", "chrono", "-include", "thread", "-include", "mutex", "-include", "iostream", "-include", "immintrin.h"]
DEFS = ["-DUSE_TBB", "-DUSE_CUDA", "-DUSE_CUDNN", "-DNDEBUG", "-DFMT_HEADER_ONLY", "-DSPDLOG_FMT_EXTERNAL"]


def site_packages() -> Path:
    return Path(sysconfig.get_paths()["purelib"])


def make_deps(out: Path) -> Path:
    """A directory of symlinks to the third-party headers, so that no unrelated header of the Python
    packages they live in can shadow one of the reference's."""
    sp = site_packages()
    deps = out / "deps"
    deps.mkdir(parents=True, exist_ok=True)
    links = {
        # the fmt copy that this spdlog release was written against (torch ships a newer, incompatible one)
        "fmt": sp / "flashinfer" / "data" / "spdlog" / "include" / "spdlog" / "fmt" / "bundled",
        "spdlog": sp / "flashinfer" / "data" / "spdlog" / "include" / "spdlog",
        "nlohmann": sp / "include" / "cudnn_frontend" / "thirdparty" / "nlohmann",
        # the cudnn-frontend headers refer to each other as "../include/...": keep them in a directory of that name
        "include": sp / "include",
    }
    for name, target in links.items():
        if not target.exists():
            raise SystemExit(f"missing dependency header: {target}")
        link = deps / name
        if link.is_symlink() or link.exists():
            link.unlink()
        link.symlink_to(target)
    return deps


def sources(src: Path):
    out = []
    for d in sorted((src / "src").iterdir()):
        if not d.is_dir() or d.name in SKIP_DIRS:
            continue
        for f in sorted(d.rglob("*")):
            if f.suffix in (".cpp", ".cu", ".S") and f.name not in SKIP_FILES:
                out.append(f)
    out.append(src / "examples" / "trainer.cpp")
    out.append(HERE / "ref_shims" / "stb_stub.cpp")
    return out


_BLOCK_FIX = """
  void on_set_engine(Engine engine) override {
    Vec<Layer> layers = this->layers();
    for (Layer &layer : layers) {
      layer.get()->set_engine(engine);
    }
  }

  void on_set_backend_handle(void *handle) override {
    Vec<Layer> layers = this->layers();
    for (Layer &layer : layers) {
      layer.get()->set_backend_handle(handle);
    }
  }
"""


def make_overlay(src: Path, out: Path) -> Path:
    """<out>/overlay/nn/block.hpp = the reference's header plus the two forwarders it lacks (see the module text)."""
    text = (src / "include" / "nn" / "block.hpp").read_text()
    anchor = "  void init_impl() override {"
    if anchor not in text or "on_set_engine(" in text:
        raise SystemExit("include/nn/block.hpp does not look as expected; not patching")
    ov = out / "overlay" / "nn"
    ov.mkdir(parents=True, exist_ok=True)
    (ov / "block.hpp").write_text(text.replace(anchor, _BLOCK_FIX.lstrip("\n") + "\n" + anchor, 1))
    return out / "overlay"


OVERLAY: list = []


def compile_cmd(f: Path, obj: Path, src: Path, deps: Path, arch: str):
    inc = [*OVERLAY, f"-I{src / 'include'}", f"-I{deps}", f"-I{deps / 'include'}", f"-I{HERE / 'ref_shims'}", "-I/usr/local/cuda/include"]
    if f.suffix == ".cu":
        return ["nvcc", "-std=c++20", "-O2", f"-arch={arch}", "-rdc=true", "--expt-relaxed-constexpr",
                "-Xcompiler", "-fPIC,-march=x86-64-v3", "-w", *FORCE_INC, *DEFS, *inc, "-c", str(f), "-o", str(obj)]
    if f.suffix == ".S":
        return ["gcc", "-c", str(f), "-o", str(obj)]
    return ["g++", "-std=c++20", "-O2", "-march=x86-64-v3", "-fPIC", "-w", *FORCE_INC, *DEFS, *inc, "-c", str(f),
            "-o", str(obj)]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", required=True)
    ap.add_argument("--out", default="")
    ap.add_argument("--fix-block-engine", action="store_true")
    ap.add_argument("-j", type=int, default=os.cpu_count() or 4)
    ap.add_argument("--arch", default="sm_100")
    a = ap.parse_args()
    a.out = a.out or str(HERE / "_ref" / ("tunx_build_fixed" if a.fix_block_engine else "tunx_build"))
    src, out = Path(a.src).resolve(), Path(a.out).resolve()
    (out / "obj").mkdir(parents=True, exist_ok=True)
    (out / "bin").mkdir(parents=True, exist_ok=True)
    deps = make_deps(out)
    if a.fix_block_engine:
        OVERLAY.append(f"-I{make_overlay(src, out)}")
        (out / "FIXED").write_text("include/nn/block.hpp: on_set_engine / on_set_backend_handle forwarders added\n")
    log = open(out / "build.log", "w")
    jobs = []
    for f in sources(src):
        rel = f.relative_to(src) if src in f.parents else Path("shims") / f.name
        obj = out / "obj" / (str(rel).replace("/", "__") + ".o")
        jobs.append((f, obj, compile_cmd(f, obj, src, deps, a.arch)))

    def run(job):
        f, obj, cmd = job
        if obj.exists() and obj.stat().st_mtime >= f.stat().st_mtime:
            return f, 0, ""
        r = subprocess.run(cmd, capture_output=True, text=True)
        return f, r.returncode, (shlex.join(cmd) + "\n" + r.stdout + r.stderr)

    failed = []
    with cf.ThreadPoolExecutor(a.j) as ex:
        for f, rc, text in ex.map(run, jobs):
            if text:
                log.write(text + "\n")
                log.flush()
            print(("ok   " if rc == 0 else "FAIL ") + str(f), flush=True)
            if rc:
                failed.append((f, text))
    if failed:
        print(f"{len(failed)} translation unit(s) failed; first error:\n{failed[0][1][-4000:]}")
        return 1
    objs = [str(o) for _, o, _ in jobs]
    dlink = out / "obj" / "device_link.o"
    cmds = [
        ["nvcc", f"-arch={a.arch}", "-dlink", "-Xcompiler", "-fPIC", *[o for (f, _, _), o in zip(jobs, objs) if f.suffix == ".cu"],
         "-o", str(dlink)],
        ["g++", "-o", str(out / "bin" / "trainer"), *objs, str(dlink), "-L/usr/local/cuda/lib64",
         "-L/usr/local/cuda/lib64/stubs", "-lcudart", "-lcublas", "-lcublasLt", "-lcudnn", "-lnvrtc", "-lcuda", "-lnvidia-ml",
         "-lpthread", "-ldl", "-lm"],
    ]
    for cmd in cmds:
        r = subprocess.run(cmd, capture_output=True, text=True)
        log.write(shlex.join(cmd) + "\n" + r.stdout + r.stderr + "\n")
        if r.returncode:
            print("link step failed:\n" + (r.stdout + r.stderr)[-4000:])
            return 1
    # the configs the stock trainer is run with travel with the binary (the checkout may not be there at run time)
    import shutil
    shutil.copytree(src / "configs", out / "configs", dirs_exist_ok=True)
    print("built", out / "bin" / "trainer")
    return 0


if __name__ == "__main__":
    sys.exit(main())
