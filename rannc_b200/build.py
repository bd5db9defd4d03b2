"""In-tree build of the two native libraries.

* ``_kernels.so`` : every CUDA kernel (``csrc/cuda/*.cu``), compiled by nvcc for
  sm_100a only and exported through a plain C ABI (called with ctypes).
* ``_core.so``    : the host-side native core (``csrc/core/*.cpp``: IR, msgpack
  codec, value classifier, partitioner, stage search, cost model, routes,
  batch arithmetic, event recorder, watchdog) as a pybind11 module.

Both are written next to this file so that they travel with the source tree.
``python -m rannc_b200.build`` builds both; nothing is rebuilt when the
outputs are newer than every source.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CUDA_SRC = HERE / "csrc" / "cuda"
CORE_SRC = HERE / "csrc" / "core"
BUILD_DIR = HERE / "csrc" / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("build command failed:\n  " + " ".join(map(str, cmd)) + "\n" + r.stdout)
    return r.stdout


def build_kernels(verbose: bool = False, debug: bool = False) -> Path:
    """``debug``: the checked build (``_kernels_debug.so``, -DRB_DEBUG_BOUNDS): data-dependent indices are
    range-checked on the device before the kernels that use them run, and a violation is recorded in the device
    error word instead of trapping (see csrc/cuda/debug_check.cuh).  Loaded instead of the regular library when
    RANNC_KERNEL_DEBUG=1."""
    out = HERE / ("_kernels_debug.so" if debug else "_kernels.so")
    srcs = sorted(CUDA_SRC.glob("*.cu"))
    hdrs = sorted(CUDA_SRC.glob("*.cuh")) + sorted(CUDA_SRC.glob("*.h"))
    if _newer(out, srcs + hdrs):
        return out
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    objs = []

    def compile_one(src: Path):
        obj = BUILD_DIR / (src.stem + ("_dbg.o" if debug else ".o"))
        if _newer(obj, [src] + hdrs):
            return obj
        cmd = [_nvcc(), *NVCC_FLAGS, *(["-DRB_DEBUG_BOUNDS"] if debug else []), "-I", str(CUDA_SRC), "-c", str(src),
               "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        log = _run(cmd)
        if verbose:
            print(log)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as ex:
        objs = list(ex.map(compile_one, srcs))
    _run([_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-lcudart"])
    return out


def build_core(verbose: bool = False) -> Path:
    import pybind11

    ext = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    out = HERE / ("_core" + ext)
    srcs = sorted(CORE_SRC.glob("*.cpp"))
    hdrs = sorted(CORE_SRC.glob("*.h"))
    if not srcs:
        return out
    if _newer(out, srcs + hdrs):
        return out
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", str(CORE_SRC)]
    flags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-sign-compare", "-pthread"]

    def compile_one(src: Path):
        obj = BUILD_DIR / ("core_" + src.stem + ".o")
        if _newer(obj, [src] + hdrs):
            return obj
        _run(["g++", *flags, *inc, "-c", str(src), "-o", str(obj)])
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, srcs))
    _run(["g++", "-shared", "-pthread", "-o", str(out), *map(str, objs)])
    return out


def build_selftest(sanitize: str = "address,undefined") -> Path:
    """The native core (everything but the Python bindings) linked into a stand-alone self-test program
    (``csrc/core/selftest.cpp``) with the host sanitizers switched on: ``address,undefined`` (default) or
    ``thread``.  The program exercises the msgpack codec, the IR, the partitioner and stage search, deployment,
    batch arithmetic, the event recorder from several threads and the watchdog; a sanitizer report makes it exit
    non-zero.  This is how the host code is checked for memory errors, undefined behaviour and data races."""
    tag = sanitize.replace(",", "_")
    out = BUILD_DIR / f"core_selftest_{tag}"
    srcs = [p for p in sorted(CORE_SRC.glob("*.cpp")) if p.name != "bindings.cpp"]
    hdrs = sorted(CORE_SRC.glob("*.h"))
    if _newer(out, srcs + hdrs):
        return out
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    flags = ["-O1", "-g", "-std=c++17", "-fno-omit-frame-pointer", f"-fsanitize={sanitize}", "-pthread", "-Wall",
             "-Wno-sign-compare", "-DRANNC_SELFTEST"]
    _run(["g++", *flags, "-I", str(CORE_SRC), *map(str, srcs), "-o", str(out)])
    return out


def build_all(verbose: bool = False):
    return build_core(verbose), build_kernels(verbose)


if __name__ == "__main__":
    if "--debug" in sys.argv:
        print("built", build_kernels(verbose="-v" in sys.argv, debug=True))
    elif "--selftest" in sys.argv:
        print("built", build_selftest("address,undefined"))
        print("built", build_selftest("thread"))
    else:
        c, k = build_all(verbose="-v" in sys.argv)
        print("built", c)
        print("built", k)
