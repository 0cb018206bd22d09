"""In-tree build of the native pieces (no network, no cmake needed).

Stands in for distributed-kernels/CMakeLists.txt of the reference (hipcc + gfx950 flags, CPM
fetch of iris, MPI, pybind11; one `tk_kernel` module per kernel directory plus `iris_py`):

  libdk_b200.so   CUDA kernels + C ABI (include/dk_b200.h), nvcc, sm_100a only
  iris_py*.so     pybind11 module, same classes as the reference's iris_py
  tk_kernel*.so   pybind11 module with dispatch_micro and the added entry points

nvcc cross-compiles without a GPU. Objects are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
ROOT = PKG.parent
OBJ = PKG / "build"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-cudart", "static"]

CUDA_SOURCES = ["dk_host.cu", "dk_gemm.cu", "dk_allreduce.cu", "dk_moe.cu", "dk_mx.cu",
                "dk_moe_gemm.cu", "dk_moe_ep.cu", "dk_moe_layer.cu", "dk_heap.cu"]
CPP_SOURCES = ["dk_comm.cpp"]
PYBIND_MODULES = {"iris_py": "iris_py.cpp", "tk_kernel": "tk_kernel.cpp"}


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + " ".join(str(c) for c in cmd))
    return r.stdout + r.stderr


def _headers():
    return list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list((ROOT / "include").glob("*.h"))


def build_lib(verbose: bool = False, ptxas_info: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    hdrs = _headers()
    objs = []
    log = ""
    for src in CUDA_SOURCES:
        s = CSRC / src
        if not s.exists():
            continue
        o = OBJ / (src + ".o")
        if ptxas_info or _newer(o, [s] + hdrs):
            extra = ["-Xptxas", "-v"] if ptxas_info else []
            log += _run([NVCC, *ARCH, *NVCC_FLAGS, *extra, "-I", ROOT / "include", "-c", s, "-o", o],
                        verbose)
        objs.append(o)
    for src in CPP_SOURCES:
        s = CSRC / src
        if not s.exists():
            continue
        o = OBJ / (src + ".o")
        if _newer(o, [s] + hdrs):
            _run(["g++", "-O2", "-std=c++17", "-fPIC", "-I", ROOT / "include", "-c", s, "-o", o],
                 verbose)
        objs.append(o)
    lib = PKG / "libdk_b200.so"
    if _newer(lib, objs):
        _run([NVCC, *ARCH, "-shared", "-cudart", "static", "-o", lib, *objs, "-lpthread", "-ldl",
              "-lrt"], verbose)
    if ptxas_info:
        (OBJ / "ptxas_info.txt").write_text(log)
    return lib


def build_pybind(verbose: bool = False):
    import pybind11

    ext = sysconfig.get_config_var("EXT_SUFFIX")
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I",
           ROOT / "include"]
    outs = []
    for name, src in PYBIND_MODULES.items():
        s = CSRC / src
        if not s.exists():
            continue
        out = PKG / f"{name}{ext}"
        if _newer(out, [s, PKG / "libdk_b200.so"] + _headers()):
            _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", *inc, s,
                  "-o", out, f"-L{PKG}", "-ldk_b200", "-Wl,-rpath,$ORIGIN"], verbose)
        outs.append(out)
    return outs


def build_all(verbose: bool = False):
    lib = build_lib(verbose)
    mods = build_pybind(verbose)
    return lib, mods


if __name__ == "__main__":
    v = "-v" in sys.argv
    if "--ptxas" in sys.argv:
        build_lib(v, ptxas_info=True)
        print((OBJ / "ptxas_info.txt").read_text())
    else:
        print(build_all(v))
