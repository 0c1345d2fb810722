"""In-tree build of the native libraries.

* ``_lib/libgvkernels.so``  -- the sm_100a CUDA kernel library (plain C ABI, loaded with ctypes)
* ``_lib/dp_core*.so``      -- the C++ dynamic-programming search core (pybind11 module)
* ``_lib/data_index*.so``   -- the C++ dataset index builder (pybind11 module)

The reference builds its single native module with setuptools (setup.py:39-44) and a Makefile
(Makefile:1-16); here nvcc / g++ are called directly so that the built objects stay inside the
package directory and a stale build is detected from a hash of the sources and flags.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "_lib"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O3",
    "--expt-relaxed-constexpr",
]

CUDA_SOURCES = [
    "gemm_sm100.cu",
    "attention_sm100.cu",
    "norm.cu",
    "elementwise.cu",
    "comm_kernels.cu",
    "fused_gemm_sm100.cu",
    "nvlink_bench.cu",
    "no_alloc.cu",
    "bench_kernels.cu",
    "runtime_host.cu",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the sm_100a kernel library cannot be built")


def _hash_sources(files, flags) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for f in sorted(files):
        h.update(str(f.name).encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def _existing(names):
    return [CSRC / n for n in names if (CSRC / n).exists()]


def cuda_lib_path() -> Path:
    return LIB_DIR / "libgvkernels.so"


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``.cu`` of the kernel library for sm_100a and link ``libgvkernels.so``."""
    LIB_DIR.mkdir(exist_ok=True)
    srcs = _existing(CUDA_SOURCES)
    headers = sorted((CSRC / "include").glob("*"))
    digest = _hash_sources(srcs + headers, NVCC_FLAGS)
    out = cuda_lib_path()
    stamp = LIB_DIR / "libgvkernels.hash"
    if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    nvcc = _nvcc()
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    cmd = [nvcc, "-shared", "-o", str(out), *map(str, objs), "-lcudart", "-Xcompiler", "-fPIC"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(digest)
    return out


def _build_pybind(name: str, source: str, force: bool = False) -> Path:
    import pybind11

    LIB_DIR.mkdir(exist_ok=True)
    src = CSRC / source
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    flags = ["-O3", "-std=c++17", "-fPIC", "-shared", "-fopenmp", "-march=x86-64-v3", "-fvisibility=hidden"]
    lib_dir = LIB_DIR
    sanitize = os.environ.get("GV_SANITIZE")          # e.g. "address,undefined": instrumented host modules in their own folder
    if sanitize:
        flags = ["-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=" + sanitize] + flags[1:]
        lib_dir = LIB_DIR / ("san_" + sanitize.replace(",", "_"))
        lib_dir.mkdir(exist_ok=True)
    out = lib_dir / f"{name}{suffix}"
    digest = _hash_sources([src], flags)
    stamp = lib_dir / f"{name}.hash"
    if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    cmd = ["g++", *flags, "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], str(src), "-o", str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed for {source}:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(digest)
    return out


def build_dp_core(force: bool = False) -> Path:
    return _build_pybind("dp_core", "dp_core.cpp", force)


def build_data_index(force: bool = False) -> Path:
    return _build_pybind("data_index", "data_index.cpp", force)


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force, verbose)
    if (CSRC / "dp_core.cpp").exists():
        build_dp_core(force)
    if (CSRC / "data_index.cpp").exists():
        build_data_index(force)


def load_pybind(name: str):
    """Import a pybind11 module built by this file (building it first if it is missing)."""
    import importlib.util

    builder = {"dp_core": build_dp_core, "data_index": build_data_index}[name]
    path = builder()
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print("built:", sorted(p.name for p in LIB_DIR.iterdir() if p.suffix == ".so"))
