"""In-tree builder and loader for the native parts of the package.

Two artefacts are produced next to the Python sources (so that they travel with
a source checkout and are visible in the process's memory map when loaded):

* ``arcticinference_b200/_kernels.so`` -- every ``csrc/*.cu`` file compiled by
  ``nvcc`` for ``sm_100a`` only and linked into one shared library with a plain
  C ABI (``csrc/api.h``); loaded with :mod:`ctypes`.
* ``arcticinference_b200/suffix_decoding/_C*.so`` -- the host-side suffix tree
  (C++17, pybind11).

The reference ships a JIT builder derived from DeepSpeed that compiles for the
visible device's compute capability (arctic_inference/op_builder/builder.py:341-463)
and a loader that looks for a prebuilt library first
(arctic_inference/py_custom_ops.py:9-37). This builder always cross-compiles
for sm_100a, needs no GPU, and rebuilds only what changed.
"""

from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import sys
import sysconfig
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = CSRC / "build"
KERNEL_LIB = PKG_DIR / "_kernels.so"
SUFFIX_LIB_DIR = PKG_DIR / "suffix_decoding"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=default",
]

_lock = threading.Lock()
_kernel_lib: ctypes.CDLL | None = None


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _headers() -> list[Path]:
    return [p for p in CSRC.rglob("*") if p.suffix in (".h", ".cuh", ".hpp")]


def _newest(paths) -> float:
    return max((p.stat().st_mtime for p in paths), default=0.0)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), proc.stdout))
    if os.environ.get("ARCTIC_B200_BUILD_VERBOSE"):
        sys.stderr.write(proc.stdout)


def kernel_sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """Compile ``csrc/*.cu`` for sm_100a and link ``_kernels.so``. Needs no GPU."""
    srcs = kernel_sources()
    hdr_time = _newest(_headers())
    OBJ_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in srcs:
        obj = OBJ_DIR / (src.stem + ".o")
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time)
        if stale:
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            list(pool.map(_run, jobs))
    if jobs or force or not KERNEL_LIB.exists() or KERNEL_LIB.stat().st_mtime < _newest(objs):
        tmp = KERNEL_LIB.with_suffix(".so.tmp%d" % os.getpid())
        _run([nvcc, "-shared", "-o", str(tmp), *[str(o) for o in objs]])
        os.replace(tmp, KERNEL_LIB)
    return KERNEL_LIB


def suffix_lib_path() -> Path:
    ext = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return SUFFIX_LIB_DIR / ("_C" + ext)


def build_suffix_tree(force: bool = False) -> Path:
    """Compile the host-side suffix tree extension (pybind11, C++17)."""
    import pybind11

    src_dir = CSRC / "suffix_tree"
    srcs = sorted(src_dir.glob("*.cc"))
    out = suffix_lib_path()
    if not srcs:
        raise RuntimeError("no suffix-tree sources under %s" % src_dir)
    deps = srcs + list(src_dir.glob("*.h"))
    if not force and out.exists() and out.stat().st_mtime >= _newest(deps):
        return out
    cxx = os.environ.get("CXX", "g++")
    tmp = out.with_suffix(".tmp%d" % os.getpid())
    cmd = [cxx, "-O3", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
           "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
           "-I", str(src_dir), *[str(s) for s in srcs], "-o", str(tmp)]
    if os.environ.get("ARCTIC_B200_SUFFIX_SANITIZE"):
        cmd[1:1] = ["-fsanitize=address,undefined", "-g", "-fno-omit-frame-pointer"]
    _run(cmd)
    os.replace(tmp, out)
    return out


TORCH_OPS_LIB = PKG_DIR / "_torch_ops.so"


def build_torch_ops(force: bool = False) -> Path:
    """Compile ``csrc/torch/torch_bindings.cpp`` (the ``torch.ops.arcticinference_b200``
    namespace) against the installed PyTorch and link it to ``_kernels.so``."""
    import torch
    from torch.utils import cpp_extension

    src = CSRC / "torch" / "torch_bindings.cpp"
    if os.environ.get("ARCTIC_B200_NO_AUTOBUILD") and TORCH_OPS_LIB.exists() and not force:
        return TORCH_OPS_LIB
    build_kernels()
    deps = [src, CSRC / "api.h"]
    if not force and TORCH_OPS_LIB.exists() and \
            TORCH_OPS_LIB.stat().st_mtime >= max(_newest(deps), KERNEL_LIB.stat().st_mtime):
        return TORCH_OPS_LIB
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = []
    for d in cpp_extension.include_paths("cuda") + [str(Path(cuda_home) / "include"),
                                                    sysconfig.get_paths()["include"]]:
        inc += ["-isystem", d]
    torch_lib = str(Path(torch.__file__).parent / "lib")
    cxx = os.environ.get("CXX", "g++")
    tmp = TORCH_OPS_LIB.with_suffix(".so.tmp%d" % os.getpid())
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, str(src), "-o", str(tmp),
           "-L", torch_lib, "-L", str(Path(cuda_home) / "lib64"), "-L", str(PKG_DIR),
           "-l:_kernels.so", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + torch_lib]
    _run(cmd)
    os.replace(tmp, TORCH_OPS_LIB)
    return TORCH_OPS_LIB


def load_torch_ops():
    """Register ``torch.ops.arcticinference_b200`` (building the library if needed)."""
    import torch
    load_kernels()
    torch.ops.load_library(str(build_torch_ops()))
    return torch.ops.arcticinference_b200


def build_all(force: bool = False) -> None:
    if any((CSRC / "suffix_tree").glob("*.cc")):
        build_suffix_tree(force)
    build_kernels(force)
    build_torch_ops(force)


def load_kernels() -> ctypes.CDLL:
    """Load ``_kernels.so`` (building it first when it is missing or stale)."""
    global _kernel_lib
    with _lock:
        if _kernel_lib is None:
            if os.environ.get("ARCTIC_B200_NO_AUTOBUILD"):
                if not KERNEL_LIB.exists():
                    raise RuntimeError("%s is missing and auto-build is disabled" % KERNEL_LIB)
            else:
                build_kernels()
            _kernel_lib = ctypes.CDLL(str(KERNEL_LIB), mode=ctypes.RTLD_GLOBAL)
        return _kernel_lib


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built", KERNEL_LIB, suffix_lib_path())
