"""In-tree build of the native code: ``python -m sageattention_rdna3_b200.build``.

Two shared objects are produced next to this file (nothing is installed anywhere else):

* ``libsage_b200.so`` - the CUDA kernels and the C ABI of ``include/sage_b200.h``; compiled by nvcc
  for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``), linked against the CUDA runtime.
* ``_C.so`` - the ``torch.ops.sageattention.*`` registrations (``csrc/torch_ops.cpp``); compiled by
  g++ against the installed torch headers and linked against ``libsage_b200.so``.

nvcc cross-compiles, so the build needs no GPU.  It replaces the reference's ROCm-only
``setup.py`` (hipcc, gfx11 arch selection).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_DIR = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
LIB_ABI = PKG_DIR / "libsage_b200.so"
LIB_OPS = PKG_DIR / "_C.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "--cudart", "shared",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _up_to_date(target: Path, sources, extra: str = "") -> bool:
    stamp = target.with_suffix(target.suffix + ".stamp")
    want = _digest(sources) + extra
    return target.exists() and stamp.exists() and stamp.read_text() == want


def _write_stamp(target: Path, sources, extra: str = "") -> None:
    target.with_suffix(target.suffix + ".stamp").write_text(_digest(sources) + extra)


def _run(cmd) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build command failed:\n  " + " ".join(map(str, cmd)) + "\n" + proc.stdout)


def build_abi(force: bool = False, verbose: bool = False) -> Path:
    sources = [CSRC / "sage_abi.cu", CSRC / "attn_kernel.cuh", CSRC / "prep_kernels.cuh", CSRC / "merge_kernels.cuh",
               CSRC / "ptx_sm100.cuh",
               REPO_DIR / "include" / "sage_b200.h"]
    if force or not _up_to_date(LIB_ABI, sources):
        cmd = [_nvcc(), *NVCC_FLAGS, "-o", str(LIB_ABI), str(CSRC / "sage_abi.cu")]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        _run(cmd)
        _write_stamp(LIB_ABI, sources)
    return LIB_ABI


def build_ops(force: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    sources = [CSRC / "torch_ops.cpp", REPO_DIR / "include" / "sage_b200.h"]
    extra = torch.__version__
    if force or not _up_to_date(LIB_OPS, sources, extra):
        torch_lib = Path(torch.__file__).parent / "lib"
        includes = cpp_extension.include_paths("cuda") + [sysconfig.get_paths()["include"]]
        cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
               f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
               "-DTORCH_EXTENSION_NAME=_C"]
        for inc in includes:
            cmd += ["-isystem", str(inc)]
        cmd += [str(CSRC / "torch_ops.cpp"), "-o", str(LIB_OPS),
                f"-L{PKG_DIR}", "-l:libsage_b200.so", f"-L{torch_lib}",
                "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
                "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
        _run(cmd)
        _write_stamp(LIB_OPS, sources, extra)
    return LIB_OPS


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_abi(force=force, verbose=verbose)
    build_ops(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(f"built {LIB_ABI.name} and {LIB_OPS.name} in {PKG_DIR}")
