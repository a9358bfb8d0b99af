"""Builds ``libanemoi_sm100.so`` in-tree with nvcc for sm_100a (no other target)."""

from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libanemoi_sm100.so"
SOURCES = ("prepare.cu", "draft.cu", "route.cu", "attention.cu", "assemble.cu", "peaks.cu", "producer.cu", "exchange.cu")
FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
)


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the sm_100a library cannot be built")
    return found


def needs_build() -> bool:
    if not LIBRARY.exists():
        return True
    stamp = LIBRARY.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PACKAGE.parent / "include" / "anemoi_sm100.h"]
    return any(d.stat().st_mtime > stamp for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source and link the shared library next to the package."""
    if not force and not needs_build():
        return LIBRARY
    nvcc = _nvcc()
    objects = []
    procs = []
    out_dir = PACKAGE / "build"
    out_dir.mkdir(exist_ok=True)
    for name in SOURCES:
        obj = out_dir / (name + ".o")
        cmd = [nvcc, *FLAGS, "-c", str(CSRC / name), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(str(obj))
    for name, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {name}:\n{out}")
        if verbose and out:
            print(out)
    link = [nvcc, "-shared", "-o", str(LIBRARY), *objects, "-gencode", "arch=compute_100a,code=sm_100a",
            "-Xcompiler", "-fPIC", "-lcudart"]
    done = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"link failed:\n{done.stdout}")
    return LIBRARY


TORCH_OPS = PACKAGE / "libanemoi_sm100_torch.so"


def build_torch_ops(force: bool = False) -> Path:
    """Compile ``csrc/torch_ops.cpp`` (host code: the ``torch.ops.anemoi_sm100`` registration over
    the C ABI) with g++ against this interpreter's torch and link it to the C-ABI library."""
    import torch
    from torch.utils import cpp_extension

    source = CSRC / "torch_ops.cpp"
    header = PACKAGE.parent / "include" / "anemoi_sm100.h"
    if (not force and TORCH_OPS.exists()
            and TORCH_OPS.stat().st_mtime >= max(source.stat().st_mtime, header.stat().st_mtime, LIBRARY.stat().st_mtime)):
        return TORCH_OPS
    build()
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", str(source), "-o", str(TORCH_OPS)]
    for path in cpp_extension.include_paths():
        cmd += ["-isystem", path]
    cmd += ["-isystem", os.path.join(cuda_home, "include")]
    for path in cpp_extension.library_paths():
        cmd += ["-L" + path, "-Wl,-rpath," + path]
    cmd += ["-L" + str(PACKAGE), "-Wl,-rpath,$ORIGIN", "-lanemoi_sm100", "-lc10", "-lc10_cuda", "-ltorch_cpu",
            "-ltorch_cuda", "-ltorch"]
    done = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"g++ failed on torch_ops.cpp:\n{done.stdout}")
    return TORCH_OPS


if __name__ == "__main__":
    print(build(force=True, verbose=True))
    print(build_torch_ops(force=True))
