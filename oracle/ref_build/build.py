"""Builds the reference's own SM120 extension for sm_100a into ``oracle/_ref/``.

Test infrastructure, not product code: the result pins the CPU oracle (and through it the
CUDA path of this repository) to what the reference's kernels compute on identical inputs.
Nothing of the reference is copied: every source is compiled from where the reference tree
lies (``ANEMOI_REFERENCE_ROOT``, default: a ``reference`` directory beside this repository)
through ``wrapper.cu``, with the reference's own nvcc flags (setup.py:158-169; its forced
include of <cassert> is an #include in the wrapper) and
``-gencode arch=compute_100a,code=sm_100a``.  The reference's build system is not run.

What is built: preparation (q128_microscaling_preparation.cu), draft probability
(h3_draft_probability.cu), route + materialise (h3_route_precision.cu), the attention host
(q64_attention_host.cu), the operator registration (bindings.cpp) and the FP16 / INT8 /
INT8+FP16 / dense-prefix instantiations for Q64 and Q128.  The NVFP4 and MXFP8 phases do not
assemble for sm_100a; the launchers they would define are replaced by stubs that abort, made
from the list of undefined symbols of the objects, so that the module loads.

Usage: ``python oracle/ref_build/build.py [-j N]``; output ``oracle/_ref/_ref_sm120.so``
(a torch extension module: importing it registers ``torch.ops.mixed_attention.*``).
"""

from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parents[1]
OUT = REPO / "oracle" / "_ref"
MODULE = "_ref_sm120"

SM120_SOURCES = (
    "q128_microscaling_preparation.cu",
    "h3_draft_probability.cu",
    "h3_route_precision.cu",
    "q64_attention_host.cu",
    "instantiations/inst_q128_k64_d128_fp16.cu",
    "instantiations/inst_q128_k64_d128_int8.cu",
    "instantiations/inst_q128_k64_d128_int8_dense.cu",
    "instantiations/inst_q64_k64_d128_fp16.cu",
    "instantiations/inst_q64_k64_d128_int8.cu",
    "instantiations/inst_q64_k64_d128_int8_fp16.cu",
    "instantiations/inst_q64_k64_d128_int8_dense.cu",
)


def reference_root() -> Path:
    root = Path(os.environ.get("ANEMOI_REFERENCE_ROOT", REPO.parent / "reference"))
    if not (root / "csrc" / "attention" / "cuda" / "sm120").is_dir():
        raise SystemExit(f"reference tree not found at {root}")
    return root


def _run(cmd, log):
    done = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log.write_text(" ".join(map(str, cmd)) + "\n" + done.stdout)
    if done.returncode != 0:
        raise RuntimeError(f"failed: {' '.join(map(str, cmd))}\n{done.stdout[-4000:]}")
    return done.stdout


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("-j", type=int, default=os.cpu_count() or 4)
    args = ap.parse_args()
    from torch.utils import cpp_extension as ext

    ref = reference_root()
    cuda = ref / "csrc" / "attention" / "cuda"
    sm120 = cuda / "sm120"
    OUT.mkdir(parents=True, exist_ok=True)
    obj_dir = OUT / "obj"
    obj_dir.mkdir(exist_ok=True)
    includes = [f"-I{p}" for p in (cuda, cuda.parent, sm120, cuda / "common",
                                   *ext.include_paths("cuda"), sysconfig.get_paths()["include"])]
    defines = [f"-DTORCH_EXTENSION_NAME={MODULE}", "-DTORCH_API_INCLUDE_EXTENSION_H",
               "-D_GLIBCXX_USE_CXX11_ABI=1"]
    nvcc = [os.path.join(ext.CUDA_HOME or "/usr/local/cuda", "bin", "nvcc"),
            "-gencode", "arch=compute_100a,code=sm_100a",
            "-O3", "-std=c++17", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
            "--use_fast_math", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", *defines, *includes]

    def compile_cu(rel: str) -> Path:
        obj = obj_dir / (rel.replace("/", "_") + ".o")
        src = sm120 / rel
        if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, (HERE / "wrapper.cu").stat().st_mtime):
            return obj
        _run([*nvcc, f'-DANEMOI_REF_SOURCE="{src}"', "-c", str(HERE / "wrapper.cu"), "-o", str(obj)],
             obj.with_suffix(".log"))
        return obj

    with ThreadPoolExecutor(max_workers=args.j) as pool:
        objects = list(pool.map(compile_cu, SM120_SOURCES))

    bindings = obj_dir / "bindings.o"
    _run(["g++", "-O3", "-std=c++17", "-fPIC", *defines, *includes, "-c", str(sm120 / "bindings.cpp"),
          "-o", str(bindings)], bindings.with_suffix(".log"))
    objects.append(bindings)

    # Launchers of the phases that cannot be built for sm_100a: every symbol the objects leave
    # undefined that one of the reference's own sources would have defined becomes a stub.
    undefined, defined = set(), set()
    for obj in objects:
        for line in subprocess.run(["nm", str(obj)], stdout=subprocess.PIPE, text=True).stdout.splitlines():
            parts = line.split()
            if len(parts) == 2 and parts[0] == "U":
                undefined.add(parts[1])
            elif len(parts) == 3 and parts[1] in "TWtw":
                defined.add(parts[2])
    wanted = sorted(s for s in undefined - defined
                    if any(k in s for k in ("sm120", "mixed_attention", "prepare_", "mxfp8", "nvfp4")))
    stub_src = obj_dir / "stubs.c"
    with stub_src.open("w") as f:
        f.write("#include <stdio.h>\n#include <stdlib.h>\n")
        for i, sym in enumerate(wanted):
            f.write(f'void anemoi_ref_stub_{i}(void) __asm__("{sym}");\n'
                    f'void anemoi_ref_stub_{i}(void) {{ fprintf(stderr, "not built for sm_100a: {sym}\\n"); abort(); }}\n')
    stubs = obj_dir / "stubs.o"
    _run(["gcc", "-O1", "-fPIC", "-c", str(stub_src), "-o", str(stubs)], stubs.with_suffix(".log"))
    objects.append(stubs)

    lib_dirs = [f"-L{p}" for p in ext.library_paths("cuda")]
    target = OUT / f"{MODULE}.so"
    _run(["g++", "-shared", "-o", str(target), *map(str, objects), *lib_dirs,
          "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
          "-lcudart", "-lcublas", *[f"-Wl,-rpath,{p}" for p in ext.library_paths("cuda")]],
         OUT / "link.log")
    print(f"built {target} ({len(wanted)} stubbed launchers)")


if __name__ == "__main__":
    sys.exit(main())
