"""Builds the UNMODIFIED reference (openucx/xccl) core, utilities, CUDA memory component and NCCL
team from a read-only source tree into ``baseline/_ref/lib`` against the UCS stand-in headers of
``baseline/ucs_shim`` (the image has no UCX, MPI or autotools, so ``./configure`` cannot run).

    python baseline/build_ref.py [--src <checkout of openucx/xccl>]   (default: the directory `reference` beside this repository)

Layout produced (what the reference's own plugin loader expects next to libxccl.so):
    baseline/_ref/lib/libxccl.so
    baseline/_ref/lib/xccl/xccl_team_lib_nccl.so
    baseline/_ref/lib/xccl/xccl_cuda_mem_component.so
Nothing of the reference is copied into the repository; only objects and shared libraries are
written, under the git-ignored ``baseline/_ref``.
"""
from __future__ import annotations

import argparse
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
SHIM = HERE / "ucs_shim"
OUT = HERE / "_ref"
NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
CUDA_HOME = Path(NVCC).resolve().parent.parent


def run(cmd: list) -> None:
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
        raise SystemExit(f"reference build failed (exit {r.returncode})")


def build(src: Path) -> Path:
    s = src / "src"
    lib = OUT / "lib"
    obj = OUT / "obj"
    (lib / "xccl").mkdir(parents=True, exist_ok=True)
    obj.mkdir(parents=True, exist_ok=True)
    (OUT / "include").mkdir(exist_ok=True)
    (OUT / "include" / "config.h").write_text("/* generated: stands in for the autoconf header */\n#define HAVE_CUDA 1\n")
    inc = [f"-I{OUT / 'include'}", f"-I{SHIM}", f"-I{s}", f"-I{s / 'api'}", f"-I{s / 'core'}", f"-I{s / 'utils'}",
           f"-I{s / 'utils' / 'cuda'}", f"-I{s / 'team_lib' / 'nccl'}", f"-I{CUDA_HOME / 'include'}"]
    cflags = ["-O2", "-g", "-fPIC", "-std=gnu11", "-w", "-D_GNU_SOURCE"]

    def cc(files, out, extra=()):
        objs = []
        for f in files:
            o = obj / (f.stem + ".o")
            run(["gcc", *cflags, *inc, "-c", f, "-o", o])
            objs.append(o)
        run(["gcc", "-shared", "-o", out, *objs, *extra])

    core = sorted((s / "core").glob("*.c")) + [s / "utils" / "mem_component.c", s / "utils" / "socketid.c", SHIM / "ucs_shim.c"]
    cc(core, lib / "libxccl.so", ["-ldl", "-lpthread"])
    # CUDA memory component: the reference's three kernels, compiled for sm_100a
    cu_objs = []
    for f in sorted((s / "utils" / "cuda" / "kernels").glob("*.cu")):
        o = obj / (f.stem + ".cu.o")
        run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-Xcompiler", "-fPIC", "-w", *inc, "-c", f, "-o", o])
        cu_objs.append(o)
    o = obj / "cuda_mem_component.o"
    run(["gcc", *cflags, *inc, "-c", s / "utils" / "cuda" / "cuda_mem_component.c", "-o", o])
    run([NVCC, "-shared", "-o", lib / "xccl" / "xccl_cuda_mem_component.so", o, *cu_objs, f"-L{lib}", "-lxccl",
         "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/.."])
    # NCCL team
    nccl = sorted((s / "team_lib" / "nccl").glob("*.c"))
    cc(nccl, lib / "xccl" / "xccl_team_lib_nccl.so",
       [f"-L{lib}", "-lxccl", "-l:libnccl.so.2", f"-L{CUDA_HOME / 'lib64'}", "-lcudart", "-Wl,-rpath,$ORIGIN/.."])
    return lib / "libxccl.so"


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--src", default=str(HERE.parent.parent / "reference"))
    a = ap.parse_args()
    print(build(Path(a.src)))
