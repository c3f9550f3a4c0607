"""In-tree build of the native library.

`python -m xccl_b200.build` compiles every source under ``csrc/`` (host code with g++,
device code with nvcc for sm_100a only) and links ``xccl_b200/lib/libxccl.so``; with
``--torch`` it also builds the c10d backend extension ``xccl_b200/lib/xccl_torch.so``.
Objects are rebuilt when their source or any header is newer. No GPU is needed to build.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
OUT_DIR = ROOT / "xccl_b200" / "lib"
OBJ_DIR = ROOT / "build" / "obj"

NVCC = os.environ.get("NVCC", shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_INC = [f"-I{ROOT / 'include'}", f"-I{CSRC}"]
CXX_FLAGS = ["-std=c++20", "-O2", "-g", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread", "-fvisibility=default"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-Wall", "-Xcompiler", "-Wno-unused-function"] + ARCH_FLAGS

TORCH_DIR = CSRC / "torch"


def _cuda_include() -> list[str]:
    home = Path(NVCC).resolve().parent.parent
    return [f"-I{home / 'include'}"]


def _newest_header() -> float:
    newest = 0.0
    for base in (CSRC, ROOT / "include"):
        for p in base.rglob("*"):
            if p.suffix in (".h", ".hpp", ".cuh"):
                newest = max(newest, p.stat().st_mtime)
    return newest


def _sources() -> list[Path]:
    out = []
    for p in sorted(CSRC.rglob("*")):
        if TORCH_DIR in p.parents:
            continue
        if p.suffix in (".cc", ".cu"):
            out.append(p)
    return out


def _obj_for(src: Path, sanitize: str | None = None) -> Path:
    rel = src.relative_to(CSRC)
    base = OBJ_DIR if not sanitize else OBJ_DIR.parent / f"obj-{sanitize}"
    return base / (str(rel).replace("/", "__") + ".o")


def _compile(src: Path, obj: Path, verbose: bool, ptxas_v: bool, sanitize: str | None = None) -> tuple[Path, int, str]:
    if sanitize == "bounds":
        # device-side bounds checks of the NVLink kernels (csrc/tl/nvlink/nvl_kernels.cu); host code as usual
        san = []
        extra = ["-DXCCL_DEBUG_BOUNDS"]
    else:
        san = [f"-fsanitize={sanitize}", "-fno-omit-frame-pointer"] if sanitize else []
        extra = []
    if src.suffix == ".cu":
        cmd = [NVCC, *NVCC_FLAGS, *extra, *COMMON_INC, "-c", str(src), "-o", str(obj)]
        for f in san:
            cmd[1:1] = ["-Xcompiler", f]
        if ptxas_v:
            cmd[1:1] = ["-Xptxas", "-v"]
    else:
        cmd = [CXX, *CXX_FLAGS, *san, *extra, *COMMON_INC, *_cuda_include(), "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    return src, r.returncode, (r.stdout + r.stderr)


def build_native(force: bool = False, verbose: bool = False, ptxas_v: bool = False, jobs: int | None = None,
                 sanitize: str | None = None) -> Path:
    """sanitize = "address" or "thread": host code (and the host side of the .cu files) is compiled with that
    sanitizer into xccl_b200/lib/libxccl_<sanitize>.so; run the CPU tests on it with
    ``LD_PRELOAD=$(gcc -print-file-name=libasan.so) XCCL_B200_LIB=.../libxccl_address.so python -m pytest ...``."""
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    if sanitize:
        (OBJ_DIR.parent / f"obj-{sanitize}").mkdir(parents=True, exist_ok=True)
    hdr = _newest_header()
    todo, objs = [], []
    for src in _sources():
        obj = _obj_for(src, sanitize)
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr)
        if stale:
            todo.append((src, obj))
    failed = False
    if todo:
        with cf.ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
            futs = [ex.submit(_compile, s, o, verbose, ptxas_v, sanitize) for s, o in todo]
            for f in cf.as_completed(futs):
                src, rc, log = f.result()
                if rc != 0:
                    failed = True
                    print(f"FAILED {src}\n{log}", file=sys.stderr, flush=True)
                elif log.strip() and (verbose or ptxas_v):
                    print(f"--- {src.relative_to(ROOT)}\n{log}", flush=True)
    if failed:
        raise RuntimeError("native build failed")
    lib = OUT_DIR / ("libxccl.so" if not sanitize else f"libxccl_{sanitize}.so")
    if todo or not lib.exists():
        cmd = [NVCC, "-shared", *ARCH_FLAGS, "-o", str(lib), *map(str, objs), "-lpthread", "-ldl", "-lrt",
               "-cudart", "static"]
        if sanitize and sanitize != "bounds":
            cmd += ["-Xcompiler", f"-fsanitize={sanitize}"]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            print(r.stdout + r.stderr, file=sys.stderr)
            raise RuntimeError("link failed")
    return lib


def build_torch_ext(force: bool = False, verbose: bool = False) -> Path | None:
    """Builds the c10d backend. Needs torch headers; returns None when there are no sources."""
    srcs = sorted(TORCH_DIR.glob("*.cpp"))
    if not srcs:
        return None
    import torch
    from torch.utils import cpp_extension as ce

    OUT_DIR.mkdir(parents=True, exist_ok=True)
    target = OUT_DIR / "xccl_torch.so"
    lib = OUT_DIR / "libxccl.so"
    newest = max([p.stat().st_mtime for p in srcs] + [_newest_header(), lib.stat().st_mtime if lib.exists() else 0])
    if target.exists() and not force and target.stat().st_mtime >= newest:
        return target
    inc = [f"-I{p}" for p in ce.include_paths()] + COMMON_INC + _cuda_include()
    import sysconfig
    inc.append(f"-I{sysconfig.get_paths()['include']}")
    torch_lib = Path(torch.__file__).parent / "lib"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [CXX, "-std=c++17", "-O2", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
           "-DTORCH_EXTENSION_NAME=xccl_torch", "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, *map(str, srcs),
           "-o", str(target), f"-L{OUT_DIR}", "-lxccl", f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10",
           "-ltorch_python", "-ltorch_cuda", "-lc10_cuda", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        print(r.stdout + r.stderr, file=sys.stderr)
        raise RuntimeError("torch extension build failed")
    return target


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-v", action="store_true", help="print registers / spills / shared memory per kernel")
    ap.add_argument("--torch", action="store_true", help="also build the c10d backend extension")
    ap.add_argument("-j", type=int, default=None)
    ap.add_argument("--sanitize", choices=["address", "thread"], default=None,
                    help="build libxccl_<sanitizer>.so with the host code instrumented (CPU tests only)")
    ap.add_argument("--debug-bounds", action="store_true",
                    help="build libxccl_bounds.so: the NVLink kernels check every workspace / peer access against the "
                         "ranges of the launch and record (never make) an access outside them")
    a = ap.parse_args()
    lib = build_native(a.force, a.verbose, a.ptxas_v, a.j, "bounds" if a.debug_bounds else a.sanitize)
    print(f"built {lib}")
    if a.torch:
        t = build_torch_ext(a.force, a.verbose)
        print(f"built {t}")


if __name__ == "__main__":
    main()
