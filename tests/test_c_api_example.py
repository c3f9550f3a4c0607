"""The public headers compile as C and a C program can drive the library end to end (the reference's
tests are C programs over the same call sequence, test/test_mpi.c:99-197)."""
import shutil
import subprocess
from pathlib import Path

import pytest

from xccl_b200 import _capi as K

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(shutil.which("cc") is None, reason="needs a C compiler")
@pytest.mark.parametrize("ranks", [1, 4, 6])
def test_c_example_builds_and_runs(tmp_path, ranks):
    K.load()  # builds the library when it is missing
    exe = tmp_path / "allreduce_host"
    lib_dir = ROOT / "xccl_b200" / "lib"
    cmd = ["cc", "-std=c11", "-Wall", "-Werror", f"-I{ROOT / 'include'}", str(ROOT / "examples" / "allreduce_host.c"),
           f"-L{lib_dir}", "-lxccl", f"-Wl,-rpath,{lib_dir}", "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe), str(ranks)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert f"correct on {ranks} ranks" in r.stdout


def _build_gpu_example(tmp_path):
    """examples/allreduce_nvlink.c (run it by hand on a box with two or more GPUs: ``./allreduce_nvlink 2``)."""
    exe = tmp_path / "allreduce_nvlink"
    lib_dir = ROOT / "xccl_b200" / "lib"
    cuda = Path("/usr/local/cuda")
    cmd = ["cc", "-std=c11", "-Wall", "-Werror", f"-I{ROOT / 'include'}", f"-I{cuda / 'include'}",
           str(ROOT / "examples" / "allreduce_nvlink.c"), f"-L{lib_dir}", "-lxccl", f"-L{cuda / 'lib64'}", "-lcudart",
           f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{cuda / 'lib64'}", "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


@pytest.mark.skipif(shutil.which("cc") is None or not Path("/usr/local/cuda/include/cuda_runtime_api.h").exists(),
                    reason="needs a C compiler and the CUDA toolkit")
def test_gpu_example_builds(tmp_path):
    """The device-buffer example compiles as C11 against the public headers and links (no GPU needed for that)."""
    K.load()
    _build_gpu_example(tmp_path)
