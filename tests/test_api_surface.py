"""The parts of the public C API that need no team, driven from a C program (tests/data/api_surface.c): header
inlines, status strings, configuration read / modify / print, the team-library list and attributes, and the capability
filter of xccl_lib_init. The header is compiled as strict C11 with warnings as errors."""
import shutil
import subprocess
from pathlib import Path

import pytest

from xccl_b200 import _capi as K

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(shutil.which("cc") is None, reason="needs a C compiler")
def test_api_surface_from_c(tmp_path):
    K.load()  # builds the library when it is missing
    exe = tmp_path / "api_surface"
    lib_dir = ROOT / "xccl_b200" / "lib"
    cmd = ["cc", "-std=c11", "-D_POSIX_C_SOURCE=200809L", "-Wall", "-Wextra", "-Werror", f"-I{ROOT / 'include'}",
           str(ROOT / "tests" / "data" / "api_surface.c"), f"-L{lib_dir}", "-lxccl", f"-Wl,-rpath,{lib_dir}", "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "api surface ok" in r.stdout
