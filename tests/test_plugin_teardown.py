"""Plugin loading through XCCL_TEAM_LIB_PATH and the library's teardown at process exit: every opened team
library is closed and plugin objects are unloaded (reference: src/core/xccl_init.c:59-124 loads
``xccl_team_lib_*.so`` from a directory, src/core/xccl_finalize.c:18-42 closes and unloads them)."""
import os
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs a C++ compiler")
def test_plugin_is_opened_closed_and_unloaded(tmp_path):
    so = tmp_path / "xccl_team_lib_demo.so"
    lib_dir = ROOT / "xccl_b200" / "lib"
    subprocess.run(["g++", "-std=c++20", "-O1", "-fPIC", "-shared", f"-I{ROOT / 'include'}", f"-I{ROOT / 'csrc'}",
                    str(ROOT / "tests" / "data" / "plugin_tl.cc"), "-o", str(so), f"-L{lib_dir}", "-lxccl",
                    f"-Wl,-rpath,{lib_dir}"], check=True)
    log = tmp_path / "life.log"
    code = ("from xccl_b200.api import Lib\n"
            "lib = Lib()\n"
            "print('tls', lib.tl_list() if hasattr(lib, 'tl_list') else '')\n"
            "lib.close()\n")
    env = dict(os.environ, XCCL_TEAM_LIB_PATH=str(tmp_path), XCCL_DEMO_PLUGIN_LOG=str(log), PYTHONPATH=str(ROOT))
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    assert log.read_text().split() == ["constructed", "opened", "closed", "unloaded"]
