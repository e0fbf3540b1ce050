"""The tiled weight layout, checked on the host: the header the kernels include is compiled with g++ and every format's
lane words, A-fragment registers and inverse maps are verified against each other."""

import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def test_layout_header_is_self_consistent(tmp_path):
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        pytest.skip("needs a C++ compiler")
    exe = tmp_path / "layout_check"
    subprocess.run([cxx, "-std=c++17", "-O1", str(ROOT / "tests" / "layout_check.cpp"), "-o", str(exe)], check=True,
                   capture_output=True, timeout=120)
    done = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert done.returncode == 0 and done.stdout.strip().endswith("OK"), done.stdout
