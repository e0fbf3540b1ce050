"""Build the oracle's native helpers.  Test infrastructure only.

* ``oracle/_ref/liboracle.so`` from ``oracle/affine_ref.c`` (this repository's own C restatement; always built).
* ``oracle/_ref/code_at.so`` from the reference's packed-bit expression ``code_at`` — the Metal header string in
  kernels/qwen/dense/v1/affine_rows.py:11-24, which compiles as plain C++ (the reference's own test does the same,
  tests/test_affine_rows.py:82-101).  Built only where a reference checkout is present; the source text is read from
  the checkout at build time and written nowhere but ``oracle/_ref/``, which is not committed.
"""

from __future__ import annotations

import ast
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).parent
OUT = HERE / "_ref"
BITS = (2, 3, 4, 5, 6, 8)


def build_port() -> Path:
    OUT.mkdir(exist_ok=True)
    lib = OUT / "liboracle.so"
    src = HERE / "affine_ref.c"
    if lib.exists() and lib.stat().st_mtime >= src.stat().st_mtime:
        return lib
    # no -march=native: the built file travels to hosts with other CPUs
    cmd = ["gcc", "-O3", "-fopenmp", "-shared", "-fPIC", str(src), "-o", str(lib), "-lm"]
    subprocess.run(cmd, check=True, capture_output=True, timeout=120)
    return lib


def build_code_at(reference: str | Path) -> Path | None:
    ref = Path(reference) / "src/tensorfold/kernels/qwen/dense/v1/affine_rows.py"
    compiler = shutil.which("g++") or shutil.which("c++")
    if not ref.exists() or compiler is None:
        return None
    header = None
    for node in ast.parse(ref.read_text()).body:
        if isinstance(node, ast.Assign) and getattr(node.targets[0], "id", "") == "_HEADER":
            header = ast.literal_eval(node.value)
    if header is None:
        return None
    OUT.mkdir(exist_ok=True)
    switches = "".join(f"case {b}: return code_at<{b}>(words + index / 32 * {b}, index % 32);" for b in BITS)
    shim = ("#include <cstdint>\n#include <cstring>\nusing uint = std::uint32_t;\n#define device\n#define thread\n"
            "template <typename T, typename U> T as_type(U u) { T t; std::memcpy(&t, &u, sizeof t); return t; }\n")
    source = OUT / "code_at.cpp"
    source.write_text(shim + header + '\nextern "C" uint decode(const uint* words, int index, int bits) { switch(bits) {'
                      + switches + "default: return 0;} }\n")
    lib = OUT / "code_at.so"
    subprocess.run([compiler, "-std=c++17", "-shared", "-fPIC", "-O1", str(source), "-o", str(lib)], check=True,
                   capture_output=True, timeout=60)
    return lib


def find_reference() -> str:
    """The reference checkout: the directory TENSORFOLD_REFERENCE names, else a ``reference`` directory beside this
    repository; empty when neither exists."""

    named = os.environ.get("TENSORFOLD_REFERENCE", "")
    beside = HERE.resolve().parent.parent / "reference"
    return named or (str(beside) if (beside / "src" / "tensorfold").is_dir() else "")


def build(reference: str | Path | None = None) -> dict:
    reference = reference or find_reference()
    return {"port": build_port(), "code_at": build_code_at(reference)}


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None))
