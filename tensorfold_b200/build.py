"""Builds ``libtensorfold_b200.so`` in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m tensorfold_b200.build [--force]

One object per translation unit, compiled in parallel; the matmul template is instantiated once per bit width
(``qmm_inst.cu`` and ``qmm_stream_inst.cu`` with ``-DTF_BITS=b``).
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "libtensorfold_b200.so"
BITS = (2, 3, 4, 5, 6, 8)
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "--threads", "2"]


def _units() -> list[tuple[Path, Path, list[str]]]:
    units = [(CSRC / "qmm_inst.cu", OBJ / f"qmm_b{b}.o", [f"-DTF_BITS={b}"]) for b in BITS]
    units += [(CSRC / "qmm_stream_inst.cu", OBJ / f"qmm_stream_b{b}.o", [f"-DTF_BITS={b}"]) for b in BITS]
    for src in sorted(CSRC.glob("*.cu")):
        if src.name not in ("qmm_inst.cu", "qmm_stream_inst.cu"):
            units.append((src, OBJ / (src.stem + ".o"), []))
    return units


def _newest_header() -> float:
    heads = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "tensorfold_b200.h"]
    return max(h.stat().st_mtime for h in heads)


def _compile(unit) -> str:
    src, obj, defs = unit
    cmd = ["nvcc", *NVCC_FLAGS, *defs, "-c", str(src), "-o", str(obj)]
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode:
        raise RuntimeError(f"nvcc failed for {src.name} {defs}:\n{done.stdout}\n{done.stderr}")
    return obj.name


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    heads = _newest_header()
    stale = [u for u in _units()
             if force or not u[1].exists() or u[1].stat().st_mtime < max(u[0].stat().st_mtime, heads)]
    if stale:
        with ThreadPoolExecutor(max_workers=min(len(stale), os.cpu_count() or 4)) as pool:
            for name in pool.map(_compile, stale):
                if verbose:
                    print("compiled", name)
    objs = [str(u[1]) for u in _units()]
    if stale or not LIB.exists():
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB), *objs]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode:
            raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
