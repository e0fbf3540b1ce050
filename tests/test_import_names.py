"""The reference's module names resolve onto this library: a family engine's ``from tensorfold.cuda.kernels import qmm``
gets the B200 implementation once ``src`` is on the path (CPU: names and host functions only)."""

import importlib
import sys
from pathlib import Path

import pytest

SRC = str(Path(__file__).resolve().parents[1] / "src")

NAMES = ["tensorfold.cuda.kernels.qmm", "tensorfold.cuda.kernels.affine", "tensorfold.cuda.experts", "tensorfold.cuda.moe",
         "tensorfold.families.qwen3_5.cuda.qmm", "tensorfold.families.qwen3_5.cuda.qmm_fast",
         "tensorfold.families.qwen3_5.cuda.distributed", "tensorfold.families.qwen3_5.cuda.weights",
         "tensorfold.families.qwen3_5.cuda.glue", "tensorfold.families.qwen3_5.cuda.decode_tp"]


@pytest.fixture()
def reference_names():
    saved = {k: v for k, v in sys.modules.items() if k == "tensorfold" or k.startswith("tensorfold.")}
    for k in saved:
        del sys.modules[k]
    sys.path.insert(0, SRC)
    yield
    sys.path.remove(SRC)
    for k in [k for k in sys.modules if k == "tensorfold" or k.startswith("tensorfold.")]:
        del sys.modules[k]
    sys.modules.update(saved)


def test_reference_import_names_load_this_library(reference_names):
    for name in NAMES:
        module = importlib.import_module(name)
        assert module is importlib.import_module(name.replace("tensorfold.", "tensorfold_b200.", 1)), name
    from tensorfold.cuda.kernels import qmm                      # the line a family engine has (cuda/kernels/qmm.py users)

    assert qmm.split_k(6144, 5120, 64) == 2 and qmm.bucket(12) == 16      # the reference's own values (golden file)
    from tensorfold.cuda import experts, moe

    assert experts.TILE == 16 and hasattr(moe, "run") and hasattr(moe, "Routed")
    from tensorfold.families.qwen3_5.cuda import qmm_fast

    assert all(hasattr(qmm_fast, f) for f in ("tile", "untile", "rows", "matmul_rows", "matmul", "matmul_partial", "stack",
                                                "stack_small", "prepare"))
