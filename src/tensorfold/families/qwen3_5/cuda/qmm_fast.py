"""``tensorfold.families.qwen3_5.cuda.qmm_fast`` of the reference, served by ``tensorfold_b200.families.qwen3_5.cuda.qmm_fast``."""

import importlib
import sys

sys.modules[__name__] = importlib.import_module("tensorfold_b200.families.qwen3_5.cuda.qmm_fast")
