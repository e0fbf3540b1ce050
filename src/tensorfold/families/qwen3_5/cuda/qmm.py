"""``tensorfold.families.qwen3_5.cuda.qmm`` of the reference, served by ``tensorfold_b200.families.qwen3_5.cuda.qmm``."""

import importlib
import sys

sys.modules[__name__] = importlib.import_module("tensorfold_b200.families.qwen3_5.cuda.qmm")
