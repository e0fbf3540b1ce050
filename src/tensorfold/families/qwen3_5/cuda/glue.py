"""``tensorfold.families.qwen3_5.cuda.glue`` of the reference, served by ``tensorfold_b200.families.qwen3_5.cuda.glue``."""

import importlib
import sys

sys.modules[__name__] = importlib.import_module("tensorfold_b200.families.qwen3_5.cuda.glue")
