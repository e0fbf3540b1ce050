"""``tensorfold.cuda.checkpoint`` of the reference, served by ``tensorfold_b200.cuda.checkpoint``."""

import importlib
import sys

sys.modules[__name__] = importlib.import_module("tensorfold_b200.cuda.checkpoint")
