"""The reference's import names for the quantized-projection hot path, resolved onto ``tensorfold_b200``.

Put this directory's parent (``src``) on ``sys.path`` ahead of the reference's own ``src`` (or copy these small files
over the same-named files of a reference checkout) and the family engines' imports (``tensorfold.cuda.kernels.qmm``,
``tensorfold.cuda.kernels.affine``, ``tensorfold.cuda.experts``, ``tensorfold.cuda.moe``,
``tensorfold.families.qwen3_5.cuda.qmm_fast`` ...) load the B200 implementation: every such module IS the
``tensorfold_b200`` module of the same path."""
