"""CPU oracle for the affine packed-row quantized-projection path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this directory: only the test suite,
``__graft_entry__.smoke`` and the CPU-baseline legs of ``bench.py`` do, and there only as the checker or as the
timed host baseline.  The product path is the CUDA library and fails loudly when it is missing.

Parity status
-------------
* Pinned against the reference's own Python, imported from a checkout of the reference when the golden vectors
  were generated (``tests/golden/make_golden.py``): ``dequantize`` (families/qwen3_5/cuda/qmm.py:132-149),
  ``split_k`` / ``bucket`` (cuda/kernels/qmm.py:105-119), ``packed_shape`` / ``input_slice``
  (cuda/kernels/affine.py:9-27), ``max_items`` (cuda/experts.py:95-98), the partition map ``output_rows``
  (families/qwen3_5/cuda/distributed.py:27-42), ``sum_rank_partials`` (:259-264), and the expert plan against the
  ``want_plan`` the reference's own test expects (tests/cuda/test_experts.py:107-115).
* The glue (``glue.py``) follows the plain-torch formulas the reference's glue test checks its kernels against
  (tests/cuda/test_qwen27_glue.py:24-44); the Triton kernels themselves need a GPU and were not run: unpinned.
* Pinned against the reference's Metal header expression ``code_at`` compiled as C++ (``oracle/build_ref.py`` builds
  ``oracle/_ref/code_at.so`` from kernels/qwen/dense/v1/affine_rows.py:11-24 where a reference checkout is present).
* Parity unpinned against MLX's own ``quantized_matmul`` kernel output: MLX (pinned by the reference at
  ``mlx>=0.32.2,<0.32.4``, pyproject.toml:27) is a third-party dependency that is neither vendored in the reference
  nor installable here.  Its published definition, ``w = scale * q + bias`` then ``x @ w.T``, is what is restated.
"""
