"""CPU restatements of the dflash-mlx target-verify hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory: it is the checker used by ``tests/``, by the smoke test and by the
CPU-baseline leg of ``bench.py``.  The product path is the CUDA library and it
raises when that library is missing.

Each function cites the reference file:line it restates (paths are relative to
the dflash-mlx project root).

Pinning status
--------------
* GatedDeltaNet tape record / tape replay / rollback-cache arithmetic: pinned.
  ``tests/golden/make_golden.py`` imports the reference's own array-op
  functions (``dflash_mlx/kernels.py:131-173, 328-358`` and
  ``dflash_mlx/recurrent_rollback_cache.py:129-171``) over a numpy stand-in for
  ``mlx.core`` and stores their outputs; ``tests/test_oracle_golden.py``
  compares this oracle with those files.
* int4 affine matmul: the arithmetic lives in MLX (``mx.quantized_matmul``,
  mlx>=0.25, benchmarks ran 0.31.1), which is not installable here.  The bit
  layout and dequantisation formula are pinned by the reference's Metal kernel
  text (``dflash_mlx/verify_qmm.py:66-88``); the accumulate order of MLX's CPU
  kernel is not knowable -> parity unpinned beyond the reference's own test
  tolerance (``tests/test_verify_qmm_parity.py:83-98``).
* verify attention: the reference's CPU path is mlx-lm's
  ``scaled_dot_product_attention`` (dependency, absent) -> parity unpinned; the
  visibility rule and 2-pass arithmetic follow ``dflash_mlx/kernels.py:504-637``.
"""
