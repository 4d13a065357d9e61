"""CPU oracle for the GEMM / attention hot path.

TEST INFRASTRUCTURE ONLY.  Nothing here is part of the product: the product is
the CUDA library behind ``include/frisk_b200.h``.  Only the test-suite, the
smoke check and the CPU-baseline legs of the benchmark may import this
package, and only as the checker.

Pinning status
--------------
* attention: PINNED.  ``attention_oracle`` restates
  ``benchmark/layout/execution/tail_attention_reference.py`` (strict fp32 and
  fp64 modes) and ``run_execution.py:59-64`` (single 64x16 tile); it is checked
  against golden vectors produced by running those reference functions
  (``tests/golden/make_golden.py``).
* GEMM: PARITY UNPINNED.  The reference holds no executed GEMM and no GEMM
  golden vector; ``gemm_oracle`` restates the contract of
  ``lib/Dialect/Frisk/IR/FriskOps.cpp:406-426`` and
  ``lib/Dialect/Frisk/IR/LegacyImportSemantics.cpp:11-46``.
"""
