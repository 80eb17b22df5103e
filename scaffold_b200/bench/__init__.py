"""Kernel benchmark harness: paired, interleaved timing with confidence intervals (``harness``), the
operations it can time (``cases``) and the tensor-core ceiling probe (``gemm_probe``)."""
