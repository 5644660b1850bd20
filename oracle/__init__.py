"""CPU restatements of the reference's algorithms for the gated-delta-rule path.

TEST INFRASTRUCTURE: only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of
``bench.py`` may import this package, and only as the checker or the timed CPU baseline.  The product
(``miles_ext_kernels_b200``) never imports it and fails loudly when its CUDA library is missing.
"""
