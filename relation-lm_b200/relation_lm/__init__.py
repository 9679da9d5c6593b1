"""Relation LM routed selection-and-reduction path, B200 (sm_100a) implementation.

The module layout mirrors the reference project's ``relation_lm`` package for
the parts that sit on the sparse decode path (``kernels`` and ``inference``),
so code written against ``relation_lm.kernels.*`` imports unchanged.  The
operators are hand-written CUDA kernels in ``librelation_lm_b200.so`` reached
through a C ABI; there is no Triton and no CPU implementation.
"""

__version__ = "0.1.0"
