"""CUDA operators of the sparse decode path (B200 / sm_100a).

Importing a kernel module loads ``librelation_lm_b200.so`` and registers its
operators with ``torch.library``; the import fails loudly when the library has
not been built.  Operators accept CUDA tensors only.
"""
