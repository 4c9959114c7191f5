"""moe_b200: the MoE-layer hot path (router, permutation, expert GEMMs, combine) for B200.

``tilelang_moe_b200.kernels`` mirrors the reference's ``kernels`` API for this path;
``tilelang_moe_b200.ops`` is the tensor-level front end of the C ABI declared in
``include/moe_b200.h``; the CUDA sources live in ``csrc/`` and are built in-tree by
``python -m tilelang_moe_b200.build``.
"""
__version__ = "0.1.0"
