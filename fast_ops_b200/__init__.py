"""fast_ops_b200: B200 (sm_100a) implementation of fast-ops' two hot paths.

    from fast_ops_b200.flash_attention import multi_head_attention
    from fast_ops_b200.lion import Lion

Both call hand-written CUDA kernels through a C-ABI library (include/fast_ops_b200.h).
"""
__version__ = "0.1.0"
