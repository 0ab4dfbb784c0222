"""B200-native drop-in for the top-k indexer op of ErkeXia/flash-float-jit-kernels.

Only the hot path is provided: ``jit_kernel.topk_indexer.fast_topk_v3`` (reference:
jit_kernel/topk_indexer.py:42-75), backed by hand-written sm_100a CUDA behind a C ABI.
"""
