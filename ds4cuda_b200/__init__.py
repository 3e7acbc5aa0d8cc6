"""ds4cuda_b200 — B200 (sm_100a) kernels for the fused elementwise /
row-reduction path of the ds4cuda forward pass, behind a C ABI.

    ds4cuda_b200.build   builds libds4b200.so in-tree with nvcc
    ds4cuda_b200._lib    ctypes binding of the C ABI (include/ds4b200*.h)
    ds4cuda_b200.ops     the same calls on torch CUDA tensors
    ds4cuda_b200.path    the T-token prefill path object
    ds4cuda_b200.shard   token-row sharding across ranks (no collective)
"""
__version__ = "0.1"
