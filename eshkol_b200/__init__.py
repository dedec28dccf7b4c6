"""B200-native f64 tensor-matmul path for Eshkol.

The product is the shared library ``libeshkol_gpu_b200.so`` (C ABI, see
``include/``).  This package is its Python-side harness: ctypes bindings that
mirror the reference's buffer API, the synthetic input generators, and the
row-sharded multi-GPU driver built on ``torch.distributed``.
"""
from .abi import (  # noqa: F401
    EshkolGPUBuffer,
    GemmOpts,
    TIER_OZAKI2,
    TIER_OZAKI1,
    TIER_OZAKI2_FAST,
    TIER_DGEMM,
    load_library,
    library_path,
)
from .api import (  # noqa: F401
    init,
    matmul,
    matmul_dispatch,
    batch_matmul_dispatch,
    matmul_backward,
    conv2d,
    gemm_device,
    conv2d_device,
    sync_status,
    stream_handle,
    launch_count,
    debug_fetch,
)
