"""B200-native flat k-NN search backend (drop-in for faiss_metal::MetalIndexFlat).

The product is ``lib/libb200flat.so`` (hand-written sm_100a CUDA kernels, the
C-ABI of ``include/b200_flat.h`` and the C++ plugin classes).  This package is a
thin ctypes mirror of the plugin surface for Python callers, plus the
one-process-per-GPU row-sharded index built on ``torch.distributed``.
There is no CPU fallback: constructing resources without an sm_100 device fails.
"""
from .abi import (  # noqa: F401
    METRIC_INNER_PRODUCT,
    METRIC_L2,
    PATH_AUTO,
    PATH_SCAN,
    PATH_TENSOR,
    STORAGE_BF16,
    STORAGE_F16,
    STORAGE_F32,
    B200Error,
    lib,
    lib_path,
    status_string,
)
from .index import B200IndexFlat, SearchToken, StandardB200Resources, device_caps  # noqa: F401
from .sharded import MultiGpuIndexFlat, ShardedIndexFlat, shard_range  # noqa: F401
from . import abi  # noqa: F401
