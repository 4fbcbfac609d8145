"""B200 (sm_100a) paged-KV attention behind the PagedAttentionMetal API.

All computation happens in libpam_cuda.so (CUDA kernels + C ABI, see
include/pam_cuda.h); this package is the ctypes face of it and fails to import
when the library has not been built.
"""
from .api_types import (BlockEvictionPolicy, KVCacheError, KVCacheMemoryStats, LogicalSequence, Operation,
                        PagedAttentionDataType, PagedAttentionDecodeRequest, PagedAttentionError,
                        PagedAttentionPrefillRequest, PagedAttentionStats, PagedKVAppendRequest,
                        PagedLayerSpec, SchedulerSequence, SequenceStatus)
from .engine import (BatchKVCacheManager, ContinuousBatchingScheduler, DeviceBuffer, KVCacheManager,
                     PagedAttentionEngine)

__all__ = [
    "BatchKVCacheManager", "BlockEvictionPolicy", "ContinuousBatchingScheduler", "DeviceBuffer",
    "KVCacheError", "KVCacheManager", "KVCacheMemoryStats", "LogicalSequence", "Operation",
    "PagedAttentionDataType", "PagedAttentionDecodeRequest", "PagedAttentionEngine",
    "PagedAttentionError", "PagedAttentionPrefillRequest", "PagedAttentionStats",
    "PagedKVAppendRequest", "PagedLayerSpec", "SchedulerSequence", "SequenceStatus",
]
