"""B200 (sm_100a) paged-KV attention behind the PagedAttentionMetal API.

All computation happens in libpam_cuda.so (CUDA kernels + C ABI, see
include/pam_cuda.h); this package is the ctypes face of it.  The API names are
resolved on first use, so that `pagedattentionmetal_b200.build` can be imported
to compile the library before it exists; using any of them without the library
raises ImportError (there is no fallback).
"""
import importlib

_API = {
    "api_types": ["BlockEvictionPolicy", "KVCacheError", "KVCacheMemoryStats", "LogicalSequence", "Operation",
                  "PagedAttentionDataType", "PagedAttentionDecodeRequest", "PagedAttentionError",
                  "PagedAttentionFusedPrefillRequest",
                  "PagedAttentionPrefillRequest", "PagedAttentionStats", "PagedKVAppendRequest", "PagedLayerSpec",
                  "SchedulerSequence", "SequenceStatus"],
    "engine": ["BatchKVCacheManager", "ContinuousBatchingScheduler", "DeviceBuffer", "KVCacheManager",
               "PagedAttentionEngine", "PagedAttentionInference"],
}
_WHERE = {name: mod for mod, names in _API.items() for name in names}
__all__ = sorted(_WHERE)


def __getattr__(name):
    if name in _WHERE:
        value = getattr(importlib.import_module(f".{_WHERE[name]}", __name__), name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
