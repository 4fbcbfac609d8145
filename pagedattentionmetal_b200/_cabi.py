"""ctypes binding of libpam_cuda.so (include/pam_cuda.h).

There is no fallback: if the library has not been built, importing this module
raises, and every compute call needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# PAM_CUDA_LIBRARY selects another build of the same library (an instrumented one, say).
LIB_PATH = os.environ.get("PAM_CUDA_LIBRARY") or os.path.join(_HERE, "libpam_cuda.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m pagedattentionmetal_b200.build` "
        "(needs nvcc). There is no CPU fallback."
    )

lib = C.CDLL(LIB_PATH)

c_void_p, c_int32, c_int64, c_size_t = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t
UNKNOWN_BYTES = (1 << (8 * C.sizeof(C.c_size_t))) - 1


class PamBuffer(C.Structure):
    _fields_ = [("ptr", c_void_p), ("bytes", c_size_t)]


class PamLayerSpec(C.Structure):
    _fields_ = [("head_dim", c_int32), ("num_heads", c_int32), ("num_kv_heads", c_int32),
                ("block_size", c_int32), ("data_type", c_int32), ("window_size", c_int32)]


class PamStats(C.Structure):
    _fields_ = [("operation", c_int32), ("batch_size", c_int32), ("sequence_length", c_int32),
                ("num_blocks", c_int32), ("temporary_bytes", c_int64), ("used_split_pass", c_int32),
                ("elapsed_ms", C.c_double)]


class PamMemoryStats(C.Structure):
    _fields_ = [("total_blocks", c_int64), ("used_blocks", c_int64), ("free_blocks", c_int64),
                ("active_sequences", c_int64), ("total_memory_bytes", c_int64),
                ("used_memory_bytes", c_int64), ("partially_filled_blocks", c_int64),
                ("fragmentation_ratio", C.c_float), ("prefix_cache_hits", c_int64),
                ("prefix_cache_entries", c_int64), ("shared_blocks", c_int64),
                ("eviction_policy", c_int32)]


class PamAppendRequest(C.Structure):
    _fields_ = [("keys", PamBuffer), ("values", PamBuffer), ("k_pool", PamBuffer), ("v_pool", PamBuffer),
                ("block_table", PamBuffer), ("token_offset", c_int32), ("num_new_tokens", c_int32),
                ("layer", PamLayerSpec), ("k_scale", PamBuffer), ("v_scale", PamBuffer)]


class PamDecodeRequest(C.Structure):
    _fields_ = [("q", PamBuffer), ("k_pool", PamBuffer), ("v_pool", PamBuffer), ("block_tables", PamBuffer),
                ("seq_lengths", PamBuffer), ("output", PamBuffer), ("batch_size", c_int32),
                ("max_num_blocks", c_int32), ("layer", PamLayerSpec), ("k_scale", PamBuffer),
                ("v_scale", PamBuffer)]


class PamPrefillRequest(C.Structure):
    _fields_ = [("q", PamBuffer), ("k_pool", PamBuffer), ("v_pool", PamBuffer), ("block_table", PamBuffer),
                ("output", PamBuffer), ("seq_len", c_int32), ("layer", PamLayerSpec), ("causal", c_int32),
                ("k_scale", PamBuffer), ("v_scale", PamBuffer), ("q_start", c_int32), ("q_len", c_int32)]


class PamBatchPrefillRequest(C.Structure):
    _fields_ = [("q", PamBuffer), ("k_pool", PamBuffer), ("v_pool", PamBuffer), ("block_tables", PamBuffer),
                ("output", PamBuffer), ("seq_lens", C.POINTER(c_int32)), ("q_starts", C.POINTER(c_int32)),
                ("q_lens", C.POINTER(c_int32)), ("num_sequences", c_int32), ("max_num_blocks", c_int32),
                ("layer", PamLayerSpec), ("causal", c_int32), ("k_scale", PamBuffer), ("v_scale", PamBuffer)]


class PamFusedPrefillRequest(C.Structure):
    _fields_ = [("q", PamBuffer), ("raw_k", PamBuffer), ("raw_v", PamBuffer), ("block_table", PamBuffer),
                ("k_pool", PamBuffer), ("v_pool", PamBuffer), ("output", PamBuffer), ("seq_len", c_int32),
                ("layer", PamLayerSpec), ("causal", c_int32), ("k_scale", PamBuffer), ("v_scale", PamBuffer)]


class PamBackwardRequest(C.Structure):
    _fields_ = [("q", PamBuffer), ("k_pool", PamBuffer), ("v_pool", PamBuffer), ("block_table", PamBuffer),
                ("d_out", PamBuffer), ("m", PamBuffer), ("l", PamBuffer), ("d_q", PamBuffer),
                ("d_k_pool", PamBuffer), ("d_v_pool", PamBuffer), ("seq_len", c_int32), ("layer", PamLayerSpec)]


class PamSchedSequence(C.Structure):
    _fields_ = [("id", c_int64), ("status", c_int32), ("num_generated_tokens", c_int32),
                ("max_new_tokens", c_int32), ("prompt_length", c_int32), ("arrival_order", c_int32)]


AVAILABLE_FN = C.CFUNCTYPE(c_int32, c_void_p)
TOKEN_FN = C.CFUNCTYPE(None, c_void_p, c_int64, c_int32)

# name -> (restype, argtypes); every symbol include/pam_cuda.h declares.
SIGNATURES = {
    # reference C ABI
    "pam_create_context": (c_void_p, []),
    "pam_destroy_context": (None, [c_void_p]),
    "pam_last_error": (C.c_char_p, [c_void_p]),
    "pam_create_cache": (c_void_p, [c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32]),
    "pam_destroy_cache": (None, [c_void_p]),
    "pam_reserve_sequence": (c_int32, [c_void_p, c_void_p, c_int64]),
    "pam_append_tokens": (c_int32, [c_void_p, c_void_p, c_int64, c_int32]),
    "pam_free_sequence": (None, [c_void_p, c_int64]),
    "pam_available_blocks": (c_int32, [c_void_p]),
    "pam_sequence_length": (c_int32, [c_void_p, c_void_p, c_int64]),
    "pam_append_kv": (c_int32, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int32, c_int32, c_int32]),
    "pam_prefill": (c_int32, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int32, c_int32, C.c_bool]),
    "pam_decode": (c_int32, [c_void_p, c_void_p, C.POINTER(c_int64), c_int32, c_void_p, c_void_p, c_int32]),
    # context / engine
    "pamc_device_count": (c_int32, []),
    "pamc_create_context_on": (c_void_p, [c_int32]),
    "pamc_create_host_context": (c_void_p, []),
    "pamc_last_error_code": (c_int32, [c_void_p]),
    "pamc_set_stream": (c_int32, [c_void_p, c_void_p]),
    "pamc_set_async": (c_int32, [c_void_p, c_int32]),
    "pamc_synchronize": (c_int32, [c_void_p]),
    "pamc_set_max_retries": (c_int32, [c_void_p, c_int32]),
    "pamc_set_graceful_degradation": (c_int32, [c_void_p, c_int32]),
    "pamc_set_split_threshold": (c_int32, [c_void_p, c_int32]),
    "pamc_set_default_window": (c_int32, [c_void_p, c_int32]),
    "pamc_set_default_chunk": (c_int32, [c_void_p, c_int32]),
    "pamc_set_prefill_tensor_path": (c_int32, [c_void_p, c_int32]),
    "pamc_set_prefill_exact_weights": (c_int32, [c_void_p, c_int32]),
    "pamc_inject_launch_failures": (c_int32, [c_void_p, c_int32]),
    "pamc_kernel_launches": (c_int64, [c_void_p]),
    "pamc_last_stats": (c_int32, [c_void_p, C.POINTER(PamStats)]),
    "pamc_recommended_max_blocks": (c_int64, [c_void_p, c_int32, c_int32, c_int32, c_int32, C.c_float, c_int32]),
    "pamc_buffer_alloc": (c_void_p, [c_void_p, c_size_t]),
    "pamc_buffer_free": (None, [c_void_p, c_void_p]),
    "pamc_memcpy": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t, c_int32]),
    # cache
    "pamc_cache_create_bookkeeping": (c_void_p, [c_int32, c_int32]),
    "pamc_cache_append_tokens": (c_int32, [c_void_p, c_void_p, c_int64, c_int32, C.POINTER(C.c_uint64), c_int32]),
    "pamc_cache_ensure_exclusive": (c_int32, [c_void_p, c_void_p, c_int64, c_int32]),
    "pamc_cache_register_block_hash": (None, [c_void_p, C.c_uint64, c_int32]),
    "pamc_cache_block_table": (c_int32, [c_void_p, c_void_p, c_int64, C.POINTER(c_int32), c_int32]),
    "pamc_cache_num_blocks": (c_int32, [c_void_p, c_void_p, c_int64]),
    "pamc_cache_active_sequences": (c_int32, [c_void_p]),
    "pamc_cache_set_eviction_policy": (c_int32, [c_void_p, c_int32]),
    "pamc_cache_memory_stats": (c_int32, [c_void_p, C.POINTER(PamMemoryStats)]),
    "pamc_cache_pools": (c_int32, [c_void_p, C.POINTER(c_void_p), C.POINTER(c_void_p), C.POINTER(c_void_p),
                                   C.POINTER(c_void_p), C.POINTER(c_size_t), C.POINTER(c_size_t)]),
    "pamc_cache_drain_cow_log": (c_int32, [c_void_p, C.POINTER(c_int32), c_int32]),
    "pamc_cache_batch_tables": (c_int32, [c_void_p, c_void_p, C.POINTER(c_int64), c_int32, c_int32, c_void_p, c_void_p]),
    "pamc_cache_slot_mapping": (c_int32, [c_void_p, c_void_p, c_int64, c_int32, c_int32, C.POINTER(c_int64)]),
    # operations
    "pamc_append_to_cache": (c_int32, [c_void_p, C.POINTER(PamAppendRequest)]),
    "pamc_reshape_and_cache": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32]),
    "pamc_copy_blocks": (c_int32, [c_void_p, c_void_p, C.POINTER(c_int32), C.POINTER(c_int32), c_int32]),
    "pamc_decode": (c_int32, [c_void_p, C.POINTER(PamDecodeRequest)]),
    "pamc_decode_noalloc": (c_int32, [c_void_p, C.POINTER(PamDecodeRequest)]),
    "pamc_prefill": (c_int32, [c_void_p, C.POINTER(PamPrefillRequest), c_int32]),
    "pamc_prefill_batch": (c_int32, [c_void_p, C.POINTER(PamBatchPrefillRequest)]),
    "pamc_decode_layers": (c_int32, [c_void_p, C.POINTER(PamDecodeRequest), c_int32]),
    "pamc_prefill_layers": (c_int32, [c_void_p, C.POINTER(PamPrefillRequest), c_int32]),
    "pamc_append_layers": (c_int32, [c_void_p, C.POINTER(PamAppendRequest), c_int32, C.POINTER(c_void_p)]),
    "pamc_fused_prefill": (c_int32, [c_void_p, C.POINTER(PamFusedPrefillRequest), c_void_p]),
    "pamc_backward": (c_int32, [c_void_p, C.POINTER(PamBackwardRequest)]),
    # scheduler
    "pamc_sched_create": (c_void_p, [c_int32, c_int32]),
    "pamc_sched_destroy": (None, [c_void_p]),
    "pamc_sched_add_request": (c_int64, [c_void_p, c_int32, c_int32]),
    "pamc_sched_complete": (None, [c_void_p, c_int64]),
    "pamc_sched_step": (c_int32, [c_void_p, C.POINTER(c_int64), c_int32]),
    "pamc_sched_mark_prefilled": (None, [c_void_p, c_int64]),
    "pamc_sched_mark_decoded": (None, [c_void_p, c_int64]),
    "pamc_sched_preempt": (None, [c_void_p, c_int64]),
    "pamc_sched_handle_memory_pressure": (c_int32, [c_void_p, c_int32, AVAILABLE_FN, c_void_p, C.POINTER(c_int64), c_int32]),
    "pamc_sched_count": (c_int32, [c_void_p, c_int32]),
    "pamc_sched_total": (c_int32, [c_void_p]),
    # inference orchestration
    "pamc_infer_create": (c_void_p, [c_void_p, c_int32, c_int32, C.POINTER(PamLayerSpec), c_int32, c_int32, c_int32]),
    "pamc_infer_destroy": (None, [c_void_p]),
    "pamc_infer_cache": (c_void_p, [c_void_p]),
    "pamc_infer_scheduler": (c_void_p, [c_void_p]),
    "pamc_infer_add_request": (c_int64, [c_void_p, c_int32, c_int32]),
    "pamc_infer_complete_sequence": (None, [c_void_p, c_int64]),
    "pamc_infer_step": (c_int32, [c_void_p, C.POINTER(c_int64), c_int32]),
    "pamc_infer_run_all": (c_int32, [c_void_p]),
    "pamc_infer_total_tokens": (c_int64, [c_void_p]),
    "pamc_infer_step_count": (c_int32, [c_void_p]),
    "pamc_infer_set_token_callback": (None, [c_void_p, TOKEN_FN, c_void_p]),
    "pamc_infer_set_incremental_preemption": (None, [c_void_p, c_int32]),
    "pamc_sched_get": (c_int32, [c_void_p, c_int64, C.POINTER(PamSchedSequence)]),
    "pamc_infer_set_batched_prefill": (None, [c_void_p, c_int32, c_int32]),
    "pamc_infer_prefill_launch_sets": (c_int64, [c_void_p]),
    # additions without a reference counterpart
    "pamc_set_wait_limit": (c_int32, [c_void_p, c_int64]),
    "pamc_test_starve_prefill": (c_int32, [c_void_p, c_int32]),
    "pamc_cache_set_hygiene": (c_int32, [c_void_p, c_int32]),
    "pamc_block_hashes": (c_int32, [C.POINTER(c_int32), c_int32, c_int32, C.c_uint64, C.POINTER(C.c_uint64), c_int32]),
    "pamc_decode_path": (c_int32, [C.POINTER(PamDecodeRequest)]),
    "pamc_comm_unique_id": (c_int32, [c_void_p]),
    "pamc_comm_create": (c_void_p, [c_void_p, c_void_p, c_int32, c_int32]),
    "pamc_comm_destroy": (None, [c_void_p]),
    "pamc_allgather_heads": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)          # AttributeError here means the library and the header disagree
    _fn.restype = _res
    _fn.argtypes = _args


def buffer(ptr, nbytes=None) -> PamBuffer:
    """PamBuffer from an int/ctypes pointer, a numpy array (host memory) or any
    object with ``data_ptr()`` and ``nbytes``/``numel()`` (a torch tensor)."""
    if ptr is None:
        return PamBuffer(None, 0)
    if hasattr(ptr, "ctypes") and hasattr(ptr, "nbytes"):          # numpy
        return PamBuffer(ptr.ctypes.data, ptr.nbytes if nbytes is None else nbytes)
    if hasattr(ptr, "data_ptr") and hasattr(ptr, "nbytes") and not hasattr(ptr, "numel"):
        return PamBuffer(ptr.data_ptr(), ptr.nbytes if nbytes is None else nbytes)
    if hasattr(ptr, "data_ptr"):                                   # torch
        n = ptr.numel() * ptr.element_size()
        return PamBuffer(ptr.data_ptr(), n if nbytes is None else nbytes)
    if isinstance(ptr, PamBuffer):
        return ptr
    return PamBuffer(int(ptr), UNKNOWN_BYTES if nbytes is None else nbytes)


def address(obj) -> int:
    """Raw address of a numpy array, torch tensor or integer pointer."""
    if hasattr(obj, "ctypes") and hasattr(obj, "nbytes"):
        return obj.ctypes.data
    if hasattr(obj, "data_ptr"):
        return obj.data_ptr()
    return int(obj)
