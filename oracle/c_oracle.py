"""ctypes binding of the C oracle (oracle/paged_oracle.c).  TEST INFRASTRUCTURE:
only tests, the smoke check and the benchmark's CPU-baseline leg import this.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build() -> str:
    """Compile liboracle.so with the Makefile next to this file."""
    subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)
    return os.path.join(_HERE, "liboracle.so")


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        src = os.path.join(_HERE, "paged_oracle.c")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
            build()
        _LIB = C.CDLL(path)
        _LIB.orc_max_threads.restype = C.c_int
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def max_threads() -> int:
    return int(lib().orc_max_threads())


def decode(q, k_pool, v_pool, tables, lens, kv_heads, block_size, dtype, window=0,
           k_scale=None, v_scale=None, nthreads=0):
    """q [B][H][D] in the query type of ``dtype`` (float32 / float16 bits as
    np.float16 / bfloat16 bits as uint16); pools [blocks][KVH][bs][D] in the
    storage type.  Returns float32 [B][H][D]."""
    B, H, D = q.shape
    q = np.ascontiguousarray(q)
    k_pool, v_pool = np.ascontiguousarray(k_pool), np.ascontiguousarray(v_pool)
    tables = np.ascontiguousarray(tables, dtype=np.int32)
    lens = np.ascontiguousarray(lens, dtype=np.uint32)
    out = np.empty((B, H, D), dtype=np.float32)
    lib().orc_decode(_p(q), _p(k_pool), _p(v_pool), _p(tables), _p(lens), _p(out),
                     C.c_int(B), C.c_int(H), C.c_int(kv_heads), C.c_int(D), C.c_int(block_size),
                     C.c_int(tables.shape[1]), C.c_int(window), C.c_int(dtype),
                     _p(None if k_scale is None else np.ascontiguousarray(k_scale)),
                     _p(None if v_scale is None else np.ascontiguousarray(v_scale)),
                     C.c_int(nthreads))
    return out


def prefill(q, k_pool, v_pool, table, seq_len, kv_heads, block_size, dtype, causal=True,
            window_start=0, q_start=0, k_scale=None, v_scale=None, nthreads=0):
    """q [q_len][H][D] (rows q_start.. of the sequence).  Returns float32."""
    q_len, H, D = q.shape
    assert D <= 1024
    q = np.ascontiguousarray(q)
    table = np.ascontiguousarray(table, dtype=np.int32)
    out = np.empty((q_len, H, D), dtype=np.float32)
    lib().orc_prefill(_p(q), _p(np.ascontiguousarray(k_pool)), _p(np.ascontiguousarray(v_pool)),
                      _p(table), _p(out), C.c_int(seq_len), C.c_int(H), C.c_int(kv_heads),
                      C.c_int(D), C.c_int(block_size), C.c_int(1 if causal else 0),
                      C.c_int(window_start), C.c_int(q_start), C.c_int(q_len), C.c_int(dtype),
                      _p(None if k_scale is None else np.ascontiguousarray(k_scale)),
                      _p(None if v_scale is None else np.ascontiguousarray(v_scale)),
                      C.c_int(nthreads))
    return out


def reshape_and_cache(keys, values, k_pool, v_pool, slots, block_size):
    """In-place scatter of [T][KVH][D] rows into [blocks][KVH][bs][D] pools."""
    T, KVH, D = keys.shape
    slots = np.ascontiguousarray(slots, dtype=np.int64)
    assert k_pool.flags.c_contiguous and v_pool.flags.c_contiguous
    lib().orc_reshape_and_cache(_p(np.ascontiguousarray(keys)), _p(np.ascontiguousarray(values)),
                                _p(k_pool), _p(v_pool), _p(slots), C.c_int(T), C.c_int(KVH),
                                C.c_int(D), C.c_int(block_size), C.c_int(keys.dtype.itemsize))


def reshape_and_cache_fp8(keys_f16, values_f16, k_codes, v_codes, k_scale, v_scale, slots, block_size):
    T, KVH, D = keys_f16.shape
    slots = np.ascontiguousarray(slots, dtype=np.int64)
    nblk = k_codes.shape[0]
    scratch = np.empty(nblk * KVH * 2, dtype=np.float32)
    lib().orc_reshape_and_cache_fp8(_p(np.ascontiguousarray(keys_f16.view(np.uint16))),
                                    _p(np.ascontiguousarray(values_f16.view(np.uint16))),
                                    _p(k_codes), _p(v_codes), _p(k_scale), _p(v_scale), _p(slots),
                                    C.c_int(T), C.c_int(KVH), C.c_int(D), C.c_int(block_size),
                                    C.c_int64(nblk), _p(scratch))


def copy_blocks(k_pool, v_pool, src, dst):
    src = np.ascontiguousarray(src, dtype=np.int32)
    dst = np.ascontiguousarray(dst, dtype=np.int32)
    block_bytes = k_pool[0].nbytes
    lib().orc_copy_blocks(_p(k_pool), _p(v_pool), _p(src), _p(dst), C.c_int(len(src)),
                          C.c_int64(block_bytes))


def quantize_fp8(values_f16, scales_f16):
    v = np.ascontiguousarray(values_f16, dtype=np.float16)
    s = np.ascontiguousarray(np.broadcast_to(np.asarray(scales_f16, dtype=np.float16), v.shape))
    out = np.empty(v.shape, dtype=np.uint8)
    lib().orc_quantize_fp8(_p(v), _p(s), _p(out), C.c_int64(v.size))
    return out


def dequant_fp8(codes, scales_f16):
    c = np.ascontiguousarray(codes, dtype=np.uint8)
    s = np.ascontiguousarray(np.broadcast_to(np.asarray(scales_f16, dtype=np.float16), c.shape))
    out = np.empty(c.shape, dtype=np.float32)
    lib().orc_dequant_fp8(_p(c), _p(s), _p(out), C.c_int64(c.size))
    return out
