"""Checks of the C ABI that need no GPU: argument validation runs before anything
that touches a device, and the choice of decode kernel only reads the request."""
import ctypes as C

import numpy as np

import pagedattentionmetal_b200 as pam
from pagedattentionmetal_b200 import _cabi
from pagedattentionmetal_b200._cabi import lib

DT = pam.PagedAttentionDataType


def decode_request(q_bytes, out_bytes, dtype, batch=4, heads=8, kv_heads=2, dim=128, bs=16, nb=4, base=1 << 20):
    """A request whose pointers are never dereferenced (validation only)."""
    elem = 4 if dtype == DT.float32 else 1 if dtype == DT.float8 else 2
    pool = nb * bs * kv_heads * dim * elem
    b = lambda addr, n: _cabi.PamBuffer(addr, n)
    return _cabi.PamDecodeRequest(b(base, q_bytes), b(base + (1 << 20), pool), b(base + (2 << 20), pool),
                                  b(base + (3 << 20), batch * nb * 4), b(base + (4 << 20), batch * 4),
                                  b(base + (5 << 20), out_bytes), batch, nb,
                                  _cabi.PamLayerSpec(dim, heads, kv_heads, bs, int(dtype), 0),
                                  b(base + (6 << 20), nb * kv_heads * 2), b(base + (7 << 20), nb * kv_heads * 2))


def test_fp8_decode_refuses_one_byte_per_element_query_and_output():
    # The reference sizes Q and the output by the cache's element width (PagedAttentionTypes.swift:149),
    # one byte for FP8; the kernels read and write float16 there.  A buffer of known length that
    # only holds the one-byte size must be refused before anything is launched.
    ctx = lib.pamc_create_host_context()
    try:
        n = 4 * 8 * 128
        for fn in (lib.pamc_decode, lib.pamc_decode_noalloc):
            rq = decode_request(n, 2 * n, DT.float8)
            assert fn(ctx, C.byref(rq)) == -1
            assert lib.pamc_last_error_code(ctx) == 5
            assert lib.pam_last_error(ctx) == f"Q buffer is too small: expected at least {2 * n} bytes, got {n}.".encode()
            rq = decode_request(2 * n, n, DT.float8)
            assert fn(ctx, C.byref(rq)) == -1
            assert lib.pam_last_error(ctx) == f"output buffer is too small: expected at least {2 * n} bytes, got {n}.".encode()
            # the right sizes pass validation; the host context then has no GPU to run on
            rq = decode_request(2 * n, 2 * n, DT.float8)
            assert fn(ctx, C.byref(rq)) == -1
            assert lib.pamc_last_error_code(ctx) == 1
        # float16: the reference's size is the real one
        rq = decode_request(2 * n - 2, 2 * n, DT.float16)
        assert lib.pamc_decode(ctx, C.byref(rq)) == -1 and lib.pamc_last_error_code(ctx) == 5
    finally:
        lib.pam_destroy_context(ctx)


def test_decode_kernel_choice_follows_shape_type_and_alignment():
    n = 4 * 8 * 128 * 2
    path = lambda rq: lib.pamc_decode_path(C.byref(rq))
    assert path(decode_request(n, n, DT.float16)) == 1
    assert path(decode_request(n, n, DT.bfloat16)) == 1
    assert path(decode_request(n, n, DT.float8)) == 1
    assert path(decode_request(2 * n, 2 * n, DT.float32)) == 0
    assert path(decode_request(n, n, DT.float16, dim=96)) == 0
    assert path(decode_request(n, n, DT.float16, bs=8)) == 0
    assert path(decode_request(n, n, DT.float16, heads=64, kv_heads=2)) == 0        # 32 query heads per KV head
    # pointers the stream kernel's 16-byte copies and word loads cannot take: the general kernel runs
    rq = decode_request(n, n, DT.float16)
    rq.k_pool.ptr += 8
    assert path(rq) == 0
    rq = decode_request(n, n, DT.float16)
    rq.q.ptr += 2
    assert path(rq) == 0
    rq = decode_request(n, n, DT.float8)
    rq.q.ptr += 4
    assert path(rq) == 0
    rq = decode_request(n, n, DT.float16)
    rq.q.ptr += 4
    assert path(rq) == 1
    assert lib.pamc_decode_path(None) == -1


def test_backward_validation_runs_before_the_device_is_needed():
    """pamc_backward checks every buffer of known length against what the kernels touch and
    refuses an FP8 cache, on a context without a GPU (the pointers are never dereferenced)."""
    ctx = lib.pamc_create_host_context()
    try:
        L, H, KVH, D, bs = 40, 8, 2, 64, 16
        nb = (L + bs - 1) // bs
        io, stats, pool = L * H * D * 4, L * H * 4, nb * bs * KVH * D * 4
        base = 1 << 22
        b = lambda i, n: _cabi.PamBuffer(base + (i << 20), n)

        def request(dtype=DT.float32, **short):
            sizes = dict(q=io, k_pool=pool, v_pool=pool, block_table=nb * 4, d_out=io, m=stats, l=stats, d_q=io, d_k_pool=pool,
                         d_v_pool=pool)
            sizes.update(short)
            order = ["q", "k_pool", "v_pool", "block_table", "d_out", "m", "l", "d_q", "d_k_pool", "d_v_pool"]
            return _cabi.PamBackwardRequest(*[b(i, sizes[name]) for i, name in enumerate(order)], L,
                                            _cabi.PamLayerSpec(D, H, KVH, bs, int(dtype), 0))

        for name, text in (("d_q", "dQ"), ("m", "m"), ("d_out", "dO"), ("d_v_pool", "dV pool"), ("block_table", "blockTable")):
            full = dict(q=io, m=stats, d_out=io, d_q=io, d_v_pool=pool, block_table=nb * 4)[name]
            rq = request(**{name: full - 4})
            assert lib.pamc_backward(ctx, C.byref(rq)) == -1
            assert lib.pamc_last_error_code(ctx) == 5
            assert lib.pam_last_error(ctx) == f"{text} buffer is too small: expected at least {full} bytes, got {full - 4}.".encode()
        rq = request(DT.float8)
        assert lib.pamc_backward(ctx, C.byref(rq)) == -1 and lib.pamc_last_error_code(ctx) == 8
        # everything in order: only the missing GPU is left to complain about
        rq = request()
        assert lib.pamc_backward(ctx, C.byref(rq)) == -1 and lib.pamc_last_error_code(ctx) == 1
        assert lib.pamc_backward(ctx, None) == -1
    finally:
        lib.pam_destroy_context(ctx)
