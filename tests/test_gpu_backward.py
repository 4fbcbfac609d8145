"""Gradients of paged attention (PagedAttentionEngine.backward) on the GPU against the oracle:
dQ written, dK / dV added to what the gradient pools hold, every storage type of the
reference's two pipelines plus bfloat16, windows, ragged tiles, host and device buffers."""
import numpy as np
import pytest

import pagedattentionmetal_b200 as pam
from gpu_helpers import DT, from_io, io_numpy_dtype, to_storage
from oracle import paged_oracle as po

pytestmark = pytest.mark.gpu


def _close(out, ref, dtype):
    """max-abs <= 2e-3 on the value before the rounding to the storage type, which adds up to
    one unit in the last place of the reference value for the 16-bit types."""
    out, ref = np.asarray(out, np.float64), np.asarray(ref, np.float64)
    bits = {DT.float32: 0, DT.float16: 10, DT.bfloat16: 7}[dtype]
    with np.errstate(divide="ignore"):
        ulp = np.where(ref != 0, 2.0 ** (np.floor(np.log2(np.abs(ref))) - bits), 0.0) if bits else 0.0
    err = np.abs(out - ref)
    assert (err <= 2e-3 + ulp).all(), f"max abs error {err.max()}"


class BackwardCase:
    def __init__(self, seed, seq_len, heads, kv_heads, head_dim, block_size, dtype, window=0, spare=3):
        rng = np.random.default_rng(seed)
        self.L, self.H, self.KVH, self.D, self.bs, self.dtype, self.window = seq_len, heads, kv_heads, head_dim, block_size, dtype, window
        nb = (seq_len + block_size - 1) // block_size
        self.table = rng.permutation(nb + spare)[:nb].astype(np.int32)
        shape = (nb + spare, kv_heads, block_size, head_dim)
        rnd = lambda *s: rng.standard_normal(s, dtype=np.float32)
        self.k_pool, self.v_pool = to_storage(rnd(*shape), dtype), to_storage(rnd(*shape), dtype)
        self.q = to_storage(rnd(seq_len, heads, head_dim), dtype)
        self.d_out = to_storage(0.5 * rnd(seq_len, heads, head_dim), dtype)
        # what the gradient pools hold before the call
        self.dk0, self.dv0 = to_storage(0.25 * rnd(*shape), dtype), to_storage(0.25 * rnd(*shape), dtype)
        self.ws = max(0, seq_len - window) if window > 0 else 0
        f = lambda a: from_io(a, dtype)
        self.m, self.l = po.attention_stats(f(self.q), f(self.k_pool), self.table, seq_len, kv_heads, block_size, self.ws)
        dq, dk, dv = po.paged_backward(f(self.q), f(self.k_pool), f(self.v_pool), self.table, f(self.d_out), self.m, self.l,
                                       seq_len, kv_heads, block_size, self.ws)
        self.ref_dq, self.ref_dk, self.ref_dv = dq, f(self.dk0).astype(np.float64) + dk, f(self.dv0).astype(np.float64) + dv

    def run(self, engine, host_io=False):
        kp, vp = engine.makeBufferFrom(self.k_pool), engine.makeBufferFrom(self.v_pool)
        dkp, dvp = engine.makeBufferFrom(self.dk0), engine.makeBufferFrom(self.dv0)
        dq_host = np.zeros(self.q.shape, dtype=io_numpy_dtype(self.dtype))
        if host_io:
            args = (self.q, kp, vp, self.table, self.d_out, self.m, self.l, dq_host, dkp, dvp)
        else:
            dq_dev = engine.makeBuffer(dq_host.nbytes)
            args = (engine.makeBufferFrom(self.q), kp, vp, engine.makeBufferFrom(self.table), engine.makeBufferFrom(self.d_out),
                    engine.makeBufferFrom(self.m), engine.makeBufferFrom(self.l), dq_dev, dkp, dvp)
        engine.backward(*args, self.L, self.D, self.H, self.KVH, self.bs, self.dtype, self.window)
        assert engine.lastStats.operation == pam.Operation.backward
        if not host_io:
            dq_host = dq_dev.download(dq_host.dtype, dq_host.shape)
        io = io_numpy_dtype(self.dtype)
        return (from_io(dq_host, self.dtype), from_io(dkp.download(io, self.k_pool.shape), self.dtype),
                from_io(dvp.download(io, self.v_pool.shape), self.dtype))

    def check(self, engine, host_io=False):
        dq, dk, dv = self.run(engine, host_io)
        _close(dq, self.ref_dq, self.dtype)
        _close(dk, self.ref_dk, self.dtype)
        _close(dv, self.ref_dv, self.dtype)


@pytest.mark.parametrize("dtype", [DT.float32, DT.float16, DT.bfloat16])
@pytest.mark.parametrize("window", [0, 70])
def test_backward_matches_oracle(engine, dtype, window):
    BackwardCase(71, 200, 8, 2, 128, 16, dtype, window).check(engine)


@pytest.mark.parametrize("seq_len,heads,kv_heads,head_dim,block_size", [
    (1, 2, 2, 16, 8), (64, 4, 4, 64, 16), (65, 4, 1, 64, 16), (130, 6, 2, 96, 8), (40, 4, 2, 16, 8),
    (100, 4, 2, 256, 16), (33, 2, 1, 200, 16), (257, 16, 2, 128, 32),
])
def test_backward_shapes(engine, seq_len, heads, kv_heads, head_dim, block_size):
    BackwardCase(72, seq_len, heads, kv_heads, head_dim, block_size, DT.float32).check(engine)
    BackwardCase(73, seq_len, heads, kv_heads, head_dim, block_size, DT.float16, window=max(1, seq_len // 3)).check(engine)


def test_backward_host_buffers_and_errors(engine):
    case = BackwardCase(74, 90, 4, 2, 64, 16, DT.float32)
    case.check(engine, host_io=True)
    # a second call adds to the pools again: twice the contributions
    kp, vp = engine.makeBufferFrom(case.k_pool), engine.makeBufferFrom(case.v_pool)
    dkp, dvp = engine.makeBufferFrom(np.zeros_like(case.dk0)), engine.makeBufferFrom(np.zeros_like(case.dv0))
    dq = np.zeros_like(case.q)
    for _ in range(2):
        engine.backward(case.q, kp, vp, case.table, case.d_out, case.m, case.l, dq, dkp, dvp, case.L, case.D, case.H, case.KVH,
                        case.bs, DT.float32, 0)
    once = case.ref_dk - case.dk0.astype(np.float64)
    _close(dkp.download(np.float32, case.k_pool.shape), 2 * once, DT.float32)
    _close(dq, case.ref_dq, DT.float32)
    graceful = engine.enableGracefulDegradation
    engine.enableGracefulDegradation = False
    try:
        with pytest.raises(pam.PagedAttentionError) as e:
            engine.backward(case.q, kp, vp, case.table, case.d_out, case.m, case.l, dq, dkp, dvp, case.L, case.D, case.H, case.KVH,
                            case.bs, DT.float8, 0)
        assert e.value.case == "unsupported"
        with pytest.raises(pam.PagedAttentionError) as e:          # the gradient pools must be device memory
            engine.backward(case.q, kp, vp, case.table, case.d_out, case.m, case.l, dq, np.zeros_like(case.dk0), dvp, case.L,
                            case.D, case.H, case.KVH, case.bs, DT.float32, 0)
        assert e.value.case == "invalidConfiguration"
    finally:
        engine.enableGracefulDegradation = graceful
