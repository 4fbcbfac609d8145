"""Paged prefill (whole sequence, chunks, batches of chunks, windows, prefix
sharing) on the GPU against the oracle and the golden vectors."""
import os

import numpy as np
import pytest

import pagedattentionmetal_b200 as pam
from gpu_helpers import DT, TOL, assert_close, from_io, io_numpy_dtype, max_abs, quantize_pool, to_storage
from oracle import c_oracle as co
from oracle import paged_oracle as po

pytestmark = pytest.mark.gpu


class PrefillCase:
    def __init__(self, seed, seq_len, heads, kv_heads, head_dim, block_size, dtype, spare=2):
        rng = np.random.default_rng(seed)
        self.S, self.H, self.KVH, self.D, self.bs, self.dtype = seq_len, heads, kv_heads, head_dim, block_size, dtype
        nb = (seq_len + block_size - 1) // block_size
        self.n_pool = nb + spare
        self.table = rng.permutation(self.n_pool)[:nb].astype(np.int32)
        shape = (self.n_pool, kv_heads, block_size, head_dim)
        k32, v32 = rng.standard_normal(shape, dtype=np.float32), rng.standard_normal(shape, dtype=np.float32)
        self.k_scale = self.v_scale = None
        if dtype == DT.float8:
            self.k_pool, self.k_scale = quantize_pool(k32)
            self.v_pool, self.v_scale = quantize_pool(v32)
        else:
            self.k_pool, self.v_pool = to_storage(k32, dtype), to_storage(v32, dtype)
        self.q = to_storage(rng.standard_normal((seq_len, heads, head_dim), dtype=np.float32), dtype)

    def layer(self, window=0):
        return pam.PagedLayerSpec(self.D, self.H, self.KVH, self.bs, self.dtype, window)

    def oracle(self, causal=True, window=0, q_start=0, q_len=None):
        q_len = self.S - q_start if q_len is None else q_len
        ws = max(0, self.S - window) if window > 0 else 0           # PagedAttentionEngine.swift:802
        ks = None if self.k_scale is None else self.k_scale.view(np.uint16)
        vs = None if self.v_scale is None else self.v_scale.view(np.uint16)
        return co.prefill(self.q[q_start:q_start + q_len], self.k_pool, self.v_pool, self.table, self.S, self.KVH,
                          self.bs, int(self.dtype), causal=causal, window_start=ws, q_start=q_start,
                          k_scale=ks, v_scale=vs)

    def run(self, engine, causal=True, window=0, q_start=0, q_len=0, chunk=0, host_io=False):
        kp, vp = engine.makeBufferFrom(self.k_pool), engine.makeBufferFrom(self.v_pool)
        ks = engine.makeBufferFrom(self.k_scale) if self.k_scale is not None else None
        vs = engine.makeBufferFrom(self.v_scale) if self.v_scale is not None else None
        rows = q_len if q_len else self.S
        qh = np.ascontiguousarray(self.q[q_start:q_start + rows])
        out_host = np.zeros(qh.shape, dtype=io_numpy_dtype(self.dtype))
        if host_io:
            q, out, table = qh, out_host, self.table
        else:
            q, out, table = engine.makeBufferFrom(qh), engine.makeBuffer(out_host.nbytes), engine.makeBufferFrom(self.table)
        req = pam.PagedAttentionPrefillRequest(q, kp, vp, table, out, self.S, self.layer(window), causal, ks, vs,
                                               q_start, q_len)
        engine.prefill(req, chunk)
        if not host_io:
            out_host = out.download(out_host.dtype, out_host.shape)
        return from_io(out_host, self.dtype)


def test_golden_prefill_small(engine, golden_dir):
    g = np.load(os.path.join(golden_dir, "prefill_small.npz"))
    kp, vp = engine.makeBufferFrom(g["k_pool"]), engine.makeBufferFrom(g["v_pool"])
    for causal, key in ((False, "out_full"), (True, "out_causal")):
        out = np.zeros_like(g["q"])
        engine.prefill(pam.PagedAttentionPrefillRequest(g["q"], kp, vp, g["table"], out, 40,
                                                        pam.PagedLayerSpec(16, 4, 2, 8, DT.float32), causal))
        assert max_abs(out, g[key]) < 1e-4


@pytest.mark.parametrize("dtype", [DT.float16, DT.bfloat16, DT.float32, DT.float8])
@pytest.mark.parametrize("causal", [True, False])
def test_prefill_matches_oracle(engine, dtype, causal):
    case = PrefillCase(31, 150, 8, 2, 128, 16, dtype)
    out = case.run(engine, causal=causal)
    assert_close(out, case.oracle(causal=causal), dtype)


@pytest.mark.parametrize("dtype", [DT.float16, DT.bfloat16])
@pytest.mark.parametrize("seq_len,heads,kv_heads,head_dim,block_size", [
    (1, 4, 2, 128, 16), (16, 4, 4, 128, 16), (129, 8, 2, 128, 16), (300, 16, 2, 128, 16),
    (257, 8, 2, 64, 16), (200, 8, 2, 128, 32), (77, 6, 2, 96, 8), (300, 6, 2, 128, 16), (600, 3, 3, 128, 16),
])
def test_prefill_shapes(engine, dtype, seq_len, heads, kv_heads, head_dim, block_size):
    case = PrefillCase(32, seq_len, heads, kv_heads, head_dim, block_size, dtype)
    out = case.run(engine)
    assert_close(out, case.oracle(), dtype)


@pytest.mark.parametrize("dtype", [DT.float16, DT.float8])
def test_prefill_host_memory_kinds(engine, dtype):
    """Queries and outputs in device memory, in pageable host arrays and in page-locked host
    memory give the same values (host buffers of either kind are staged)."""
    torch = pytest.importorskip("torch")
    case = PrefillCase(61, 700, 8, 2, 128, 16, dtype)
    on_device = case.run(engine)                        # (float32 values of the output)
    assert_close(on_device, case.oracle(), dtype)
    assert np.array_equal(case.run(engine, host_io=True), on_device)
    kp, vp = engine.makeBufferFrom(case.k_pool), engine.makeBufferFrom(case.v_pool)
    ks = engine.makeBufferFrom(case.k_scale) if case.k_scale is not None else None
    vs = engine.makeBufferFrom(case.v_scale) if case.v_scale is not None else None
    q_pin = torch.from_numpy(np.ascontiguousarray(case.q).view(np.uint16).copy()).pin_memory()
    out_pin = torch.zeros_like(q_pin).pin_memory()
    engine.prefill(pam.PagedAttentionPrefillRequest(q_pin.data_ptr(), kp, vp, engine.makeBufferFrom(case.table), out_pin.data_ptr(),
                                                    case.S, case.layer(), True, ks, vs, 0, 0))
    got = from_io(out_pin.numpy().view(io_numpy_dtype(dtype)).reshape(case.q.shape), dtype)
    assert np.array_equal(got, on_device)


@pytest.mark.parametrize("dtype", [DT.float16, DT.bfloat16])
def test_chunked_prefill_equals_full(engine, dtype):
    """Rows of a chunk equal the same rows of a full prefill
    (PagedAttentionEngine.swift:740-756), through q_start/q_len and through the
    engine's chunk loop."""
    case = PrefillCase(33, 400, 8, 2, 128, 16, dtype)
    full = case.oracle()
    for q_start, q_len in ((0, 128), (128, 128), (256, 144), (399, 1), (100, 37)):
        out = case.run(engine, q_start=q_start, q_len=q_len)
        assert_close(out, full[q_start:q_start + q_len], dtype)
    out = case.run(engine, chunk=128)
    assert_close(out, full, dtype)
    engine.defaultChunkSize = 96
    out = case.run(engine, host_io=True)
    engine.defaultChunkSize = 0
    assert_close(out, full, dtype)


@pytest.mark.parametrize("dtype", [DT.float16, DT.float8])
@pytest.mark.parametrize("window", [16, 64, 256])
def test_prefill_window(engine, dtype, window):
    """One window start for all rows, max(0, S - W) (PagedAttentionEngine.swift:802);
    causal rows before the window see no key and are don't-care (zeros here)."""
    case = PrefillCase(34, 208, 8, 2, 128, 16, dtype)
    ref = case.oracle(window=window)
    out = case.run(engine, window=window)
    ws = max(0, 208 - window)
    assert_close(out[ws:], ref[ws:], dtype)
    assert np.all(out[:ws] == 0)
    ref = case.oracle(causal=False, window=window)
    out = case.run(engine, causal=False, window=window)
    assert_close(out, ref, dtype)


def test_batch_prefill_with_shared_prefix(engine):
    """Several sequences sharing prefix pages (refcounted by the manager), one
    chunk each in a single launch; every row equals the oracle's."""
    rng = np.random.default_rng(35)
    n_seq, prefix, total, chunk, H, KVH, D, bs = 4, 64, 160, 48, 8, 2, 128, 16
    dtype = DT.bfloat16
    cache = pam.KVCacheManager(engine, 64, bs, D, KVH, dtype)
    shared_k = rng.standard_normal((prefix, KVH, D), dtype=np.float32)
    shared_v = rng.standard_normal((prefix, KVH, D), dtype=np.float32)
    ks, vs, qs = [], [], []
    for s in range(n_seq):
        k = np.concatenate([shared_k, rng.standard_normal((total - prefix, KVH, D), dtype=np.float32)])
        v = np.concatenate([shared_v, rng.standard_normal((total - prefix, KVH, D), dtype=np.float32)])
        ks.append(to_storage(k, dtype)); vs.append(to_storage(v, dtype))
        qs.append(to_storage(rng.standard_normal((total, H, D), dtype=np.float32), dtype))
        cache.allocateSequence(s)
        cache.appendTokens(s, prefix, list(range(prefix // bs)))
        if s == 0:
            engine.appendKV(cache, 0, ks[0][:prefix], vs[0][:prefix], 0, prefix, H)       # written once
        cache.appendTokens(s, total - prefix)
        engine.appendKV(cache, s, ks[s][prefix:], vs[s][prefix:], prefix, total - prefix, H)
    assert cache.memoryStats().sharedBlocks == prefix // bs
    assert cache.memoryStats().prefixCacheHits == (n_seq - 1) * (prefix // bs)
    tables, lens = cache.batchTables(list(range(n_seq)), total // bs)
    gk, gv, _, _ = cache.readPools()
    q_starts = [64, 96, 112, 64]
    q_lens = [chunk, chunk, chunk, 17]
    q_cat = np.concatenate([qs[s][q_starts[s]:q_starts[s] + q_lens[s]] for s in range(n_seq)])
    out = np.zeros(q_cat.shape, dtype=np.uint16)
    engine.prefillBatch(q_cat, cache.kPoolBuffer, cache.vPoolBuffer, tables, out, [total] * n_seq, q_starts, q_lens,
                        total // bs, pam.PagedLayerSpec(D, H, KVH, bs, dtype))
    o = 0
    for s in range(n_seq):
        ref = co.prefill(qs[s][q_starts[s]:q_starts[s] + q_lens[s]], gk, gv, tables[s], total, KVH, bs, int(dtype),
                         q_start=q_starts[s])
        assert_close(from_io(out[o:o + q_lens[s]], dtype), ref, dtype)
        o += q_lens[s]
    cache.close()


def test_reference_cabi_prefill(engine):
    rng = np.random.default_rng(36)
    H, KVH, D, bs, S = 4, 2, 128, 16, 70
    cache = pam.KVCacheManager(engine, 8, bs, D, KVH, DT.float16)
    cache.allocateSequence(5)
    cache.appendTokens(5, S)
    k = rng.standard_normal((S, KVH, D)).astype(np.float16)
    v = rng.standard_normal((S, KVH, D)).astype(np.float16)
    q = rng.standard_normal((S, H, D)).astype(np.float16)
    engine.appendKV(cache, 5, k, v, 0, S, H)
    out = np.zeros_like(q)
    engine.prefillSequence(cache, 5, q, out, S, H, True)
    gk, gv, _, _ = cache.readPools()
    ref = co.prefill(q, gk, gv, np.array(cache.getBlockTable(5), np.int32), S, KVH, bs, 1)
    assert_close(out.astype(np.float32), ref, DT.float16)
    assert engine.lastStats.sequenceLength == S and engine.lastStats.numBlocks == 5
    cache.close()


@pytest.mark.parametrize("seq_len,window,q_start,q_len", [(700, 0, 0, 0), (1000, 256, 0, 0), (900, 300, 512, 388), (520, 64, 0, 0)])
def test_prefill_fp8_tensor_path(engine, seq_len, window, q_start, q_len):
    """FP8 KV with head_dim 128 goes through the tensor-core kernel: the visible pages are
    dequantised to float16 first (dequant_fp8, kernels.metal:553-562), so the result obeys
    the FP8 bound against the oracle, which dequantises the same way."""
    case = PrefillCase(41, seq_len, 8, 2, 128, 16, DT.float8)
    ref = case.oracle(window=window, q_start=q_start, q_len=q_len or None)
    out = case.run(engine, window=window, q_start=q_start, q_len=q_len)
    assert engine.lastStats.operation == pam.Operation.prefillMMA
    lo = max(0, max(0, seq_len - window) - q_start) if window > 0 else 0     # rows before the window: don't-care
    assert_close(out[lo:], ref[lo:], DT.float8)
    # and the general kernel gives the same within the bound
    engine.setPrefillTensorPath(False)
    try:
        gen = case.run(engine, window=window, q_start=q_start, q_len=q_len)
        assert engine.lastStats.operation != pam.Operation.prefillMMA
    finally:
        engine.setPrefillTensorPath(True)
    assert_close(gen[lo:], ref[lo:], DT.float8)


@pytest.mark.parametrize("dtype", [DT.bfloat16, DT.float16])
def test_prefill_batch_many_items_per_cta(engine, dtype):
    """A ragged batch with far more work items than multiprocessors (each CTA of the
    tensor-core kernel walks several items, of very different lengths, with chunks that
    start inside a tile): every row of every sequence against the oracle."""
    rng = np.random.default_rng(37)
    H, KVH, D, bs = 32, 8, 128, 16
    seq_lens = [1500, 700, 1029, 130, 2048, 333, 1, 900]
    q_starts = [1000, 0, 517, 0, 1536, 300, 0, 128]
    q_lens = [500, 700, 512, 130, 512, 33, 1, 700]
    n_seq = len(seq_lens)
    max_nb = (max(seq_lens) + bs - 1) // bs
    n_pool = sum((L + bs - 1) // bs for L in seq_lens) + 8
    perm = rng.permutation(n_pool).astype(np.int32)
    tables = np.zeros((n_seq, max_nb), np.int32)
    o = 0
    for s, L in enumerate(seq_lens):
        nb = (L + bs - 1) // bs
        tables[s, :nb] = perm[o:o + nb]
        o += nb
    shape = (n_pool, KVH, bs, D)
    k_pool = to_storage(rng.standard_normal(shape, dtype=np.float32), dtype)
    v_pool = to_storage(rng.standard_normal(shape, dtype=np.float32), dtype)
    qs = [to_storage(rng.standard_normal((q_lens[s], H, D), dtype=np.float32), dtype) for s in range(n_seq)]
    q_cat = np.concatenate(qs)
    kp, vp = engine.makeBufferFrom(k_pool), engine.makeBufferFrom(v_pool)
    out_buf = engine.makeBuffer(q_cat.nbytes)
    engine.prefillBatch(engine.makeBufferFrom(q_cat), kp, vp, engine.makeBufferFrom(tables), out_buf, seq_lens, q_starts,
                        q_lens, max_nb, pam.PagedLayerSpec(D, H, KVH, bs, dtype))
    assert engine.lastStats.operation == pam.Operation.prefillMMA
    out = out_buf.download(io_numpy_dtype(dtype), q_cat.shape)
    o = 0
    for s in range(n_seq):
        ref = co.prefill(qs[s], k_pool, v_pool, tables[s], seq_lens[s], KVH, bs, int(dtype), q_start=q_starts[s])
        assert_close(from_io(out[o:o + q_lens[s]], dtype), ref, dtype)
        o += q_lens[s]


@pytest.mark.parametrize("dtype", [DT.float32, DT.float16, DT.bfloat16, DT.float8])
@pytest.mark.parametrize("seq_len,window", [(128, 0), (301, 0), (640, 256)])
def test_fused_prefill_equals_append_then_prefill(engine, dtype, seq_len, window):
    """PagedAttentionEngine.fusedPrefill (PagedAttentionEngine.swift:633-710): the reference's
    own test of the call (PagedAttentionMetalTests.swift:927-1037) compares the output and
    both pools with a separate append followed by prefill; here they must be identical bit
    for bit (FP8 codes and scales included), and the output must meet the oracle's bound
    over the pools the oracle's append produces."""
    rng = np.random.default_rng(70 + seq_len)
    H, KVH, D, bs = 8, 2, 128, 16
    n_pool = (seq_len + bs - 1) // bs + 3
    layer = pam.PagedLayerSpec(D, H, KVH, bs, dtype, window)
    io = DT.float16 if dtype == DT.float8 else dtype                       # FP8 pools take float16 rows
    q = to_storage(rng.standard_normal((seq_len, H, D), dtype=np.float32), io)
    k = to_storage(rng.standard_normal((seq_len, KVH, D), dtype=np.float32), io)
    v = to_storage(rng.standard_normal((seq_len, KVH, D), dtype=np.float32), io)

    def run(fused):
        cache = pam.KVCacheManager(engine, n_pool, bs, D, KVH, dtype)
        cache.allocateSequence(1)
        cache.appendTokens(1, seq_len)
        table = np.asarray(cache.getBlockTable(1), dtype=np.int32)
        out = np.zeros_like(q)
        if fused:
            engine.fusedPrefill(pam.PagedAttentionFusedPrefillRequest(
                q, k, v, table, cache.kPoolBuffer, cache.vPoolBuffer, out, seq_len, layer, True,
                cache.kScaleBuffer, cache.vScaleBuffer), cache)
            assert engine.lastStats.operation == pam.Operation.prefillSinglePass
            assert engine.lastStats.sequenceLength == seq_len
        else:
            engine.appendKV(cache, 1, k, v, 0, seq_len, H)
            engine.prefill(pam.PagedAttentionPrefillRequest(q, cache.kPoolBuffer, cache.vPoolBuffer, table, out,
                                                            seq_len, layer, True, cache.kScaleBuffer,
                                                            cache.vScaleBuffer))
        pools = cache.readPools()
        cache.close()
        return out, pools, table

    out_f, pools_f, table = run(True)
    out_s, pools_s, table_s = run(False)
    assert np.array_equal(table, table_s)
    for a, b in zip(pools_f, pools_s):
        assert (a is None) == (b is None)
        if a is not None:
            assert np.array_equal(a.view(np.uint8), b.view(np.uint8))
    assert np.array_equal(out_f.view(np.uint8), out_s.view(np.uint8))
    # against the oracle, over the pools the oracle's own append makes
    ws = max(0, seq_len - window) if window > 0 else 0
    kp, vp, ks, vs = pools_f
    ref = co.prefill(q, kp, vp, table, seq_len, KVH, bs, int(dtype), causal=True, window_start=ws, q_start=0,
                     k_scale=None if ks is None else ks.view(np.uint16),
                     v_scale=None if vs is None else vs.view(np.uint16))
    assert_close(from_io(out_f, dtype)[ws:], ref[ws:], dtype)
    if dtype == DT.float8:
        okp, ovp = np.zeros_like(kp), np.zeros_like(vp)
        oks, ovs = np.zeros(ks.shape, np.uint16), np.zeros(vs.shape, np.uint16)
        co.reshape_and_cache_fp8(k, v, okp, ovp, oks, ovs, po.slot_mapping(table, 0, seq_len, bs), bs)
        assert np.array_equal(okp, kp) and np.array_equal(ovp, vp)
        assert np.array_equal(oks, ks.view(np.uint16)) and np.array_equal(ovs, vs.view(np.uint16))


def test_fused_prefill_errors(engine):
    """seqLen and buffer checks in the reference's order (PagedAttentionEngine.swift:634-640)."""
    D, H, KVH, bs = 128, 4, 2, 16
    layer = pam.PagedLayerSpec(D, H, KVH, bs, DT.float16)
    cache = pam.KVCacheManager(engine, 4, bs, D, KVH, DT.float16)
    q = np.zeros((20, H, D), np.float16)
    kv = np.zeros((20, KVH, D), np.float16)
    table = np.array([0, 1], np.int32)
    mk = lambda seq_len, tbl, out: pam.PagedAttentionFusedPrefillRequest(
        q, kv, kv, tbl, cache.kPoolBuffer, cache.vPoolBuffer, out, seq_len, layer)
    with pytest.raises(pam.PagedAttentionError, match="seqLen must be positive"):
        engine.fusedPrefill(mk(0, table, np.zeros_like(q)))
    with pytest.raises(pam.PagedAttentionError, match="blockTable"):
        engine.fusedPrefill(mk(20, table[:1], np.zeros_like(q)))
    with pytest.raises(pam.PagedAttentionError, match="output"):
        engine.fusedPrefill(mk(20, table, np.zeros((10, H, D), np.float16)))
    fp8 = pam.PagedLayerSpec(D, H, KVH, bs, DT.float8)
    with pytest.raises(pam.PagedAttentionError, match="cache handle"):
        engine.fusedPrefill(pam.PagedAttentionFusedPrefillRequest(
            q, kv, kv, table, cache.kPoolBuffer, cache.vPoolBuffer, np.zeros_like(q), 20, fp8))
    cache.close()


def test_prefill_shared_prefix_with_copy_on_write(engine):
    """The prefill configuration with a shared prefix that ends inside a block: 2048-token
    bfloat16 sequences of 32 query / 8 KV heads in chunks of 512, the first 1032 tokens (65
    block hashes, the last block half full) shared.  Every follower's first own append
    copies that block (KVCacheManager.swift:134-140, 176-194).  Block tables and the
    copy-on-write log must equal the oracle manager's, the pools the oracle's scatter and
    block copies bit for bit, and chunk rows on both sides of the copied block the oracle's
    attention."""
    rng = np.random.default_rng(1003)
    n_seq, prefix, total, chunk, H, KVH, D, bs = 4, 1032, 2048, 512, 32, 8, 128, 16
    dtype = DT.bfloat16
    n_hash = (prefix + bs - 1) // bs                                        # 65
    n_pool = 128 + (n_seq - 1) * 64 + 8
    cache = pam.KVCacheManager(engine, n_pool, bs, D, KVH, dtype)
    ora = po.OracleKVCacheManager(n_pool, bs)
    ok_pool = np.zeros((n_pool, KVH, bs, D), np.uint16)
    ov_pool = np.zeros_like(ok_pool)
    shared_k = rng.standard_normal((prefix, KVH, D), dtype=np.float32)
    shared_v = rng.standard_normal((prefix, KVH, D), dtype=np.float32)
    ks, vs, qs = [], [], []
    cow_log = []
    for s in range(n_seq):
        k = to_storage(np.concatenate([shared_k, rng.standard_normal((total - prefix, KVH, D), dtype=np.float32)]), dtype)
        v = to_storage(np.concatenate([shared_v, rng.standard_normal((total - prefix, KVH, D), dtype=np.float32)]), dtype)
        ks.append(k); vs.append(v)
        qs.append(to_storage(rng.standard_normal((total, H, D), dtype=np.float32), dtype))
        cache.allocateSequence(s); ora.allocate_sequence(s)
        cache.appendTokens(s, prefix, list(range(n_hash))); ora.append_tokens(s, prefix, list(range(n_hash)))
        if s == 0:
            engine.appendKV(cache, 0, k[:prefix], v[:prefix], 0, prefix, H)           # the prefix is written once
            po.reshape_and_cache(ok_pool, ov_pool, k[:prefix], v[:prefix], po.slot_mapping(ora.block_table(0), 0, prefix, bs), bs)
        before = list(ora.block_table(s))
        cache.appendTokens(s, total - prefix); ora.append_tokens(s, total - prefix)
        after = list(ora.block_table(s))
        assert cache.getBlockTable(s) == after
        log = cache.drainCopyOnWriteLog()
        if s == 0:
            assert log == [] and after[:n_hash] == before
        else:
            # block 64 was shared and half full: it is replaced by a private copy before the append
            assert after[:n_hash - 1] == before[:n_hash - 1] and after[n_hash - 1] != before[n_hash - 1]
            assert log == [(before[n_hash - 1], after[n_hash - 1])]
            po.copy_blocks([ok_pool, ov_pool], [before[n_hash - 1]], [after[n_hash - 1]])
            cow_log += log
        engine.appendKV(cache, s, k[prefix:], v[prefix:], prefix, total - prefix, H)
        po.reshape_and_cache(ok_pool, ov_pool, k[prefix:], v[prefix:], po.slot_mapping(after, prefix, total - prefix, bs), bs)
    assert len(cow_log) == n_seq - 1
    stats = cache.memoryStats()
    want = ora.memory_stats()
    assert stats.sharedBlocks == want["sharedBlocks"] == n_hash - 1
    assert stats.prefixCacheHits == want["prefixCacheHits"] == (n_seq - 1) * n_hash
    assert cache.availableBlocks == ora.available_blocks
    gk, gv, _, _ = cache.readPools()
    assert np.array_equal(gk, ok_pool) and np.array_equal(gv, ov_pool)
    # the chunk loop of the configuration: four launches, all sequences in each
    tables, _ = cache.batchTables(list(range(n_seq)), total // bs)
    layer = pam.PagedLayerSpec(D, H, KVH, bs, dtype)
    for c in range(total // chunk):
        q_cat = np.concatenate([qs[s][c * chunk:(c + 1) * chunk] for s in range(n_seq)])
        out = np.zeros(q_cat.shape, dtype=np.uint16)
        engine.prefillBatch(q_cat, cache.kPoolBuffer, cache.vPoolBuffer, tables, out, [(c + 1) * chunk] * n_seq,
                            [c * chunk] * n_seq, [chunk] * n_seq, total // bs, layer)
        assert engine.lastStats.operation == pam.Operation.prefillMMA
        # rows checked: around the copied block in chunk 2 (tokens 1024 .. 1055), else the chunk's last 16
        r0, nr = (0, 32) if c == 2 else (chunk - 16, 16)
        for s in range(n_seq):
            ref = co.prefill(qs[s][c * chunk + r0:c * chunk + r0 + nr], gk, gv, tables[s], (c + 1) * chunk, KVH, bs,
                             int(dtype), q_start=c * chunk + r0)
            assert_close(from_io(out[s * chunk + r0:s * chunk + r0 + nr], dtype), ref, dtype)
    cache.close()


def test_fp8_staged_pages_follow_the_reference_dequant_chain(engine):
    """The float16 pages the tensor-core prefill reads for FP8 KV must be dequant_fp8's
    all-half chain (kernels.metal:553-562) exactly.  One token per sequence: the only weight
    is 1, so a head's output row is the value row of its KV head after dequantisation — every
    code against scales over sixteen binades, zero, sub-normal and 0x7F/0xFF codes included."""
    rng = np.random.default_rng(43)
    n_seq, H, KVH, D, bs = 512, 8, 8, 128, 16
    shape = (n_seq, KVH, bs, D)
    k_codes = rng.integers(0, 256, size=shape, dtype=np.uint8)
    v_codes = rng.integers(0, 256, size=shape, dtype=np.uint8)
    v_codes[:, :, 0, :] = (np.arange(n_seq * KVH * D, dtype=np.int64) * 37 % 256).reshape(n_seq, KVH, D).astype(np.uint8)
    mant = 1.0 + rng.integers(0, 1024, size=(n_seq, KVH)) / 1024.0
    v_scale = (mant * 2.0 ** rng.integers(-12, 4, size=(n_seq, KVH))).astype(np.float16)
    k_scale = np.full((n_seq, KVH), 0.01, np.float16)
    q = rng.standard_normal((n_seq, H, D)).astype(np.float16)
    tables = np.arange(n_seq, dtype=np.int32).reshape(n_seq, 1)
    out = np.zeros_like(q)
    engine.prefillBatch(q, engine.makeBufferFrom(k_codes), engine.makeBufferFrom(v_codes), tables, out, [1] * n_seq,
                        [0] * n_seq, [1] * n_seq, 1, pam.PagedLayerSpec(D, H, KVH, bs, DT.float8), True,
                        engine.makeBufferFrom(k_scale), engine.makeBufferFrom(v_scale))
    assert engine.lastStats.operation == pam.Operation.prefillMMA
    want = po.dequant_fp8(v_codes[:, :, 0, :], v_scale[:, :, None])           # [seq][kv head = head][dim]
    finite = np.isfinite(want)
    assert finite.mean() > 0.99
    assert np.array_equal(out[finite], want[finite])
    assert len(np.unique(v_codes[:, :, 0, :])) == 256


def test_golden_prefill_window(engine, golden_dir):
    """Prefill with a block-aligned window start against the reference's numpy
    implementation run over the window's tokens (tests/golden/make_golden.py, case 6); causal
    rows below the window start see no key (0/0 in the reference) and come back as zeros."""
    g = np.load(os.path.join(golden_dir, "prefill_window.npz"))
    S, W = g["q"].shape[0], int(g["window"])
    kp, vp = engine.makeBufferFrom(g["k_pool"]), engine.makeBufferFrom(g["v_pool"])
    for causal, key in ((False, "out_full"), (True, "out_causal")):
        out = np.full_like(g["q"], 7.0)
        engine.prefill(pam.PagedAttentionPrefillRequest(g["q"], kp, vp, g["table"], out, S,
                                                        pam.PagedLayerSpec(16, 4, 2, 8, DT.float32, W), causal))
        seen = ~np.isnan(g[key])
        assert max_abs(out[seen], g[key][seen]) < 1e-4
        assert np.all(out[~seen] == 0)
