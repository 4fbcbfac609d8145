"""Paged decode on the GPU against the oracle and the golden vectors."""
import os

import numpy as np
import pytest

import pagedattentionmetal_b200 as pam
from gpu_helpers import DT, TOL, DecodeCase, assert_close, from_io, max_abs
from oracle import paged_oracle as po
from test_oracle import c0_inputs

pytestmark = pytest.mark.gpu


def _flat_decode_f32(engine, q, k_pool, v_pool, tables, lens, kvh, bs, window=0):
    B, H, D = q.shape
    out = np.zeros_like(q)
    req = pam.PagedAttentionDecodeRequest(q, engine.makeBufferFrom(k_pool), engine.makeBufferFrom(v_pool), tables,
                                          lens, out, B, tables.shape[1],
                                          pam.PagedLayerSpec(D, H, kvh, bs, DT.float32, window))
    engine.decode(req)
    return out


def test_golden_decode_small(engine, golden_dir):
    g = np.load(os.path.join(golden_dir, "decode_small.npz"))
    out = _flat_decode_f32(engine, g["q"], g["k_pool"], g["v_pool"], g["tables"], g["lens"], 2, 16)
    assert max_abs(out, g["out"]) < 1e-4


def test_golden_decode_c0(engine, golden_dir):
    """The CPU-runnable benchmark configuration against the outputs of the
    reference's numpy implementation: max-abs <= 2e-3."""
    g = np.load(os.path.join(golden_dir, "decode_c0.npz"))
    q, k_pool, v_pool, tables, lens = c0_inputs()
    out = _flat_decode_f32(engine, q, k_pool, v_pool, tables, lens, 8, 16)
    assert max_abs(out, g["out"]) <= 2e-3
    assert engine.lastStats.operation == pam.Operation.decode and engine.lastStats.batchSize == 8


@pytest.mark.parametrize("dtype", [DT.float16, DT.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,block_size", [
    (8, 2, 128, 16),      # GQA 4
    (16, 2, 128, 16),     # GQA 8
    (32, 2, 128, 16),     # GQA 16: both halves of the MMA tile
    (2, 2, 128, 16),      # MHA
    (6, 2, 128, 16),      # GQA 3
    (8, 2, 64, 16),       # head_dim 64
    (8, 2, 128, 32),      # two tiles per page
    (24, 2, 64, 48),      # GQA 12, three tiles per page
])
def test_fast_decode_matches_oracle(engine, dtype, heads, kv_heads, head_dim, block_size):
    case = DecodeCase(11, 7, 1, 333, heads, kv_heads, head_dim, block_size, dtype)
    out = case.run(engine)
    assert_close(out, case.oracle(), dtype)
    assert np.isfinite(out).all()


@pytest.mark.parametrize("dtype", [DT.float16, DT.bfloat16, DT.float8, DT.float32])
@pytest.mark.parametrize("window", [1, 16, 17, 100, 4096])
def test_sliding_window(engine, dtype, window):
    case = DecodeCase(12, 5, 1, 400, 8, 2, 128, 16, dtype)
    out = case.run(engine, window=window)
    assert_close(out, case.oracle(window=window), dtype)


def test_split_k_many_splits(engine):
    """Few sequences with long contexts: the plan cuts each into many splits
    and the merge kernel combines them."""
    case = DecodeCase(13, 2, 5000, 9000, 8, 2, 128, 16, DT.float16)
    out = case.run(engine)
    assert_close(out, case.oracle(), DT.float16)
    assert engine.lastStats.temporaryBytes > 0
    case = DecodeCase(14, 1, 3000, 3000, 16, 1, 128, 16, DT.bfloat16)
    out = case.run(engine, window=1000)
    assert_close(out, case.oracle(window=1000), DT.bfloat16)


@pytest.mark.parametrize("dtype,heads,kv_heads,head_dim,block_size", [
    (DT.float8, 8, 2, 128, 16),
    (DT.float8, 16, 2, 128, 16),
    (DT.float8, 4, 4, 64, 8),
    (DT.float32, 4, 2, 32, 4),
    (DT.float32, 12, 4, 256, 16),
    (DT.float16, 8, 2, 96, 16),       # head_dim outside the fast path
    (DT.float16, 8, 2, 128, 8),       # block size outside the fast path
    (DT.bfloat16, 40, 2, 128, 16),    # GQA 20: more heads per KV head than one MMA tile
])
def test_general_decode_matches_oracle(engine, dtype, heads, kv_heads, head_dim, block_size):
    case = DecodeCase(15, 4, 1, 150, heads, kv_heads, head_dim, block_size, dtype)
    out = case.run(engine)
    assert_close(out, case.oracle(), dtype)


@pytest.mark.parametrize("heads,kv_heads,block_size", [(8, 2, 16), (16, 2, 16), (32, 2, 32), (2, 2, 16), (64, 8, 16),
                                                        (6, 2, 16), (10, 2, 16), (14, 2, 16), (24, 2, 16)])
def test_fp8_fast_decode_matches_oracle(engine, heads, kv_heads, block_size):
    """FP8 KV through the stream kernel (head_dim 128) with 1 to 16 query heads per KV head
    (up to 8 the products are taken transposed, odd group sizes leave columns empty; above 8
    both halves of the 16-row tile are used), against the oracle's half-precision
    dequantisation chain: max-abs <= 1e-2."""
    case = DecodeCase(20, 6, 1, 400, heads, kv_heads, 128, block_size, DT.float8)
    out = case.run(engine)
    assert_close(out, case.oracle(), DT.float8)
    # long contexts, several splits, sliding window
    case = DecodeCase(21, 2, 3000, 7000, heads, kv_heads, 128, block_size, DT.float8)
    out = case.run(engine, window=2048)
    assert_close(out, case.oracle(window=2048), DT.float8)
    assert engine.lastStats.temporaryBytes > 0


def test_edge_lengths(engine):
    """Length 0 (0/0 in the reference: zeros here), 1, exact tile and block
    multiples, and a length larger than the table can hold (clamped like
    kernels.metal:1451-1452)."""
    for dtype in (DT.float16, DT.float32):
        case = DecodeCase(16, 6, 1, 1, 8, 2, 128, 16, dtype, lens=[0, 1, 16, 17, 32, 48])
        out = case.run(engine)
        ref = case.oracle()
        assert np.all(out[0] == 0)
        assert_close(out[1:], ref[1:], dtype)
    case = DecodeCase(17, 2, 1, 1, 8, 2, 128, 16, DT.float16, lens=[40, 64])
    case.tables = np.ascontiguousarray(case.tables[:, :3])          # room for 48 tokens only
    out = case.run(engine)
    assert_close(out, case.oracle(), DT.float16)


def test_host_buffers_are_staged(engine):
    case = DecodeCase(18, 4, 10, 200, 8, 2, 128, 16, DT.float16)
    out = case.run(engine, host_io=True)
    assert_close(out, case.oracle(), DT.float16)


@pytest.mark.parametrize("dtype", [DT.float16, DT.float8])
def test_reference_cabi_decode_end_to_end(engine, dtype):
    """pam_reserve_sequence / pam_append_tokens / pam_append_kv / pam_decode with
    host buffers, the call sequence of the reference's C ABI (FP8: float16 rows in,
    codes and scales in the pools, float16 queries)."""
    rng = np.random.default_rng(19)
    H, KVH, D, bs = 8, 2, 128, 16
    cache = pam.KVCacheManager(engine, 64, bs, D, KVH, dtype)
    lens = [37, 5, 80, 1, 130]
    ks, vs = {}, {}
    for sid, L in enumerate(lens):
        cache.allocateSequence(sid)
        cache.appendTokens(sid, L)
        ks[sid] = rng.standard_normal((L, KVH, D)).astype(np.float16)
        vs[sid] = rng.standard_normal((L, KVH, D)).astype(np.float16)
        # append in two pieces to exercise token offsets
        cut = L // 2
        if cut:
            engine.appendKV(cache, sid, ks[sid][:cut], vs[sid][:cut], 0, cut, H)
        engine.appendKV(cache, sid, ks[sid][cut:], vs[sid][cut:], cut, L - cut, H)
    ids = [2, 0, 4, 3, 1]
    gk, gv, gks, gvs = cache.readPools()
    if dtype == DT.float16:
        # oracle on its own pools, filled by its own scatter
        kp = np.zeros((64, KVH, bs, D), np.float16)
        vp = np.zeros_like(kp)
        for sid, L in enumerate(lens):
            po.reshape_and_cache(kp, vp, ks[sid], vs[sid], po.slot_mapping(cache.getBlockTable(sid), 0, L, bs), bs)
        assert np.array_equal(gk, kp) and np.array_equal(gv, vp)
    from oracle import c_oracle as co
    for _ in range(2):                                   # the second call reuses the context's staging buffers
        q = rng.standard_normal((len(ids), H, D)).astype(np.float16)
        out = np.zeros_like(q)
        engine.decodeBatch(cache, ids, q, out, H)
        tables, l = cache.batchTables(ids, 9)
        ref = co.decode(q, gk, gv, tables, l, KVH, bs, int(dtype),
                        k_scale=None if gks is None else gks.view(np.uint16),
                        v_scale=None if gvs is None else gvs.view(np.uint16))
        assert_close(out.astype(np.float32), ref, dtype)
    cache.close()


def test_golden_decode_window(engine, golden_dir):
    """Sliding-window decode against the reference's numpy implementation run over the
    window's tokens (tests/golden/make_golden.py, case 5): float32 through the general
    kernel, and the same data as float16 through the stream kernel (head_dim 64 copy)."""
    g = np.load(os.path.join(golden_dir, "decode_window.npz"))
    for wi, w in enumerate(g["windows"]):
        out = _flat_decode_f32(engine, g["q"], g["k_pool"], g["v_pool"], g["tables"], g["lens"], 2, 16, window=int(w))
        assert max_abs(out, g["out"][wi]) < 1e-4


@pytest.mark.parametrize("dtype", [DT.float16, DT.bfloat16, DT.float8])
@pytest.mark.parametrize("window", [0, 700])
def test_ragged_batch_matches_oracle(engine, dtype, window):
    """Lengths from 0 to several thousand tokens in one batch (the kernel cuts the list of
    their tiles into equal pieces, so long sequences are shared by many warps and short ones
    sit inside one piece), with the lengths in host memory and in device memory, with the
    same bits from both and from a second call, then with other lengths."""
    lens = [0, 1, 15, 16, 17, 300, 1024, 1025, 2500, 4000, 6000, 33, 512, 4096, 5, 7000]
    case = DecodeCase(31, len(lens), 1, 1, 8, 2, 128, 16, dtype, lens=lens)
    kp, vp = engine.makeBufferFrom(case.k_pool), engine.makeBufferFrom(case.v_pool)
    ks = engine.makeBufferFrom(case.k_scale) if case.k_scale is not None else None
    vs = engine.makeBufferFrom(case.v_scale) if case.v_scale is not None else None
    q, tables = engine.makeBufferFrom(case.q), engine.makeBufferFrom(case.tables)
    ref = case.oracle(window=window)

    def run(lens_arg):
        out = engine.makeBuffer(case.q.nbytes)
        engine.decode(pam.PagedAttentionDecodeRequest(q, kp, vp, tables, lens_arg, out, len(lens), case.tables.shape[1],
                                                      case.layer(window), ks, vs))
        return from_io(out.download(case.q.dtype, case.q.shape), dtype)

    host = run(case.lens)
    assert np.all(host[0] == 0)
    assert_close(host[1:], ref[1:], dtype)
    assert np.array_equal(run(case.lens), host)
    assert np.array_equal(run(engine.makeBufferFrom(case.lens)), host)
    shorter = np.maximum(case.lens // 3, 1).astype(np.uint32)
    case.lens = shorter
    assert_close(run(shorter), case.oracle(window=window), dtype)


def test_misaligned_query_takes_the_general_kernel(engine):
    """A query pointer the stream kernel's word loads cannot take: the general kernel
    runs instead and the result is the same."""
    case = DecodeCase(32, 3, 10, 300, 8, 2, 128, 16, DT.float16)
    kp, vp = engine.makeBufferFrom(case.k_pool), engine.makeBufferFrom(case.v_pool)
    raw = engine.makeBuffer(case.q.nbytes + 16)
    raw.upload(case.q, offset=2)
    out = engine.makeBuffer(case.q.nbytes)
    req = pam.PagedAttentionDecodeRequest(raw.data_ptr() + 2, kp, vp, case.tables, case.lens, out, 3, case.tables.shape[1],
                                          case.layer())
    assert pam.PagedAttentionEngine.decodePath(req) == 0
    engine.decode(req)
    assert_close(from_io(out.download(np.float16, case.q.shape), DT.float16), case.oracle(), DT.float16)


def _oracle_of_cache(cache, ids, q, kvh, bs, dtype, window=0):
    from oracle import c_oracle as co
    gk, gv, gks, gvs = cache.readPools()
    tables, l = cache.batchTables(ids, max(max(cache.getNumBlocks(i) for i in ids), 1))
    return co.decode(q, gk, gv, tables, l, kvh, bs, int(dtype), window=window,
                     k_scale=None if gks is None else gks.view(np.uint16),
                     v_scale=None if gvs is None else gvs.view(np.uint16))


def test_pam_decode_follows_table_changes(engine):
    """pam_decode keeps the batch's block tables on the device and sends only what changed.
    Every kind of change between two calls must reach the kernels: tokens appended inside a
    block and across a block boundary, a block replaced by copy-on-write, a sequence freed
    and allocated again under the same id, the id list reordered, shortened and extended."""
    rng = np.random.default_rng(33)
    H, KVH, D, bs = 8, 2, 128, 16
    cache = pam.KVCacheManager(engine, 256, bs, D, KVH, DT.float16)
    lens = {}

    def grow(sid, n, hashes=None):
        if sid not in lens:
            cache.allocateSequence(sid)
            lens[sid] = 0
        cache.appendTokens(sid, n, hashes)
        k = rng.standard_normal((n, KVH, D)).astype(np.float16)
        v = rng.standard_normal((n, KVH, D)).astype(np.float16)
        engine.appendKV(cache, sid, k, v, lens[sid], n, H)
        lens[sid] += n

    def check(ids):
        q = rng.standard_normal((len(ids), H, D)).astype(np.float16)
        out = np.zeros_like(q)
        engine.decodeBatch(cache, ids, q, out, H)
        assert_close(out.astype(np.float32), _oracle_of_cache(cache, ids, q, KVH, bs, DT.float16), DT.float16)

    for sid, n in enumerate((37, 5, 80, 1, 130, 600)):
        grow(sid, n)
    ids = [2, 0, 4, 3, 1, 5]
    check(ids)
    check(ids)                                   # nothing changed: only the lengths go up again
    for sid in ids:
        grow(sid, 1)                             # one decode step: sequence 2 crosses a block boundary (80 -> 81)
    check(ids)
    grow(0, 40)
    grow(5, 500)                                 # many new blocks in one row
    check(ids)
    check([5, 1, 0])                             # reordered and shorter
    check(ids + [3, 3])                          # longer, with a repeated id
    # free + allocate under the same id: other pages, possibly fewer of them
    cache.freeSequence(4)
    del lens[4]
    grow(4, 20)
    check(ids)
    # copy-on-write replaces a table entry without changing the table's length
    grow(10, 24, [901, 902])
    grow(11, 24, [901, 902])                     # shares block 0 and the half-full block 1
    check([10, 11, 2])
    before = cache.getBlockTable(11)
    grow(11, 3)                                  # the shared last block is copied first
    after = cache.getBlockTable(11)
    assert before[0] == after[0] and before[1] != after[1] and len(after) == 2
    check([10, 11, 2])
    cache.ensureExclusiveAccess(11, 0)
    assert cache.getBlockTable(11)[0] != after[0]
    check([10, 11, 2])
    # an unknown id fails like the reference's and leaves the cache usable
    with pytest.raises(pam.KVCacheError) as e:
        check([2, 999])
    assert e.value.case == "sequenceNotFound"
    check(ids)
    cache.close()


def test_pam_decode_host_memory_kinds(engine):
    """Query and output in pageable host memory (staged), in page-locked host memory (the
    output is written by the kernels through its device-side address) and in device memory
    give the same bits."""
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(34)
    H, KVH, D, bs = 16, 2, 128, 16
    cache = pam.KVCacheManager(engine, 512, bs, D, KVH, DT.float16)
    ids = list(range(5))
    for sid, L in zip(ids, (900, 3000, 17, 1500, 260)):
        cache.allocateSequence(sid)
        cache.appendTokens(sid, L)
        engine.appendKV(cache, sid, rng.standard_normal((L, KVH, D)).astype(np.float16),
                        rng.standard_normal((L, KVH, D)).astype(np.float16), 0, L, H)
    q = rng.standard_normal((5, H, D)).astype(np.float16)
    pageable = np.zeros_like(q)
    engine.decodeBatch(cache, ids, q, pageable, H)
    assert_close(pageable.astype(np.float32), _oracle_of_cache(cache, ids, q, KVH, bs, DT.float16), DT.float16)
    q_pin = torch.from_numpy(q).pin_memory()
    out_pin = torch.zeros_like(q_pin).pin_memory()
    engine.decodeBatch(cache, ids, q_pin.data_ptr(), out_pin.data_ptr(), H)
    assert np.array_equal(out_pin.numpy().view(np.uint16), pageable.view(np.uint16))
    q_dev, out_dev = engine.makeBufferFrom(q), engine.makeBuffer(q.nbytes)
    engine.decodeBatch(cache, ids, q_dev.data_ptr(), out_dev.data_ptr(), H)
    assert np.array_equal(out_dev.download(np.float16, q.shape).view(np.uint16), pageable.view(np.uint16))
    cache.close()
