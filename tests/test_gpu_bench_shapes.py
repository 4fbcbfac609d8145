"""Parity on the shapes the benchmark runs: the headline decode configuration (batch 256,
contexts uniform in [512, 8192], 32 query / 8 KV heads, float16, scrambled block tables)
and the long-context FP8 sliding-window decode (64 sequences, 64 query / 8 KV heads,
window 4096), both through the reference-shaped C ABI (pam_append_kv, pam_decode) and the
flat decode.  The oracle checks a sample of the sequences: the shortest, the longest and
a seeded choice of the rest; their pages are fetched from the device pools."""
import numpy as np
import pytest

import pagedattentionmetal_b200 as pam
from gpu_helpers import DT, assert_close
from oracle import c_oracle as co

pytestmark = pytest.mark.gpu

BLOCK, HEAD_DIM = 16, 128


def scramble_free_list(cache, n_blocks, rng):
    """Blocks come back from the allocator in a random order, as after a long server run."""
    base = 1 << 40
    for i in range(n_blocks):
        cache.allocateSequence(base + i)
        cache.appendTokens(base + i, 1)
    for i in rng.permutation(n_blocks):
        cache.freeSequence(base + int(i))


def fetch_pages(engine, cache, blocks, kv_heads, elem_bytes, with_scales):
    """The pages `blocks` of the device pools as a compact host pool (page i = blocks[i])."""
    from pagedattentionmetal_b200._cabi import lib
    page = kv_heads * BLOCK * HEAD_DIM * elem_bytes
    dt = np.uint8 if elem_bytes == 1 else np.float16
    k = np.empty((len(blocks), kv_heads, BLOCK, HEAD_DIM), dt)
    v = np.empty_like(k)
    ks = np.empty((len(blocks), kv_heads), np.float16) if with_scales else None
    vs = np.empty_like(ks) if with_scales else None
    kp, vp = cache.kPoolBuffer.ptr, cache.vPoolBuffer.ptr
    for i, b in enumerate(blocks):
        assert lib.pamc_memcpy(engine._ctx, k[i].ctypes.data, kp + int(b) * page, page, 1) == 0
        assert lib.pamc_memcpy(engine._ctx, v[i].ctypes.data, vp + int(b) * page, page, 1) == 0
        if with_scales:
            row = kv_heads * 2
            assert lib.pamc_memcpy(engine._ctx, ks[i].ctypes.data, cache.kScaleBuffer.ptr + int(b) * row, row, 1) == 0
            assert lib.pamc_memcpy(engine._ctx, vs[i].ctypes.data, cache.vScaleBuffer.ptr + int(b) * row, row, 1) == 0
    return k, v, ks, vs


def oracle_on_sample(engine, cache, sample, tables, lens, q, kv_heads, dtype, window=0):
    """co.decode for the sequences `sample` (rows of tables / lens / q) on their own pages."""
    first = [((int(lens[i]) - window) // BLOCK if window and lens[i] > window else 0) for i in sample]
    last = [(int(lens[i]) + BLOCK - 1) // BLOCK for i in sample]
    used = np.unique(np.concatenate([tables[i, f:l] for i, f, l in zip(sample, first, last)]))
    remap = np.zeros(int(tables.max()) + 1, np.int32)
    remap[used] = np.arange(len(used), dtype=np.int32)
    sub = remap[tables[sample]]
    fp8 = dtype == DT.float8
    k, v, ks, vs = fetch_pages(engine, cache, used, kv_heads, 1 if fp8 else 2, fp8)
    return co.decode(np.ascontiguousarray(q[sample]), k, v, sub, lens[sample].astype(np.uint32), kv_heads, BLOCK, int(dtype),
                     window=window, k_scale=None if ks is None else ks.view(np.uint16),
                     v_scale=None if vs is None else vs.view(np.uint16))


def pick_sample(lens, n, seed):
    rng = np.random.default_rng(seed)
    fixed = [int(np.argmin(lens)), int(np.argmax(lens))]
    rest = [i for i in rng.permutation(len(lens)) if i not in fixed][: n - 2]
    return np.array(fixed + [int(i) for i in rest])


def test_headline_decode_shape_sampled_parity():
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda", 0)
    B, H, KVH, seed = 256, 32, 8, 1002
    lens = np.random.default_rng(seed).integers(512, 8192 + 1, size=B).astype(np.int64)
    nblk = (lens + BLOCK - 1) // BLOCK
    n_pool = int(nblk.sum()) + 1024
    engine = pam.PagedAttentionEngine(0)
    cache = pam.KVCacheManager(engine, n_pool, BLOCK, HEAD_DIM, KVH, DT.float16)
    scramble_free_list(cache, n_pool, np.random.default_rng(seed + 2))
    gen = torch.Generator(device=dev)
    for sid in range(B):
        L = int(lens[sid])
        cache.allocateSequence(sid)
        cache.appendTokens(sid, L)
        gen.manual_seed(seed * 1000 + sid)
        kv = torch.randn((2, L, KVH, HEAD_DIM), generator=gen, device=dev, dtype=torch.float32).to(torch.float16)
        engine.appendKV(cache, sid, kv[0].contiguous(), kv[1].contiguous(), 0, L, H)
    ids = list(range(B))
    tables, lens_u = cache.batchTables(ids, int(nblk.max()))
    assert np.array_equal(lens_u.astype(np.int64), lens)
    # the tables are non-contiguous: consecutive entries are rarely neighbours in the pool
    steps = np.diff(tables[0, : nblk[0]])
    assert (steps != 1).mean() > 0.9
    gen.manual_seed(seed * 1000 + 999983)
    q = torch.randn((B, H, HEAD_DIM), generator=gen, device=dev, dtype=torch.float32).to(torch.float16)
    q_host = q.cpu().numpy()
    sample = pick_sample(lens, 32, seed)
    ref = oracle_on_sample(engine, cache, sample, tables, lens_u, q_host, KVH, DT.float16)

    # the reference-shaped call, host buffers
    out = np.zeros_like(q_host)
    engine.decodeBatch(cache, ids, q_host, out, H)
    assert_close(out[sample].astype(np.float32), ref, DT.float16)
    # the flat call, everything resident on the device, lengths read by the host
    out_dev = torch.empty_like(q)
    layer = pam.PagedLayerSpec(HEAD_DIM, H, KVH, BLOCK, DT.float16)
    t_dev = torch.from_numpy(tables).to(dev)
    req = pam.PagedAttentionDecodeRequest(q, cache.kPoolBuffer, cache.vPoolBuffer, t_dev, lens_u, out_dev, B,
                                          tables.shape[1], layer)
    engine.decode(req)
    assert_close(out_dev.cpu().numpy()[sample].astype(np.float32), ref, DT.float16)
    # ... and with the lengths on the device
    l_dev = torch.from_numpy(lens_u.view(np.int32)).to(dev)
    out_dev2 = torch.empty_like(q)
    engine.decode(pam.PagedAttentionDecodeRequest(q, cache.kPoolBuffer, cache.vPoolBuffer, t_dev, l_dev, out_dev2, B,
                                                  tables.shape[1], layer))
    assert_close(out_dev2.cpu().numpy()[sample].astype(np.float32), ref, DT.float16)
    # a decode step later: every sequence one token longer (about one in sixteen gets a new block)
    for sid in ids:
        cache.appendTokens(sid, 1)
        gen.manual_seed(seed * 2000 + sid)
        kv = torch.randn((2, 1, KVH, HEAD_DIM), generator=gen, device=dev, dtype=torch.float32).to(torch.float16)
        engine.appendKV(cache, sid, kv[0].contiguous(), kv[1].contiguous(), int(lens[sid]), 1, H)
    tables2, lens2 = cache.batchTables(ids, int(nblk.max()) + 1)
    ref2 = oracle_on_sample(engine, cache, sample, tables2, lens2, q_host, KVH, DT.float16)
    engine.decodeBatch(cache, ids, q_host, out, H)
    assert_close(out[sample].astype(np.float32), ref2, DT.float16)
    cache.close()
    engine.close()


def test_long_context_fp8_window_decode_shape_sampled_parity():
    """The decode shape of the long-context configuration at reduced context: 64 sequences,
    contexts of two to five windows, window 4096 (several splits per sequence), FP8 KV with
    (block, kv_head) scales written by the append kernels, 64 query / 8 KV heads."""
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda", 0)
    B, H, KVH, W, seed = 64, 64, 8, 4096, 1004
    lens = np.random.default_rng(seed).integers(2 * W, 5 * W + 1, size=B).astype(np.int64)
    nblk = (lens + BLOCK - 1) // BLOCK
    engine = pam.PagedAttentionEngine(0)
    cache = pam.KVCacheManager(engine, int(nblk.sum()) + 64, BLOCK, HEAD_DIM, KVH, DT.float8)
    gen = torch.Generator(device=dev)
    for sid in range(B):
        L = int(lens[sid])
        cache.allocateSequence(sid)
        cache.appendTokens(sid, L)
        first = ((L - W) // BLOCK) * BLOCK             # only what a decode can see is written
        gen.manual_seed(seed * 1000 + sid)
        kv = torch.randn((2, L - first, KVH, HEAD_DIM), generator=gen, device=dev).to(torch.float16)
        engine.appendKV(cache, sid, kv[0].contiguous(), kv[1].contiguous(), first, L - first, H)
    ids = list(range(B))
    tables, lens_u = cache.batchTables(ids, int(nblk.max()))
    q = torch.randn((B, H, HEAD_DIM), generator=gen, device=dev).to(torch.float16)
    q_host = q.cpu().numpy()
    sample = pick_sample(lens, 32, seed)
    ref = oracle_on_sample(engine, cache, sample, tables, lens_u, q_host, KVH, DT.float8, window=W)
    layer = pam.PagedLayerSpec(HEAD_DIM, H, KVH, BLOCK, DT.float8, W)
    t_dev = torch.from_numpy(tables).to(dev)
    for lens_arg in (lens_u, torch.from_numpy(lens_u.view(np.int32)).to(dev)):
        out = torch.empty_like(q)
        engine.decode(pam.PagedAttentionDecodeRequest(q, cache.kPoolBuffer, cache.vPoolBuffer, t_dev, lens_arg, out, B,
                                                      tables.shape[1], layer, cache.kScaleBuffer, cache.vScaleBuffer))
        assert engine.lastStats.temporaryBytes > 0          # several splits per sequence
        assert_close(out.cpu().numpy()[sample].astype(np.float32), ref, DT.float8)
    # the reference-shaped call with the window as the engine's default (PagedAttentionEngine.swift:1028)
    engine.defaultWindowSize = W
    out_h = np.zeros_like(q_host)
    engine.decodeBatch(cache, ids, q_host, out_h, H)
    assert_close(out_h[sample].astype(np.float32), ref, DT.float8)
    cache.close()
    engine.close()
