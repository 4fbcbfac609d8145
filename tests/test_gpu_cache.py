"""KV append (plain and FP8), copy-on-write block copies and the allocator with
real pools on the GPU: pools, codes and scales are bit-exact with the oracle."""
import numpy as np
import pytest

import pagedattentionmetal_b200 as pam
from gpu_helpers import DT, to_storage
from oracle import c_oracle as co
from oracle import paged_oracle as po

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [DT.float16, DT.bfloat16, DT.float32])
@pytest.mark.parametrize("kv_heads,head_dim,block_size", [(8, 128, 16), (2, 64, 4), (3, 20, 5)])
def test_reshape_and_cache_bit_exact(engine, dtype, kv_heads, head_dim, block_size):
    rng = np.random.default_rng(21)
    T = 333
    nblk = T // block_size + 30
    cache = pam.KVCacheManager(engine, nblk, block_size, head_dim, kv_heads, dtype)
    k = to_storage(rng.standard_normal((T, kv_heads, head_dim), dtype=np.float32), dtype)
    v = to_storage(rng.standard_normal((T, kv_heads, head_dim), dtype=np.float32), dtype)
    slots = rng.choice(nblk * block_size, T, replace=False).astype(np.int64)
    # first half from host memory, second half from device memory
    engine.reshapeAndCache(cache, k[:100], v[:100], slots[:100], 100)
    dk, dv, ds = engine.makeBufferFrom(k[100:]), engine.makeBufferFrom(v[100:]), engine.makeBufferFrom(slots[100:])
    engine.reshapeAndCache(cache, dk, dv, ds, T - 100)
    kp = np.zeros((nblk, kv_heads, block_size, head_dim), dtype=k.dtype)
    vp = np.zeros_like(kp)
    po.reshape_and_cache(kp, vp, k, v, slots, block_size)
    gk, gv, _, _ = cache.readPools()
    assert np.array_equal(gk.view(np.uint8), kp.view(np.uint8)) and np.array_equal(gv.view(np.uint8), vp.view(np.uint8))
    assert engine.lastStats.operation == pam.Operation.append
    cache.close()


@pytest.mark.parametrize("kv_heads,head_dim,block_size", [(8, 128, 16), (2, 64, 4), (3, 20, 5)])
def test_fp8_append_bit_exact(engine, kv_heads, head_dim, block_size):
    """Codes and scales after three appends (fresh groups, groups that grow,
    groups whose absmax shrinks) equal the oracle's, bit for bit."""
    rng = np.random.default_rng(22)
    T = 400
    nblk = T // block_size + 15
    cache = pam.KVCacheManager(engine, nblk, block_size, head_dim, kv_heads, DT.float8)
    kc = np.zeros((nblk, kv_heads, block_size, head_dim), np.uint8)
    vc = np.zeros_like(kc)
    ks = np.zeros((nblk, kv_heads), np.float16)
    vs = np.zeros_like(ks)
    slots = rng.choice(nblk * block_size, T, replace=False).astype(np.int64)
    amp = [1.0, 3.0, 0.25]
    for i, (a, b) in enumerate([(0, 150), (150, 300), (300, 400)]):
        k = (rng.standard_normal((b - a, kv_heads, head_dim)) * amp[i]).astype(np.float16)
        v = (rng.standard_normal((b - a, kv_heads, head_dim)) * amp[i]).astype(np.float16)
        if i == 1:
            k[::7] = 0            # whole zero rows and exact ties
            v[::5] = np.float16(0.5)
        engine.reshapeAndCache(cache, k, v, slots[a:b], b - a)
        po.reshape_and_cache_fp8(kc, vc, ks, vs, k, v, slots[a:b], block_size)
    gk, gv, gks, gvs = cache.readPools()
    assert np.array_equal(gks.view(np.uint16), ks.view(np.uint16)) and np.array_equal(gvs.view(np.uint16), vs.view(np.uint16))
    assert np.array_equal(gk, kc) and np.array_equal(gv, vc)
    cache.close()


def test_fp8_quantiser_all_halves(engine):
    """Every finite float16 value through the GPU quantiser at several scales."""
    allh = np.arange(65536, dtype=np.uint32).astype(np.uint16).view(np.float16)
    allh = allh[np.isfinite(allh)]
    D = 128
    n = (len(allh) // D) * D
    vals = allh[:n].reshape(-1, 1, D)                                  # [T][1][D]
    tail = np.resize(allh[n - D:], D).reshape(1, 1, D)
    tail[0, 0, : len(allh) - n] = allh[n:]
    vals = np.concatenate([vals, tail])
    T = vals.shape[0]
    for seed_scale in (1.0, 0.37, 143.0):
        # the scale of a group is absmax/448 of its tokens: one token per block, so that
        # each row gets its own scale; an extra factor stretches the range of quotients
        x = (vals.astype(np.float32) * np.float32(seed_scale)).astype(np.float16)
        x = np.where(np.isfinite(x), x, np.float16(0))
        cache = pam.KVCacheManager(engine, T, 1, D, 1, DT.float8)
        slots = np.arange(T, dtype=np.int64)
        engine.reshapeAndCache(cache, x, x[::-1].copy(), slots, T)
        kc = np.zeros((T, 1, 1, D), np.uint8)
        vc = np.zeros_like(kc)
        ks = np.zeros((T, 1), np.float16)
        vs = np.zeros_like(ks)
        co.reshape_and_cache_fp8(x, x[::-1].copy(), kc, vc, ks.view(np.uint16), vs.view(np.uint16), slots, 1)
        gk, gv, gks, gvs = cache.readPools()
        assert np.array_equal(gks, ks) and np.array_equal(gvs, vs)
        # A group whose absmax is below 448 * 2^-25 gets the half scale 0; a zero
        # in such a group is 0/0, which the reference leaves undefined
        # (kernels.metal:565-566, clamp of a NaN).  Everything else must match.
        xr = x[::-1]
        defined_k = ~((ks[:, :, None, None] == 0) & (x.reshape(kc.shape) == 0))
        defined_v = ~((vs[:, :, None, None] == 0) & (xr.reshape(vc.shape) == 0))
        assert np.array_equal(gk[defined_k], kc[defined_k]) and np.array_equal(gv[defined_v], vc[defined_v])
        assert defined_k.mean() > 0.99
        cache.close()


def test_out_of_pool_slots_are_rejected_or_skipped(engine):
    cache = pam.KVCacheManager(engine, 4, 4, 8, 1, DT.float16)
    k = np.ones((2, 1, 8), np.float16)
    with pytest.raises(pam.PagedAttentionError) as e:
        engine.reshapeAndCache(cache, k, k, np.array([0, 16], dtype=np.int64), 2)      # host slots are checked
    assert e.value.case == "invalidConfiguration"
    # device slots are checked in the kernel: the bad token is skipped, the good one lands
    engine.reshapeAndCache(cache, k, k, engine.makeBufferFrom(np.array([3, 99], dtype=np.int64)), 2)
    gk, _, _, _ = cache.readPools()
    assert gk[0, 0, 3].tolist() == [1.0] * 8 and gk.sum() == 8
    cache.close()


@pytest.mark.parametrize("dtype", [DT.float16, DT.float8])
def test_copy_blocks_bit_exact(engine, dtype):
    rng = np.random.default_rng(23)
    nblk, kvh, bs, D = 64, 8, 16, 128
    cache = pam.KVCacheManager(engine, nblk, bs, D, kvh, dtype)
    T = nblk * bs // 2
    k = rng.standard_normal((T, kvh, D)).astype(np.float16)
    v = rng.standard_normal((T, kvh, D)).astype(np.float16)
    slots = rng.choice(nblk * bs, T, replace=False).astype(np.int64)
    engine.reshapeAndCache(cache, k, v, slots, T)
    before = cache.readPools()
    perm = rng.permutation(nblk)
    src, dst = perm[:20], perm[20:40]
    engine.copyBlocks(cache, src, dst)
    after = cache.readPools()
    for a, b in zip(before, after):
        if a is None:
            continue
        exp = a.copy()
        po.copy_blocks([exp], src, dst)
        assert np.array_equal(exp.view(np.uint8), b.view(np.uint8))
    # a chain (dst of one pair is the src of a later one) behaves like sequential copies
    engine.copyBlocks(cache, [perm[40], perm[41]], [perm[41], perm[42]])
    chained = cache.readPools()[0]
    assert np.array_equal(chained[perm[42]], after[0][perm[40]])
    cache.close()


def test_copy_on_write_copies_pages_on_the_gpu(engine):
    """Prefix sharing with a half-filled last block: the follower's first
    divergent append copies that block (K, V) before it writes."""
    rng = np.random.default_rng(24)
    kvh, bs, D, H = 2, 16, 64, 4
    cache = pam.KVCacheManager(engine, 32, bs, D, kvh, DT.float16)
    prefix = 40                                                          # 2.5 blocks
    hashes = [7, 8, 9]
    k0 = rng.standard_normal((prefix, kvh, D)).astype(np.float16)
    v0 = rng.standard_normal((prefix, kvh, D)).astype(np.float16)
    cache.allocateSequence(0)
    cache.appendTokens(0, prefix, hashes)
    engine.appendKV(cache, 0, k0, v0, 0, prefix, H)
    cache.allocateSequence(1)
    cache.appendTokens(1, prefix, hashes)
    assert cache.getBlockTable(1) == cache.getBlockTable(0)
    assert cache.memoryStats().sharedBlocks == 3
    k1 = rng.standard_normal((3, kvh, D)).astype(np.float16)
    v1 = rng.standard_normal((3, kvh, D)).astype(np.float16)
    cache.appendTokens(1, 3)                                             # copy-on-write of block 2
    t0, t1 = cache.getBlockTable(0), cache.getBlockTable(1)
    assert t1[:2] == t0[:2] and t1[2] != t0[2]
    assert cache.drainCopyOnWriteLog() == [(t0[2], t1[2])]
    engine.appendKV(cache, 1, k1, v1, prefix, 3, H)
    gk, gv, _, _ = cache.readPools()
    # sequence 0's block is untouched, sequence 1's copy holds the prefix rows plus its own
    assert np.array_equal(gk[t0[2], :, :8], np.transpose(k0[32:40], (1, 0, 2)))
    assert np.all(gk[t0[2], :, 8:] == 0)
    assert np.array_equal(gk[t1[2], :, :8], np.transpose(k0[32:40], (1, 0, 2)))
    assert np.array_equal(gk[t1[2], :, 8:11], np.transpose(k1, (1, 0, 2)))
    assert np.array_equal(gv[t1[2], :, 8:11], np.transpose(v1, (1, 0, 2)))
    cache.close()


def test_append_through_block_table_on_device(engine):
    """PagedAttentionEngine.appendToCache with a device block table and a
    token offset (the slot is derived in the kernel, kernels.metal:1823-1827)."""
    rng = np.random.default_rng(25)
    kvh, bs, D = 4, 16, 128
    cache = pam.KVCacheManager(engine, 16, bs, D, kvh, DT.float16)
    table = np.array([5, 2, 9, 11], dtype=np.int32)
    k = rng.standard_normal((30, kvh, D)).astype(np.float16)
    v = rng.standard_normal((30, kvh, D)).astype(np.float16)
    req = pam.PagedKVAppendRequest(engine.makeBufferFrom(k), engine.makeBufferFrom(v), cache.kPoolBuffer,
                                   cache.vPoolBuffer, engine.makeBufferFrom(table), 21, 30,
                                   pam.PagedLayerSpec(D, kvh, kvh, bs, DT.float16))
    engine.appendToCache(req)
    kp = np.zeros((16, kvh, bs, D), np.float16)
    vp = np.zeros_like(kp)
    po.reshape_and_cache(kp, vp, k, v, po.slot_mapping(table, 21, 30, bs), bs)
    gk, gv, _, _ = cache.readPools()
    assert np.array_equal(gk, kp) and np.array_equal(gv, vp)
    cache.close()


def test_config_append_fp8_cow_full_size(engine):
    """The append configuration at full size: 4096 tokens of 8 KV heads x 128
    into a pool of 4096 blocks x 16 at random distinct slots, as float16 and
    as FP8 with per-(block, kv_head) scales, then a copy of 512 random blocks."""
    rng = np.random.default_rng(1001)
    T, kvh, D, bs, nblk = 4096, 8, 128, 16, 4096
    k = rng.standard_normal((T, kvh, D), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((T, kvh, D), dtype=np.float32).astype(np.float16)
    slots = rng.choice(nblk * bs, T, replace=False).astype(np.int64)
    perm = rng.permutation(nblk)
    src, dst = perm[:512], perm[512:1024]
    # float16
    cache = pam.KVCacheManager(engine, nblk, bs, D, kvh, DT.float16)
    engine.reshapeAndCache(cache, k, v, slots, T)
    engine.copyBlocks(cache, src, dst)
    kp = np.zeros((nblk, kvh, bs, D), np.float16)
    vp = np.zeros_like(kp)
    co.reshape_and_cache(k, v, kp, vp, slots, bs)
    co.copy_blocks(kp, vp, src, dst)
    gk, gv, _, _ = cache.readPools()
    assert np.array_equal(gk, kp) and np.array_equal(gv, vp)
    cache.close()
    # FP8
    cache = pam.KVCacheManager(engine, nblk, bs, D, kvh, DT.float8)
    engine.reshapeAndCache(cache, k, v, slots, T)
    engine.copyBlocks(cache, src, dst)
    kc = np.zeros((nblk, kvh, bs, D), np.uint8)
    vc = np.zeros_like(kc)
    ks = np.zeros((nblk, kvh), np.float16)
    vs = np.zeros_like(ks)
    co.reshape_and_cache_fp8(k, v, kc, vc, ks.view(np.uint16), vs.view(np.uint16), slots, bs)
    co.copy_blocks(kc, vc, src, dst)
    po.copy_blocks([ks, vs], src, dst)
    gk, gv, gks, gvs = cache.readPools()
    assert np.array_equal(gk, kc) and np.array_equal(gv, vc)
    assert np.array_equal(gks, ks) and np.array_equal(gvs, vs)
    cache.close()


def test_fp8_codes_of_every_float16_value(engine):
    """quantize_fp8 (kernels.metal:564-601) over every finite float16 value, against group
    scales from 2^-20 to 146: powers of two (where thousands of quotients sit exactly on a
    rounding point of the 3-bit mantissa or of the sub-normal steps) and scales with full
    mantissas.  Each (block, kv_head) group holds 2048 of the 65 536 bit patterns plus the
    value that fixes its absmax; a second append with smaller values then reuses the stored
    scales (max(absmax, scale * 448), kernels.metal:1945-1951).  Codes and scales bit for
    bit against the oracle."""
    kvh, bs, D = 8, 16, 128
    caps = [448.0 * 2.0 ** k for k in (-20, -17, -14, -11, -8, -5, -2, 0, 1, 4, 7)]
    caps += [65504.0, 1000.5, 3.140625, 1.0, 0.333251953125, 6.103515625e-05, 0.00123596191]
    caps = np.asarray(caps, dtype=np.float16)
    patterns = np.arange(65536, dtype=np.uint16).view(np.float16)
    n_sets = len(caps)
    n_blocks = 4 * n_sets                                            # 4 blocks x 8 kv heads = 32 groups of 2048 values
    T = n_blocks * bs
    rng = np.random.default_rng(26)

    def build(order, shrink):
        rows = np.zeros((T, kvh, D), np.float16)
        for s, cap in enumerate(caps):
            vals = patterns[order].copy()
            limit = np.float16(float(cap) * shrink)
            vals[~np.isfinite(vals) | (np.abs(vals.astype(np.float32)) > float(limit))] = np.float16(0)
            groups = vals.reshape(4, kvh, bs, D)                     # [block][kv_head][slot][dim]
            groups[:, :, 0, 0] = limit if s % 2 == 0 else -limit     # the group's absmax
            rows[4 * s * bs:4 * (s + 1) * bs] = np.transpose(groups, (0, 2, 1, 3)).reshape(4 * bs, kvh, D)
        return rows

    k1, v1 = build(np.arange(65536), 1.0), build(rng.permutation(65536), 1.0)
    k2, v2 = build(rng.permutation(65536), 0.5), build(rng.permutation(65536), 0.25)   # below the stored scales
    slots = np.arange(T, dtype=np.int64)
    cache = pam.KVCacheManager(engine, n_blocks, bs, D, kvh, DT.float8)
    kc = np.zeros((n_blocks, kvh, bs, D), np.uint8)
    vc = np.zeros_like(kc)
    ks = np.zeros((n_blocks, kvh), np.uint16)
    vs = np.zeros_like(ks)
    for k, v in ((k1, v1), (k2, v2)):
        engine.reshapeAndCache(cache, k, v, slots, T)
        co.reshape_and_cache_fp8(k, v, kc, vc, ks, vs, slots, bs)
        gk, gv, gks, gvs = cache.readPools()
        assert np.array_equal(gks.view(np.uint16), ks) and np.array_equal(gvs.view(np.uint16), vs)
        assert np.array_equal(gk, kc), f"{np.count_nonzero(gk != kc)} K codes differ"
        assert np.array_equal(gv, vc), f"{np.count_nonzero(gv != vc)} V codes differ"
    assert len(np.unique(ks)) >= n_sets - 1 and np.all(ks != 0)
    cache.close()
