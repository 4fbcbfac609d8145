"""The batched-layer calls (PagedAttentionEngine.swift:1433-1895: appendLayers,
prefillLayers, decodeLayers) on the GPU: every layer must give what the
single-layer call gives, bit for bit, and meet the oracle's bound."""
import numpy as np
import pytest

import pagedattentionmetal_b200 as pam
from gpu_helpers import DT, assert_close, from_io, to_storage
from oracle import c_oracle as co

pytestmark = pytest.mark.gpu

H, KVH, D, BS = 8, 2, 128, 16
LENS = (200, 77, 130)


def _caches(engine, n_layers, dtype):
    """One manager (one pair of pools) per layer, all with the same block tables."""
    caches = [pam.KVCacheManager(engine, 40, BS, D, KVH, dtype) for _ in range(n_layers)]
    for c in caches:
        for s, n in enumerate(LENS):
            c.allocateSequence(s)
            c.appendTokens(s, n)
    tables = [np.asarray(caches[0].getBlockTable(s), dtype=np.int32) for s in range(len(LENS))]
    for c in caches[1:]:
        assert [c.getBlockTable(s) for s in range(len(LENS))] == [t.tolist() for t in tables]
    return caches, tables


def _scales(caches, which):
    return [getattr(c, which) for c in caches]


@pytest.mark.parametrize("dtype", [DT.float16, DT.bfloat16, DT.float8])
def test_layers_equal_single_layer_calls(engine, dtype):
    rng = np.random.default_rng(90 + int(dtype))
    n_layers = 3
    io = DT.float16 if dtype == DT.float8 else dtype
    layers = [pam.PagedLayerSpec(D, H, KVH, BS, dtype) for _ in range(n_layers)]
    rand = lambda *shape: to_storage(rng.standard_normal(shape, dtype=np.float32), io)
    keys = [[rand(n, KVH, D) for n in LENS] for _ in range(n_layers)]
    values = [[rand(n, KVH, D) for n in LENS] for _ in range(n_layers)]

    # ---- append: all layers in one call per sequence, against one call per layer
    batched, tables = _caches(engine, n_layers, dtype)
    single, _ = _caches(engine, n_layers, dtype)
    for s, n in enumerate(LENS):
        engine.appendLayers([keys[l][s] for l in range(n_layers)], [values[l][s] for l in range(n_layers)],
                            [c.kPoolBuffer for c in batched], [c.vPoolBuffer for c in batched], tables[s], 0, n,
                            layers, _scales(batched, "kScaleBuffer"), _scales(batched, "vScaleBuffer"), batched)
        assert engine.lastStats.operation == pam.Operation.append
        for l in range(n_layers):
            engine.appendKV(single[l], s, keys[l][s], values[l][s], 0, n, H)
    pools = [c.readPools() for c in batched]
    for l in range(n_layers):
        for a, b in zip(pools[l], single[l].readPools()):
            assert (a is None) == (b is None)
            if a is not None:
                assert np.array_equal(a.view(np.uint8), b.view(np.uint8))
    assert not np.array_equal(pools[0][0].view(np.uint8), pools[1][0].view(np.uint8))    # layers hold different data

    def scale_bits(l):
        ks, vs = pools[l][2], pools[l][3]
        return (None if ks is None else ks.view(np.uint16)), (None if vs is None else vs.view(np.uint16))

    # ---- prefill of sequence 0 in every layer
    S = LENS[0]
    q = [rand(S, H, D) for _ in range(n_layers)]
    out = [np.zeros_like(q[0]) for _ in range(n_layers)]
    engine.prefillLayers(q, [c.kPoolBuffer for c in batched], [c.vPoolBuffer for c in batched], tables[0], out, S,
                         layers, True, 0, _scales(batched, "kScaleBuffer"), _scales(batched, "vScaleBuffer"))
    for l in range(n_layers):
        one = np.zeros_like(q[l])
        engine.prefill(pam.PagedAttentionPrefillRequest(q[l], batched[l].kPoolBuffer, batched[l].vPoolBuffer,
                                                        tables[0], one, S, layers[l], True,
                                                        batched[l].kScaleBuffer, batched[l].vScaleBuffer))
        assert np.array_equal(out[l].view(np.uint8), one.view(np.uint8))
        ks, vs = scale_bits(l)
        ref = co.prefill(q[l], pools[l][0], pools[l][1], tables[0], S, KVH, BS, int(dtype), causal=True,
                         k_scale=ks, v_scale=vs)
        assert_close(from_io(out[l], dtype), ref, dtype)

    # ---- decode of the three sequences in every layer, with a window on top
    B = len(LENS)
    max_nb = max(len(t) for t in tables)
    bt = np.zeros((B, max_nb), np.int32)
    for s, t in enumerate(tables):
        bt[s, :len(t)] = t
    lens = np.asarray(LENS, np.uint32)
    for window in (0, 64):
        qd = [rand(B, H, D) for _ in range(n_layers)]
        od = [np.zeros_like(qd[0]) for _ in range(n_layers)]
        engine.decodeLayers(qd, [c.kPoolBuffer for c in batched], [c.vPoolBuffer for c in batched], bt, lens, od, B,
                            max_nb, layers, window, _scales(batched, "kScaleBuffer"), _scales(batched, "vScaleBuffer"))
        assert engine.lastStats.operation == pam.Operation.decode
        for l in range(n_layers):
            one = np.zeros_like(qd[l])
            spec = pam.PagedLayerSpec(D, H, KVH, BS, dtype, window)
            engine.decode(pam.PagedAttentionDecodeRequest(qd[l], batched[l].kPoolBuffer, batched[l].vPoolBuffer, bt, lens,
                                                          one, B, max_nb, spec, batched[l].kScaleBuffer,
                                                          batched[l].vScaleBuffer))
            assert np.array_equal(od[l].view(np.uint8), one.view(np.uint8))
            ks, vs = scale_bits(l)
            ref = co.decode(qd[l], pools[l][0], pools[l][1], bt, lens, KVH, BS, int(dtype), window=window,
                            k_scale=ks, v_scale=vs)
            assert_close(from_io(od[l], dtype), ref, dtype)
    for c in batched + single:
        c.close()


def test_layers_shared_pool_like_the_reference(engine):
    """The reference hands every layer the same kPool / vPool
    (PagedAttentionEngine.swift:1436-1437): a single buffer stands for all layers."""
    rng = np.random.default_rng(95)
    (cache,), tables = _caches(engine, 1, DT.float16)
    k = rng.standard_normal((LENS[0], KVH, D)).astype(np.float16)
    v = rng.standard_normal((LENS[0], KVH, D)).astype(np.float16)
    engine.appendKV(cache, 0, k, v, 0, LENS[0], H)
    layers = [pam.PagedLayerSpec(D, H, KVH, BS, DT.float16), pam.PagedLayerSpec(D, 4, KVH, BS, DT.float16)]
    q = [rng.standard_normal((LENS[0], l.numHeads, D)).astype(np.float16) for l in layers]
    out = [np.zeros_like(x) for x in q]
    engine.prefillLayers(q, cache.kPoolBuffer, cache.vPoolBuffer, tables[0], out, LENS[0], layers)
    kp, vp, _, _ = cache.readPools()
    for l, spec in enumerate(layers):
        ref = co.prefill(q[l], kp, vp, tables[0], LENS[0], KVH, BS, int(DT.float16), causal=True)
        assert_close(out[l].astype(np.float32), ref, DT.float16)
    cache.close()


def test_layers_count_mismatch(engine):
    """PagedAttentionEngine.swift:1445-1447, 1652-1654, 1757-1759"""
    layers = [pam.PagedLayerSpec(D, H, KVH, BS, DT.float16)] * 2
    buf = np.zeros((4, H, D), np.float16)
    t = np.zeros(1, np.int32)
    with pytest.raises(pam.PagedAttentionError, match="buffer/layer count mismatch"):
        engine.prefillLayers([buf], buf, buf, t, [buf, buf], 4, layers)
    with pytest.raises(pam.PagedAttentionError, match="buffer/layer count mismatch"):
        engine.decodeLayers([buf, buf], buf, buf, t, np.zeros(1, np.uint32), [buf], 1, 1, layers)
    with pytest.raises(pam.PagedAttentionError, match="buffer/layer count mismatch"):
        engine.appendLayers([buf], [buf, buf], buf, buf, t, 0, 4, layers)
    with pytest.raises(pam.PagedAttentionError, match="buffer/layer count mismatch"):
        engine.decodeLayers([], buf, buf, t, np.zeros(1, np.uint32), [], 1, 1, [])
