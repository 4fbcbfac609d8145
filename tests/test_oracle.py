"""The oracle against the reference's own outputs and known facts (CPU only)."""
import hashlib
import os

import numpy as np
import pytest

from oracle import c_oracle as co
from oracle import paged_oracle as po


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_sim_selfcheck_vector(golden_dir):
    # The reference's own self-check case (Reference/paged_attention_sim.py:143-176):
    # one head, no softmax scale, not causal, queries == keys.
    g = _load(golden_dir, "sim_selfcheck.npz")
    q = g["q"][:, None, :] * np.sqrt(np.float32(8))          # undo the 1/sqrt(d) the oracle applies
    kp, vp = g["k_pool"][:, None], g["v_pool"][:, None]
    out = po.paged_prefill(q, kp, vp, g["table"], 8, 1, 4, causal=False)
    assert np.abs(out[:, 0] - g["out"]).max() < 1e-5
    out_c = co.prefill(q.astype(np.float32), kp, vp, g["table"], 8, 1, 4, po.DT_F32, causal=False)
    assert np.abs(out_c[:, 0] - g["out"]).max() < 1e-5


@pytest.mark.parametrize("online", [False, True])
def test_decode_small_vs_sim(golden_dir, online):
    g = _load(golden_dir, "decode_small.npz")
    out = po.paged_decode(g["q"], g["k_pool"], g["v_pool"], g["tables"], g["lens"], 2, 16, online=online)
    assert np.abs(out - g["out"]).max() < 1e-5


def test_c_decode_small_vs_sim(golden_dir):
    g = _load(golden_dir, "decode_small.npz")
    out = co.decode(g["q"], g["k_pool"], g["v_pool"], g["tables"], g["lens"], 2, 16, po.DT_F32)
    assert np.abs(out - g["out"]).max() < 1e-5


def c0_inputs():
    """The CPU-runnable benchmark configuration, regenerated from its seed."""
    rng, lens, tables, n_pool = po.make_decode_case(1000, batch=8, len_lo=1, len_hi=512, heads=32, kv_heads=8,
                                                    head_dim=128, block_size=16, pool_blocks=256)
    k_pool = np.zeros((n_pool, 8, 16, 128), dtype=np.float32)
    v_pool = np.zeros_like(k_pool)
    for b in range(8):
        L = int(lens[b])
        k = rng.standard_normal((L, 8, 128), dtype=np.float32)
        v = rng.standard_normal((L, 8, 128), dtype=np.float32)
        po.reshape_and_cache(k_pool, v_pool, k, v, po.slot_mapping(tables[b], 0, L, 16), 16)
    q = rng.standard_normal((8, 32, 128), dtype=np.float32)
    return q, k_pool, v_pool, tables, lens


def test_decode_c0_vs_sim(golden_dir):
    g = _load(golden_dir, "decode_c0.npz")
    q, k_pool, v_pool, tables, lens = c0_inputs()
    h = hashlib.sha256()
    for a in (q, k_pool, v_pool):
        h.update(np.ascontiguousarray(a).tobytes())
    assert h.hexdigest() == str(g["inputs_sha256"]), "seeded inputs differ from the ones the golden outputs were made from"
    assert np.array_equal(tables, g["tables"]) and np.array_equal(lens, g["lens"])
    out = co.decode(q, k_pool, v_pool, tables, lens, 8, 16, po.DT_F32)
    assert np.abs(out - g["out"]).max() <= 2e-3          # the stated tolerance; measured ~1e-6
    assert np.abs(out - g["out"]).max() < 1e-5
    out_np = po.paged_decode(q, k_pool, v_pool, tables, lens, 8, 16)
    assert np.abs(out_np - g["out"]).max() < 1e-5


def test_prefill_small_vs_sim(golden_dir):
    g = _load(golden_dir, "prefill_small.npz")
    args = (g["q"], g["k_pool"], g["v_pool"], g["table"], 40, 2, 8)
    assert np.abs(po.paged_prefill(*args, causal=False) - g["out_full"]).max() < 1e-5
    assert np.abs(po.paged_prefill(*args, causal=True) - g["out_causal"]).max() < 1e-5
    assert np.abs(co.prefill(*args, po.DT_F32, causal=False) - g["out_full"]).max() < 1e-5
    assert np.abs(co.prefill(*args, po.DT_F32, causal=True) - g["out_causal"]).max() < 1e-5
    # a chunk of rows equals the same rows of the full result (Engine.swift:740-756)
    chunk = co.prefill(g["q"][8:24], g["k_pool"], g["v_pool"], g["table"], 40, 2, 8, po.DT_F32, causal=True, q_start=8)
    assert np.abs(chunk - g["out_causal"][8:24]).max() < 1e-5


def test_window_decode_vs_sim(golden_dir):
    """Sliding-window decode against the reference's numpy implementation run over tokens
    [L - W, L) re-packed into fresh blocks (tests/golden/make_golden.py, case 5)."""
    g = _load(golden_dir, "decode_window.npz")
    for wi, w in enumerate(g["windows"]):
        args = (g["q"], g["k_pool"], g["v_pool"], g["tables"], g["lens"], 2, 16)
        assert np.abs(co.decode(*args, po.DT_F32, window=int(w)) - g["out"][wi]).max() < 1e-5
        for online in (False, True):
            assert np.abs(po.paged_decode(*args, window=int(w), online=online) - g["out"][wi]).max() < 1e-5
    # the windows really cut: the unwindowed result differs
    full = co.decode(g["q"], g["k_pool"], g["v_pool"], g["tables"], g["lens"], 2, 16, po.DT_F32)
    assert np.abs(full - g["out"][0]).max() > 1e-2


def test_window_prefill_vs_sim(golden_dir):
    """Prefill with a block-aligned window start against the same (case 6): rows below the
    window start see no key when causal (0/0 in the reference) and are not compared."""
    g = _load(golden_dir, "prefill_window.npz")
    S, W = g["q"].shape[0], int(g["window"])
    ws = S - W
    args = (g["q"], g["k_pool"], g["v_pool"], g["table"], S, 2, 8)
    seen = ~np.isnan(g["out_causal"])
    assert seen[ws:].all() and not seen[:ws].any()
    for causal, want in ((False, g["out_full"]), (True, g["out_causal"])):
        for got in (po.paged_prefill(*args, causal=causal, window_start=ws),
                    co.prefill(*args, po.DT_F32, causal=causal, window_start=ws)):
            mask = ~np.isnan(want)
            assert np.abs(got[mask] - want[mask]).max() < 1e-5
    chunk = co.prefill(g["q"][40:56], g["k_pool"], g["v_pool"], g["table"], S, 2, 8, po.DT_F32, causal=True,
                       window_start=ws, q_start=40)
    assert np.abs(chunk - g["out_causal"][40:56]).max() < 1e-5


def test_window_decode_np_vs_c():
    rng, lens, tables, n_pool = po.make_decode_case(3, 4, 30, 90, 4, 2, head_dim=16, block_size=8, spare_blocks=2)
    k_pool = rng.standard_normal((n_pool, 2, 8, 16), dtype=np.float32)
    v_pool = rng.standard_normal((n_pool, 2, 8, 16), dtype=np.float32)
    q = rng.standard_normal((4, 4, 16), dtype=np.float32)
    for w in (0, 5, 16, 33, 200):
        a = po.paged_decode(q, k_pool, v_pool, tables, lens, 2, 8, window=w, online=True)
        b = co.decode(q, k_pool, v_pool, tables, lens, 2, 8, po.DT_F32, window=w)
        assert np.abs(a - b).max() < 1e-5
        # windowed decode == full decode over the last w tokens only
        if 0 < w < 30:
            L = int(lens[0])
            kk = po._gather_kv(k_pool, tables[0], 0, L, 8)[L - w:]
            vv = po._gather_kv(v_pool, tables[0], 0, L, 8)[L - w:]
            s = kk @ q[0, 0] / np.sqrt(np.float32(16))
            p = np.exp(s - s.max())
            assert np.abs(p @ vv / p.sum() - a[0, 0]).max() < 1e-5


# ---- FP8 codec (kernels.metal:553-601): source-pinned facts ----

def test_fp8_quantize_known_answers():
    q = lambda v, s=1.0: int(po.quantize_fp8(np.float16(v), np.float16(s)))
    assert q(0.0) == 0x00 and q(-0.0) == 0x00                  # :571, sign from v < 0
    assert q(1.0) == 0x38 and q(-1.0) == 0xB8
    assert q(448.0) == 0x7E and q(1000.0) == 0x7E and q(-1000.0) == 0xFE   # clamp, :566
    assert q(136.0) == 0x71                                    # tie rounds away from zero (RNE gives 0x70)
    assert q(3.125) == 0x45 and q(-0.1328) == 0xA1
    assert q(2.0 ** -9) == 0x01 and q(2.0 ** -10) == 0x01      # round(0.5) = 1 (half away)
    assert q(-(2.0 ** -12)) == 0x80                            # rounds to mantissa 0, keeps the sign bit
    assert q(0.015625 * 0.999) == 0x07                         # subnormal branch caps at 7, no promotion (:575)
    assert q(464.0) == 0x7E


def test_fp8_codec_c_matches_numpy_exhaustively():
    allh = np.arange(65536, dtype=np.uint32).astype(np.uint16).view(np.float16)
    allh = allh[np.isfinite(allh)]
    for s in (1.0, 0.0123, 0.5, 3e-3, 7.0):
        s = np.float16(s)
        assert np.array_equal(po.quantize_fp8(allh, s), co.quantize_fp8(allh, s))
    codes = np.arange(256, dtype=np.uint8)
    rng = np.random.default_rng(5)
    for s in list(rng.uniform(1e-4, 3, 40).astype(np.float16)) + [np.float16(1), np.float16(6e-5), np.float16(100)]:
        a = po.dequant_fp8(codes, s).astype(np.float32)
        b = co.dequant_fp8(codes, s)
        assert np.array_equal(a, b)


def test_fp8_dequant_known_answers():
    d = lambda c, s=1.0: float(po.dequant_fp8(np.uint8(c), np.float16(s)))
    assert d(0x00) == 0.0 and d(0x80) == 0.0
    assert d(0x38) == 1.0 and d(0xB8) == -1.0 and d(0x7E) == 448.0
    assert d(0x7F) == 480.0                                    # not a NaN in the reference codec
    assert d(0x01) == 2.0 ** -9 and d(0x07) == 7 * 2.0 ** -9
    assert d(0x40, 0.5) == 1.0


def test_fp8_scale_rule():
    s = po.fp8_scale_update(np.float32(0.0), np.float16(0.0))
    assert s == np.float16(1.0)                                # metal:1953, nothing seen yet
    s1 = po.fp8_scale_update(np.float32(4.0), np.float16(0.0))
    assert s1 == np.float16(np.float32(4.0) / np.float32(448.0))
    # a smaller later absmax keeps (a fixed point of) the old scale
    s2 = po.fp8_scale_update(np.float32(1.0), s1)
    assert po.fp8_scale_update(np.float32(1.0), s2) == s2
    # reading the already updated scale gives the same result (the shader's benign race)
    rng = np.random.default_rng(0)
    amax = rng.uniform(0, 8, 2000).astype(np.float32)
    old = rng.uniform(0, 0.02, 2000).astype(np.float16)
    new = po.fp8_scale_update(amax, old)
    assert np.array_equal(po.fp8_scale_update(amax, new), new)


def test_fp8_append_c_matches_numpy():
    rng = np.random.default_rng(1)
    T, KVH, D, bs, NB = 300, 4, 32, 16, 40
    k = rng.standard_normal((T, KVH, D)).astype(np.float16)
    v = rng.standard_normal((T, KVH, D)).astype(np.float16)
    slots = rng.choice(NB * bs, T, replace=False)

    def run(fn):
        kc = np.zeros((NB, KVH, bs, D), np.uint8)
        vc = np.zeros_like(kc)
        ks = np.zeros((NB, KVH), np.float16)
        vs = np.zeros_like(ks)
        fn(kc, vc, ks, vs, k[:200], v[:200], slots[:200])
        fn(kc, vc, ks, vs, k[200:], v[200:], slots[200:])
        return kc, vc, ks, vs

    a = run(lambda kc, vc, ks, vs, k_, v_, s: po.reshape_and_cache_fp8(kc, vc, ks, vs, k_, v_, s, bs))
    b = run(lambda kc, vc, ks, vs, k_, v_, s: co.reshape_and_cache_fp8(k_, v_, kc, vc, ks.view(np.uint16), vs.view(np.uint16), s, bs))
    for x, y in zip(a, b):
        assert np.array_equal(x, y)
    # one call on empty groups: dequantised values stay within half a code step
    # (1/16 relative) of the input
    kc = np.zeros((NB, KVH, bs, D), np.uint8)
    vc = np.zeros_like(kc)
    ks = np.zeros((NB, KVH), np.float16)
    vs = np.zeros_like(ks)
    po.reshape_and_cache_fp8(kc, vc, ks, vs, k, v, slots, bs)
    blk, off = slots // bs, slots % bs
    deq = po.dequant_fp8(kc[blk, :, off, :], ks[blk][:, :, None]).astype(np.float32)
    kf = k.astype(np.float32)
    assert np.all(np.abs(deq - kf) <= np.abs(kf) / 16 + ks[blk].astype(np.float32)[:, :, None] * 2.0 ** -9 + 1e-6)


def test_slot_mapping_formula():
    table = [7, 2, 9]
    s = po.slot_mapping(table, 5, 19, 8)                       # kernels.metal:1823-1827
    assert list(s[:3]) == [7 * 8 + 5, 7 * 8 + 6, 7 * 8 + 7]
    assert s[3] == 2 * 8 and s[11] == 9 * 8 and s[-1] == 9 * 8 + 7


def test_copy_blocks_np_vs_c():
    rng = np.random.default_rng(2)
    k = rng.standard_normal((12, 2, 4, 8)).astype(np.float16)
    v = rng.standard_normal((12, 2, 4, 8)).astype(np.float16)
    k2, v2 = k.copy(), v.copy()
    src, dst = [1, 5, 7], [0, 2, 11]
    po.copy_blocks([k, v], src, dst)
    co.copy_blocks(k2, v2, src, dst)
    assert np.array_equal(k, k2) and np.array_equal(v, v2)
    assert np.array_equal(k[0], k[1]) and np.array_equal(v[11], v[7])


def test_inference_state_machine_hand_checked():
    """OracleInference (PagedAttentionInference.swift:119-299).  The reference has no test
    of this class, so the restatement is checked against a run worked out by hand from the
    source: batch of 3, prompts (40, 3 new), (17, 1), (100, 5), (5, 2), (64, 4)."""
    ora = po.OracleInference(64, 16, 3)
    for prompt, new in ((40, 3), (17, 1), (100, 5), (5, 2), (64, 4)):
        ora.add_request(prompt, new)
    # step 1: the first three waiting sequences are prefilled (3 + 2 + 7 blocks), nothing decodes
    assert ora.step() == [0, 1, 2]
    assert [l[0] for l in ora.launches] == ["prefill"] * 3
    assert ora.cache.available_blocks == 64 - 12 and ora.total_tokens == 157 and ora.tokens == []
    # step 2: waiting sequences come first (Scheduler.swift:90-95), one running one fits
    assert ora.step() == [3, 4, 0]
    assert ora.launches[-1] == ("decode", [0], [40], [ora.cache.block_table(0)])
    assert ora.cache.sequence_length(0) == 41 and ora.tokens == [(0, 0)]
    # step 3: all five are running, the first three by arrival decode; sequence 1 is done
    assert ora.step() == [0, 1, 2]
    assert ora.sched.seqs[1]["status"] == po.COMPLETED and 1 not in ora.cache.sequences
    ora.run_all()
    assert ora.step_count == 8 and ora.total_tokens == 226 + 15 and len(ora.tokens) == 15
    assert ora.cache.available_blocks == 64 and ora.sched.count(po.COMPLETED) == 5


def test_inference_memory_pressure_policies():
    """ensureBlocksAvailable (PagedAttentionInference.swift:280-299): the free count handed to
    handleMemoryPressure is read once, so every running sequence is paused; the incremental
    option pauses one at a time (newest first, the sequence being prefilled included, since
    the scheduler's step has already promoted it)."""
    for incremental, paused, new_one in ((False, [0, 1, 2], po.RUNNING), (True, [2], po.PAUSED)):
        ora = po.OracleInference(14, 16, 4, 128, incremental)
        for _ in range(3):
            ora.add_request(48, 8)
        assert ora.step() == [0, 1, 2] and ora.step() == [0, 1, 2]
        assert ora.cache.available_blocks == 2
        ora.add_request(90, 2)
        with pytest.raises(po.SequenceNotFound):       # a victim was part of the same batch
            ora.step()
        assert [i for i in range(3) if ora.sched.seqs[i]["status"] == po.PAUSED] == paused
        # incremental: the decode of the same step needs one more block for the sequence whose
        # pages are gone (its length falls back to the prompt's, :226-231), and the newest
        # running sequence, the one just prefilled, pays for it
        assert ora.sched.seqs[3]["status"] == new_one and (3 in ora.prefilled) == (new_one == po.RUNNING)
    ora = po.OracleInference(4, 16, 2)
    ora.add_request(200, 1)
    with pytest.raises(po.OutOfMemory):
        ora.step()


def test_backward_formulas_match_autograd():
    """The backward restatement (kernels.metal:1217-1315 as dense algebra) against the gradient
    that automatic differentiation of softmax(q k^T / sqrt(d)) v gives, in float64, over a
    paged cache with a window: the reference has no test of its backward kernels, so this is
    what pins the oracle's formulas (not the reference's arithmetic order)."""
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(5)
    L, H, KVH, D, bs = 37, 4, 2, 16, 8
    nb = (L + bs - 1) // bs
    table = rng.permutation(nb + 3)[:nb].astype(np.int32)
    kp = rng.standard_normal((nb + 3, KVH, bs, D)).astype(np.float32)
    vp = rng.standard_normal((nb + 3, KVH, bs, D)).astype(np.float32)
    q = rng.standard_normal((L, H, D)).astype(np.float32)
    d_out = rng.standard_normal((L, H, D)).astype(np.float32)
    for ws in (0, 10):
        m, l = po.attention_stats(q, kp, table, L, KVH, bs, ws)
        dq, dk, dv = po.paged_backward(q, kp, vp, table, d_out, m, l, L, KVH, bs, ws)
        tq = torch.tensor(q, dtype=torch.float64, requires_grad=True)
        tk = torch.tensor(kp, dtype=torch.float64, requires_grad=True)
        tv = torch.tensor(vp, dtype=torch.float64, requires_grad=True)
        toks = np.arange(ws, L)
        blk, slot = torch.tensor(table[toks // bs].astype(np.int64)), torch.tensor(toks % bs)
        heads = []
        for h in range(H):
            kvh = h // (H // KVH)
            s = (tq[:, h] @ tk[blk, kvh, slot].T) / float(np.sqrt(np.float32(D)))
            heads.append(torch.softmax(s, dim=1) @ tv[blk, kvh, slot])
        (torch.stack(heads, dim=1) * torch.tensor(d_out, dtype=torch.float64)).sum().backward()
        assert np.abs(dq - tq.grad.numpy()).max() < 1e-6
        assert np.abs(dk - tk.grad.numpy()).max() < 1e-6
        assert np.abs(dv - tv.grad.numpy()).max() < 1e-6
