"""Generate the golden vectors under tests/golden/ from the reference's own
numpy implementation (Reference/paged_attention_sim.py, imported unchanged).

Run once, in a checkout that has the reference project next to it:

    python tests/golden/make_golden.py /path/to/PagedAttentionMetal

The reference function handles one head, applies no softmax scale, is not
causal and takes ``q.shape[0]`` as both the number of queries and the number
of keys.  A decode over a context of L tokens is therefore obtained by tiling
the pre-scaled query to L rows and keeping row 0; a causal prefill row i is the
same call over the first i+1 keys.  The stored outputs are what that function
returned; the tests compare the oracle (and, on a GPU, the CUDA kernels)
against them.
"""
from __future__ import annotations

import contextlib
import hashlib
import importlib.util
import io
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from oracle import paged_oracle as po  # noqa: E402


def load_sim(ref_root: str):
    path = os.path.join(ref_root, "Reference", "paged_attention_sim.py")
    spec = importlib.util.spec_from_file_location("paged_attention_sim", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def sim_call(sim, q, k_pool, v_pool, table, bs, hd):
    with contextlib.redirect_stdout(io.StringIO()):
        out, _, _ = sim.paged_attention_forward(q, k_pool, v_pool, table, block_size=bs, head_dim=hd)
    return out


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def sim_decode(sim, q, k_pool, v_pool, tables, lens, kvh_count, bs):
    """q [B][H][D] f32; pools [blocks][KVH][bs][D] f32 -> [B][H][D] f64."""
    B, H, D = q.shape
    G = H // kvh_count
    inv = np.float32(1.0) / np.sqrt(np.float32(D))
    out = np.zeros((B, H, D), dtype=np.float64)
    for b in range(B):
        L = int(lens[b])
        nb = (L + bs - 1) // bs
        table = tables[b, :nb]
        for h in range(H):
            kvh = h // G
            kp = np.ascontiguousarray(k_pool[:, kvh])
            vp = np.ascontiguousarray(v_pool[:, kvh])
            qs = np.tile((q[b, h] * inv)[None, :], (L, 1))
            out[b, h] = sim_call(sim, qs, kp, vp, table, bs, D)[0]
    return out


def fill_pools(rng, n_pool, kvh, bs, hd, tables, lens, dtype=po.DT_F32):
    """Write N(0,1) K/V for every live token through the block tables."""
    k_pool = np.zeros((n_pool, kvh, bs, hd), dtype=np.float32)
    v_pool = np.zeros((n_pool, kvh, bs, hd), dtype=np.float32)
    for b in range(len(lens)):
        L = int(lens[b])
        k = po.round_to(rng.standard_normal((L, kvh, hd), dtype=np.float32), dtype)
        v = po.round_to(rng.standard_normal((L, kvh, hd), dtype=np.float32), dtype)
        slots = po.slot_mapping(tables[b], 0, L, bs)
        po.reshape_and_cache(k_pool, v_pool, k, v, slots, bs)
    return k_pool, v_pool


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <checkout of the reference project>")
    ref_root = sys.argv[1]
    sim = load_sim(ref_root)

    # 1. The reference's own self-check case (sim:143-176): seed 42, S=8,
    #    block 4, dim 8, 16 physical blocks, table [3, 7].
    np.random.seed(42)
    q = np.random.randn(8, 8).astype(np.float32)
    k_pool = np.random.randn(16, 4, 8).astype(np.float32)
    v_pool = np.random.randn(16, 4, 8).astype(np.float32)
    table = np.array([3, 7], dtype=np.int32)
    out = sim_call(sim, q, k_pool, v_pool, table, 4, 8)
    np.savez(os.path.join(HERE, "sim_selfcheck.npz"), q=q, k_pool=k_pool, v_pool=v_pool,
             table=table, out=out)

    # 2. Small decode case, inputs stored in full.
    rng, lens, tables, n_pool = po.make_decode_case(7, batch=5, len_lo=1, len_hi=70, heads=8,
                                                    kv_heads=2, head_dim=32, block_size=16,
                                                    spare_blocks=3)
    k_pool, v_pool = fill_pools(rng, n_pool, 2, 16, 32, tables, lens)
    q = rng.standard_normal((5, 8, 32), dtype=np.float32)
    out = sim_decode(sim, q, k_pool, v_pool, tables, lens, 2, 16)
    np.savez(os.path.join(HERE, "decode_small.npz"), q=q, k_pool=k_pool, v_pool=v_pool,
             tables=tables, lens=lens, out=out)

    # 3. The CPU-runnable benchmark configuration: 8 sequences, lengths in
    #    [1, 512], 32 query / 8 KV heads, dim 128, block 16, pool of 256 blocks,
    #    seed 1000.  Inputs are regenerated from the seed by the tests (their
    #    SHA-256 is stored); outputs are stored.
    rng, lens, tables, n_pool = po.make_decode_case(1000, batch=8, len_lo=1, len_hi=512, heads=32,
                                                    kv_heads=8, head_dim=128, block_size=16,
                                                    pool_blocks=256)
    k_pool, v_pool = fill_pools(rng, n_pool, 8, 16, 128, tables, lens)
    q = rng.standard_normal((8, 32, 128), dtype=np.float32)
    out = sim_decode(sim, q, k_pool, v_pool, tables, lens, 8, 16)
    np.savez(os.path.join(HERE, "decode_c0.npz"), tables=tables, lens=lens,
             out=out.astype(np.float32), inputs_sha256=np.array(digest(q, k_pool, v_pool)))

    # 4. Small prefill case: S=40, block 8, dim 16, 4 query / 2 KV heads, both
    #    non-causal (one call per head) and causal (one call per row and head).
    rng = np.random.default_rng(11)
    S, bs, hd, H, KVH = 40, 8, 16, 4, 2
    nb = (S + bs - 1) // bs
    table = rng.permutation(9)[:nb].astype(np.int32)
    k_pool = rng.standard_normal((9, KVH, bs, hd), dtype=np.float32)
    v_pool = rng.standard_normal((9, KVH, bs, hd), dtype=np.float32)
    q = rng.standard_normal((S, H, hd), dtype=np.float32)
    inv = np.float32(1.0) / np.sqrt(np.float32(hd))
    full = np.zeros((S, H, hd))
    caus = np.zeros((S, H, hd))
    for h in range(H):
        kvh = h // (H // KVH)
        kp, vp = np.ascontiguousarray(k_pool[:, kvh]), np.ascontiguousarray(v_pool[:, kvh])
        full[:, h] = sim_call(sim, q[:, h] * inv, kp, vp, table, bs, hd)
        for i in range(S):
            n = i + 1
            qs = np.tile((q[i, h] * inv)[None, :], (n, 1))
            caus[i, h] = sim_call(sim, qs, kp, vp, table[: (n + bs - 1) // bs], bs, hd)[0]
    np.savez(os.path.join(HERE, "prefill_small.npz"), q=q, k_pool=k_pool, v_pool=v_pool,
             table=table, out_full=full, out_causal=caus)
    # 5. Sliding-window decode (kernels.metal:1442, 1464: keys [L - W, L) when L > W).  The
    #    reference function has no window argument; the same arithmetic over the same token
    #    set is obtained by re-packing tokens [ws, L) of a sequence into fresh blocks and
    #    calling it on those.  Windows that do and do not start on a block boundary.
    rng, lens, tables, n_pool = po.make_decode_case(21, batch=6, len_lo=20, len_hi=200, heads=8,
                                                    kv_heads=2, head_dim=32, block_size=16,
                                                    spare_blocks=2)
    k_pool, v_pool = fill_pools(rng, n_pool, 2, 16, 32, tables, lens)
    q = rng.standard_normal((6, 8, 32), dtype=np.float32)
    windows = np.array([48, 50, 1, 16, 500], dtype=np.int32)
    outs = np.zeros((len(windows), 6, 8, 32), dtype=np.float64)
    for wi, W in enumerate(windows):
        for b in range(6):
            L = int(lens[b])
            ws = L - int(W) if L > int(W) else 0
            n = L - ws
            slots = po.slot_mapping(tables[b], ws, n, 16)
            # tokens [ws, L) of every KV head, in order, into blocks 0, 1, ... of a fresh pool
            nb = (n + 15) // 16
            kp = np.zeros((nb, 2, 16, 32), dtype=np.float32)
            vp = np.zeros_like(kp)
            for t, slot in enumerate(slots):
                kp[t // 16, :, t % 16] = k_pool[slot // 16, :, slot % 16]
                vp[t // 16, :, t % 16] = v_pool[slot // 16, :, slot % 16]
            outs[wi, b] = sim_decode(sim, q[b:b + 1], kp, vp, np.arange(nb, dtype=np.int32)[None, :],
                                     np.array([n]), 2, 16)[0]
    np.savez(os.path.join(HERE, "decode_window.npz"), q=q, k_pool=k_pool, v_pool=v_pool, tables=tables,
             lens=lens, windows=windows, out=outs)

    # 6. Prefill with a window that starts on a block boundary (the only case in which the
    #    reference's loop reads the keys it labels, kernels.metal:734-746): S = 64, block 8,
    #    window 40, so window_start = 24.  Non-causal rows see keys [24, 64); causal row
    #    i >= 24 sees keys [24, i]; causal rows below 24 see nothing (0/0 in the reference),
    #    stored as NaN.
    rng = np.random.default_rng(23)
    S, bs, hd, H, KVH, W = 64, 8, 16, 4, 2, 40
    ws = S - W
    nb = S // bs
    table = rng.permutation(10)[:nb].astype(np.int32)
    k_pool = rng.standard_normal((10, KVH, bs, hd), dtype=np.float32)
    v_pool = rng.standard_normal((10, KVH, bs, hd), dtype=np.float32)
    q = rng.standard_normal((S, H, hd), dtype=np.float32)
    inv = np.float32(1.0) / np.sqrt(np.float32(hd))
    wtable = table[ws // bs:]                      # the pages of tokens [ws, S), already block aligned
    full = np.zeros((S, H, hd))
    caus = np.full((S, H, hd), np.nan)
    for h in range(H):
        kvh = h // (H // KVH)
        kp, vp = np.ascontiguousarray(k_pool[:, kvh]), np.ascontiguousarray(v_pool[:, kvh])
        for i in range(S):
            qs = np.tile((q[i, h] * inv)[None, :], (W, 1))
            full[i, h] = sim_call(sim, qs, kp, vp, wtable, bs, hd)[0]
            if i >= ws:
                n = i + 1 - ws
                qs = np.tile((q[i, h] * inv)[None, :], (n, 1))
                caus[i, h] = sim_call(sim, qs, kp, vp, wtable[: (n + bs - 1) // bs], bs, hd)[0]
    np.savez(os.path.join(HERE, "prefill_window.npz"), q=q, k_pool=k_pool, v_pool=v_pool, table=table,
             window=np.array(W), out_full=full, out_causal=caus)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
