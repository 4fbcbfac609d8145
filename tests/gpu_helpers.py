"""Shared helpers of the GPU parity tests: seeded cases in every storage type,
upload to the device, and the matching oracle call."""
import numpy as np

import pagedattentionmetal_b200 as pam
from oracle import c_oracle as co
from oracle import paged_oracle as po

DT = pam.PagedAttentionDataType
TOL = {DT.float32: 2e-3, DT.float16: 2e-3, DT.bfloat16: 2e-3, DT.float8: 1e-2}   # max-abs, from the build contract


def to_storage(x32, dtype):
    """float32 -> (storage array, io array type) for a dtype."""
    if dtype == DT.float32:
        return x32.astype(np.float32)
    if dtype == DT.float16 or dtype == DT.float8:
        return x32.astype(np.float16)
    return po.to_bf16_bits(x32)


def from_io(a, dtype):
    if dtype == DT.bfloat16:
        return po.from_bf16_bits(a)
    return a.astype(np.float32)


def io_numpy_dtype(dtype):
    return {DT.float32: np.float32, DT.float16: np.float16, DT.float8: np.float16, DT.bfloat16: np.uint16}[dtype]


def quantize_pool(pool32):
    """[blocks][kvh][bs][d] float32 -> e4m3 codes + float16 scales [blocks][kvh]
    with the reference codec (absmax / 448 per group)."""
    h = pool32.astype(np.float16)
    amax = np.abs(h.astype(np.float32)).max(axis=(2, 3))
    scale = po.fp8_scale_update(amax, np.zeros_like(amax, dtype=np.float16))
    codes = po.quantize_fp8(h, scale[:, :, None, None])
    return codes, scale


class DecodeCase:
    def __init__(self, seed, batch, lo, hi, heads, kv_heads, head_dim, block_size, dtype, spare=3, poison=True,
                 lens=None):
        rng, self.lens, self.tables, self.n_pool = po.make_decode_case(seed, batch, lo, hi, heads, kv_heads,
                                                                       head_dim, block_size, spare_blocks=spare)
        if lens is not None:
            # fixed lengths: rebuild tables for them
            self.lens = np.asarray(lens, dtype=np.uint32)
            nblk = (self.lens.astype(np.int64) + block_size - 1) // block_size
            self.n_pool = int(nblk.sum()) + spare
            perm = rng.permutation(self.n_pool).astype(np.int32)
            self.tables = np.zeros((batch, max(int(nblk.max()), 1)), dtype=np.int32)
            o = 0
            for i in range(batch):
                self.tables[i, : nblk[i]] = perm[o: o + nblk[i]]
                o += int(nblk[i])
        self.dtype, self.heads, self.kv_heads, self.head_dim, self.block_size = dtype, heads, kv_heads, head_dim, block_size
        shape = (self.n_pool, kv_heads, block_size, head_dim)
        k32 = rng.standard_normal(shape, dtype=np.float32)
        v32 = rng.standard_normal(shape, dtype=np.float32)
        self.k_scale = self.v_scale = None
        if dtype == DT.float8:
            self.k_pool, self.k_scale = quantize_pool(k32)
            self.v_pool, self.v_scale = quantize_pool(v32)
        else:
            self.k_pool, self.v_pool = to_storage(k32, dtype), to_storage(v32, dtype)
            if poison:
                # slots past the end of each sequence hold NaN: they must never reach the result
                nan = to_storage(np.full(1, np.nan, dtype=np.float32), dtype)[0]
                for b in range(batch):
                    L = int(self.lens[b])
                    if L % block_size:
                        blk = self.tables[b, L // block_size]
                        self.k_pool[blk, :, L % block_size:, :] = nan
                        self.v_pool[blk, :, L % block_size:, :] = nan
        self.q = to_storage(rng.standard_normal((batch, heads, head_dim), dtype=np.float32), dtype)

    def layer(self, window=0):
        return pam.PagedLayerSpec(self.head_dim, self.heads, self.kv_heads, self.block_size, self.dtype, window)

    def oracle(self, window=0):
        ks = None if self.k_scale is None else self.k_scale.view(np.uint16)
        vs = None if self.v_scale is None else self.v_scale.view(np.uint16)
        return co.decode(self.q, self.k_pool, self.v_pool, self.tables, self.lens, self.kv_heads, self.block_size,
                         int(self.dtype), window=window, k_scale=ks, v_scale=vs)

    def run(self, engine, window=0, host_io=False):
        """Flat decode through pamc_decode; pools on the device, q/out on the
        device or (host_io) staged from host arrays by the library."""
        kp, vp = engine.makeBufferFrom(self.k_pool), engine.makeBufferFrom(self.v_pool)
        ks = engine.makeBufferFrom(self.k_scale) if self.k_scale is not None else None
        vs = engine.makeBufferFrom(self.v_scale) if self.v_scale is not None else None
        out_host = np.zeros(self.q.shape, dtype=io_numpy_dtype(self.dtype))
        if host_io:
            q, out, tables, lens = self.q, out_host, self.tables, self.lens
        else:
            q, out = engine.makeBufferFrom(self.q), engine.makeBuffer(out_host.nbytes)
            tables, lens = engine.makeBufferFrom(self.tables), engine.makeBufferFrom(self.lens)
        req = pam.PagedAttentionDecodeRequest(q, kp, vp, tables, lens, out, len(self.lens), self.tables.shape[1],
                                              self.layer(window), ks, vs)
        engine.decode(req)
        if not host_io:
            out_host = out.download(out_host.dtype, out_host.shape)
        return from_io(out_host, self.dtype)


def assert_close(out, ref, dtype):
    """max-abs error within the contract's bound.  The bound is on the value
    before the final rounding to the output type; a bfloat16 result carries one
    more rounding step of up to 2^-9 relative (2^-8 if the rounding flips), which
    alone exceeds 2e-3 once |x| > 0.5, so that one bfloat16 unit in the last place
    of the reference value is allowed on top for bfloat16."""
    out = np.asarray(out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    if dtype == DT.bfloat16:
        # one bfloat16 unit in the last place of the reference value: 2^(exponent - 7)
        with np.errstate(divide="ignore", invalid="ignore"):
            ulp = np.where(ref != 0, 2.0 ** (np.floor(np.log2(np.abs(ref))) - 7), 0.0)
        ulp = np.nan_to_num(ulp, nan=0.0)
    else:
        ulp = 0.0
    ok = np.abs(out - ref) <= TOL[dtype] + ulp
    ok |= np.isnan(ref)
    assert ok.all(), f"max abs error {np.nanmax(np.abs(out - ref))}"
    assert np.isfinite(out).all()


def max_abs(a, b):
    return float(np.nanmax(np.abs(np.asarray(a, dtype=np.float64) - np.asarray(b, dtype=np.float64))))
