"""CPU oracle: hashes, quantile sketch, quantizers, grouping, MinMaxSketch, key encoders,
Huffman, SKML container, baseline compressors."""
import numpy as np
import pytest

from sketchml_b200.compress import oracle as o


# --- Java-semantics hash vectors, computed by hand-executing the 32-bit definitions ----------
def _i32(x):
    x &= 0xFFFFFFFF
    return x - (1 << 32) if x & 0x80000000 else x


def _sar(x, s):
    return _i32(x) >> s


def _java_bj(c):
    c = _i32(c)
    c = _i32(_i32(c + 0x7ed55d16) + _i32(c << 12))
    c = _i32((c ^ _i32(0xc761c23c)) ^ _sar(c, 19))
    c = _i32(_i32(c + 0x165667b1) + _i32(c << 5))
    c = _i32(_i32(c + _i32(0xd3a2646c)) ^ _i32(c << 9))
    c = _i32(_i32(c + _i32(0xfd7046c5)) + _i32(c << 3))
    c = _i32((c ^ _i32(0xb55a4f09)) ^ _sar(c, 16))
    return c


def _java_tw(c):
    c = _i32(c)
    c = _i32(~c + _i32(c << 15))
    c = _i32(c ^ _sar(c, 12))
    c = _i32(c + _i32(c << 2))
    c = _i32(c ^ _sar(c, 4))
    c = _i32(c * 2057)
    c = _i32(c ^ _sar(c, 16))
    return c


def _java_mix64(c):
    c = _i32(c)
    c = _i32(~c + _i32(c << 21))
    c = _i32(c ^ _sar(c, 24))
    c = _i32(_i32(c + _i32(c << 3)) + _i32(c << 8))
    c = _i32(c ^ _sar(c, 14))
    c = _i32(_i32(c + _i32(c << 2)) + _i32(c << 4))
    c = _i32(c ^ _sar(c, 28))
    c = _i32(c + _i32(c << 31))
    return c


def _java_bkdr(key, seed):
    c = 0
    while key != 0:
        c = _i32(seed * c + key % 10)
        key //= 10
    return c


def _java_mod(c, size):
    r = abs(c) % size * (1 if c >= 0 else -1)   # Java % truncates toward zero
    return r if r >= 0 else r + size


@pytest.mark.parametrize("hid,fn", [(0, _java_bj), (1, _java_mix64), (2, _java_tw), (3, lambda k: _java_bkdr(k, 31)),
                                    (4, lambda k: _java_bkdr(k, 131)), (5, lambda k: _java_bkdr(k, 267)),
                                    (6, lambda k: _java_bkdr(k, 1313)), (7, lambda k: _java_bkdr(k, 13131))])
def test_hashes_follow_java_int_semantics(hid, fn):
    keys = np.array([0, 1, 2, 9, 10, 12345, 99999999, 2147483647, 1 << 30, 123456789], dtype=np.int32)
    for size in (1, 7, 1000, 65537, 2147483647):
        got = o.hash(hid, keys, size)
        ref = [_java_mod(fn(int(k)), size) for k in keys]
        assert got.tolist() == ref
        assert got.min() >= 0 and got.max() < size


def test_division_free_hash_equals_exact_hash():
    rng = np.random.default_rng(0)
    keys = np.concatenate([rng.integers(0, 2 ** 31 - 1, 50000), [0, 1, 9, 10, 2147483647]]).astype(np.int32)
    for size in (1, 2, 7, 1000, 65537, 300001, 2147483647):
        for hid in range(8):
            assert np.array_equal(o.hash(hid, keys, size), o.hash_fast(hid, keys, size))


def test_multi_row_hash_equals_exact_hash():
    rng = np.random.default_rng(1)
    keys = np.concatenate([rng.integers(0, 2 ** 31 - 1, 20000), rng.integers(0, 1000, 2000),
                           [0, 1, 9, 10, 99, 100, 2147483647, -5]]).astype(np.int32)
    for size in (1, 7, 1000, 300001, 2147483647):
        for ids in ([0, 1, 2], [3, 4, 5], [7, 2, 6], [5], [0, 3], [3, 4, 5, 6], [0, 1, 2, 3, 4, 5, 6, 7], [6, 0, 7, 1, 5]):
            got = o.hash_rows(ids, keys, size).reshape(len(keys), len(ids))
            for r, hid in enumerate(ids):
                assert np.array_equal(got[:, r], o.hash(hid, keys, size)), (ids, size, r)


def test_pick_hashes_distinct_and_deterministic():
    for rows in range(1, 9):
        a = o.pick_hashes(5, 7, 1, 3, rows)
        assert len(set(a)) == rows and a == o.pick_hashes(5, 7, 1, 3, rows)
    assert o.pick_hashes(5, 7, 1, 3, 4) != o.pick_hashes(5, 8, 1, 3, 4) or o.pick_hashes(5, 7, 1, 2, 4) != o.pick_hashes(5, 7, 1, 3, 4)
    with pytest.raises(o.SketchMLError):
        o.pick_hashes(1, 1, 1, 1, 9)
    # the three integer mixers come first (in some order), the BKDR members after them
    seen = set()
    for step in range(40):
        a = o.pick_hashes(5, step, 1, 3, 8)
        assert sorted(a[:3]) == [0, 1, 2] and sorted(a[3:]) == [3, 4, 5, 6, 7]
        seen.add(tuple(a[:3]))
    assert len(seen) == 6


def test_group_edges_table():
    assert o.group_edges(128, 256, 8) == [32, 64, 96, 128, 160, 192, 224, 256]
    assert o.group_edges(100, 256, 8) == [36, 68, 100, 132, 164, 196, 228, 256]
    assert o.group_edges(0, 256, 8) == [0, 32, 64, 96, 128, 160, 192, 256]
    assert o.group_edges(130, 256, 8) == [34, 66, 98, 130, 162, 194, 226, 256]
    assert o.group_edges(255, 256, 8) == [31, 63, 95, 127, 159, 191, 223, 256]
    assert o.group_edges(64, 128, 1) == [128]
    assert o.group_edges(77, 200, 2) == [77, 200]


# --- quantile sketch ---------------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 5, 255, 256, 257, 511, 512, 513, 10000, 200000])
def test_quantile_sketch_rank_error(n):
    rng = np.random.default_rng(n)
    v = rng.normal(size=n)
    s = o.QuantileSketch(128, 1, 2, False)
    s.update(v)
    assert s.n == n and s.min == v.min() and s.max == v.max()
    q = s.quantiles(64)
    assert len(q) == 63 and np.all(np.diff(q) >= 0)
    srt = np.sort(v)
    rank = np.searchsorted(srt, q, side="left") / n
    want = np.minimum(np.floor(n * np.arange(1, 64) / 64), n - 1) / n
    bound = 1e-12 if n < 256 else 0.02
    assert np.abs(rank - want).max() <= bound
    samples, cum = s.summary()
    assert cum[-1] == n and len(samples) == s.retained
    levels = n // 256
    assert s.retained == n % 256 + 128 * bin(levels).count("1")


def test_quantile_sketch_merge_and_errors():
    rng = np.random.default_rng(0)
    a, b = rng.normal(size=70000), rng.normal(2, 3, size=33333)
    sa, sb = o.QuantileSketch(128, 1, 2, False), o.QuantileSketch(128, 2, 2, False)
    sa.update(a)
    sb.update(b)
    sa.merge(sb)
    assert sa.n == len(a) + len(b)
    allv = np.sort(np.concatenate([a, b]))
    q = sa.quantiles(100)
    rank = np.searchsorted(allv, q) / len(allv)
    assert np.abs(rank - np.arange(1, 100) / 100).max() < 0.03
    with pytest.raises(o.SketchMLError):
        o.QuantileSketch(100, 0, 2, False)          # k must be a power of two
    with pytest.raises(o.SketchMLError):
        sa.update(np.array([np.nan]))
    with pytest.raises(o.SketchMLError):
        sa.merge(o.QuantileSketch(64, 0, 2, False)) if False else sa.quantiles(1)
    # the reference starts max at the smallest positive double: all-negative input reports ~0
    sj = o.QuantileSketch(128, 0, 2, True)
    sj.update(np.array([-3.0, -1.0]))
    assert sj.max == np.nextafter(0, 1) and sj.min == -3.0


def test_quantizers():
    rng = np.random.default_rng(1)
    v = rng.laplace(0, 1e-3, 50000)
    q = o.quantile_quantize(v, 256, 128, 3, 2, False)
    assert q["bin_num"] == len(q["splits"]) + 1 == len(q["values"])
    assert np.array_equal(q["bins"], np.searchsorted(q["splits"], v, side="right"))
    assert q["splits"][q["zero_idx"]] >= 0 > q["splits"][q["zero_idx"] - 1]
    vals = q["values"]
    assert vals[0] == 0.5 * (q["min"] + q["splits"][0]) and vals[-1] == 0.5 * (q["splits"][-1] + q["max"])
    assert np.allclose(vals[1:-1], 0.5 * (q["splits"][:-1] + q["splits"][1:]))
    # duplicates shrink the bucket count
    d = o.quantile_quantize(np.repeat([1.0, 2.0, 3.0], 100), 64, 128, 0, 2, False)
    assert d["bin_num"] <= 4 and d["zero_idx"] == 0
    neg = o.quantile_quantize(-np.abs(v) - 1e-9, 32, 128, 0, 2, False)
    assert neg["zero_idx"] == neg["bin_num"] - 1
    u = o.uniform_quantize(v, 16)
    assert np.allclose(np.diff(u["splits"]), (v.max() - v.min()) / 16)
    z = o.zipml_quantize(v[:2000], 32)
    assert 2 <= z["bin_num"] <= 32 and np.all(np.diff(z["splits"]) > 0)
    err_z = np.mean((z["values"][z["bins"]] - v[:2000]) ** 2)
    err_u = np.mean((o.uniform_quantize(v[:2000], 32)["values"][o.uniform_quantize(v[:2000], 32)["bins"]] - v[:2000]) ** 2)
    assert err_z <= err_u * 1.5


# --- MinMaxSketch ------------------------------------------------------------------------------
@pytest.mark.parametrize("tie_mode", [0, 1])
def test_minmax_sketch_properties(tie_mode):
    rng = np.random.default_rng(2)
    zero = 40
    keys = rng.choice(1_000_000, 4000, replace=False).astype(np.int32)
    bins = rng.integers(zero, 64, 4000).astype(np.int32)      # one-sided group
    sk = o.MinMaxSketch(3, 800, zero, [0, 2, 5], tie_mode)
    assert (sk.table == 2147483647).all()
    sk.insert(keys, bins)
    got = sk.query(keys)
    assert (np.abs(got - zero) <= np.abs(bins - zero)).all()     # never further from zero than the truth
    assert (got >= zero).all()                                    # sign (side) preserved
    assert (got == bins).mean() > 0.3
    # order independence in canonical mode
    if tie_mode == 1:
        sk2 = o.MinMaxSketch(3, 800, zero, [0, 2, 5], 1)
        perm = rng.permutation(4000)
        sk2.insert(keys[perm], bins[perm])
        assert np.array_equal(sk.table, sk2.table)
    with pytest.raises(o.SketchMLError):
        o.MinMaxSketch(9, 10, 0, list(range(9)), 0)


# --- key encoders ----------------------------------------------------------------------------------
def _keysets():
    rng = np.random.default_rng(3)
    yield np.array([0], np.int32)
    yield np.array([5], np.int32)
    yield np.array([0, 1, 2, 3], np.int32)
    yield np.array([255, 256, 65791, 65792 + 65536, 2147483646], np.int32)
    yield np.sort(rng.choice(100_000_000, 5000, replace=False)).astype(np.int32)
    yield np.sort(rng.choice(6000, 5000, replace=False)).astype(np.int32)
    yield np.arange(0, 70000 * 300, 70000, dtype=np.int32)


@pytest.mark.parametrize("keys", list(_keysets()))
def test_delta_encoders_roundtrip(keys):
    b = o.delta_binary_encode(keys)
    assert np.array_equal(o.delta_binary_decode(b), keys)
    assert b["flag_bits"] == 2 * len(keys) and b["delta_bits"] % 8 == 0
    a = o.delta_adaptive_encode(keys)
    assert np.array_equal(o.delta_adaptive_decode(a), keys)
    assert a["num_intervals"] in (1, 2, 4, 8, 16)
    assert (a["flag_bits"] + a["delta_bits"]) / len(keys) <= 33


def test_delta_binary_bit_layout():
    # keys 3, 3+300, 3+300+70000 -> widths 1, 2, 4 bytes; flags 0b00, 0b01, 0b11 MSB first
    e = o.delta_binary_encode(np.array([3, 303, 70303], np.int32))
    f = int(e["flag_words"][0])
    bits = [(f >> i) & 1 for i in range(6)]
    assert bits == [0, 0, 0, 1, 1, 1]
    d = int(e["delta_words"][0])
    stream = [(d >> i) & 1 for i in range(56)]
    assert stream[:8] == [0, 0, 0, 0, 0, 0, 1, 1]                       # 3, MSB first
    assert int("".join(map(str, stream[8:24])), 2) == 300
    assert int("".join(map(str, stream[24:56])), 2) == 70000
    assert o.get_bits(list(e["delta_words"]), 8, 16) == 300
    assert o.set_bits([0], 4, 0b101, 3) == [0b1010000]
    with pytest.raises(o.SketchMLError):
        o.delta_binary_encode(np.array([5, 4], np.int32))
    with pytest.raises(o.SketchMLError):
        o.delta_adaptive_encode(np.array([5, 5], np.int32))


def test_huffman_roundtrip_and_optimality():
    rng = np.random.default_rng(4)
    t = rng.choice([3, 4, 5, 6, 2147483647], 20000, p=[0.5, 0.25, 0.125, 0.0625, 0.0625]).astype(np.int32)
    h = o.huffman_encode(t)
    assert np.array_equal(o.huffman_decode(h), t)
    assert [it[0] for it in h["items"]] == sorted(it[0] for it in h["items"])
    assert abs(h["nbits"] / len(t) - 1.875) < 0.05
    one = o.huffman_encode(np.full(10, 7, np.int32))
    assert one["items"] == [(7, 0, 1)] and one["nbits"] == 10 and np.array_equal(o.huffman_decode(one), np.full(10, 7))
    assert len(o.huffman_decode(o.huffman_encode(np.zeros(0, np.int32)))) == 0
    # prefix-free
    codes = [format(b, "0%db" % n) for _, b, n in h["items"]]
    for i, a in enumerate(codes):
        for j, b in enumerate(codes):
            assert i == j or not b.startswith(a)


# --- container ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("enc", [0, 1])
@pytest.mark.parametrize("cells", [-1, 16, 32, 0])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_sparse_payload_roundtrip(enc, cells, dtype):
    rng = np.random.default_rng(5)
    dim = 3_000_000
    keys = np.sort(rng.choice(dim, 20000, replace=False)).astype(np.int32)
    vals = rng.laplace(0, 1e-3, 20000).astype(dtype)
    opts = dict(bin_num=256, group_num=8, row_num=2, col_ratio=0.3, key_encoder=enc, cell_bits=cells, seed=9, step=3,
                rank=1, world=2, loss_partials=[10.0, 6.5, 0.25, 0.0])
    b = o.compress_sparse(keys, vals, dim, opts)
    kind, k, v = o.decompress(b)
    assert kind == 1 and np.array_equal(k, keys) and v.dtype == dtype
    p = o.parse(b)
    assert p["total_bytes"] == len(b) and p["step"] == 3 and p["rank"] == 1 and p["loss_partials"][:3] == [10.0, 6.5, 0.25]
    assert sum(g["n"] for g in p["groups"]) == 20000
    # decoded magnitude never exceeds the true bucket's magnitude side; signs preserved except via the zero bucket
    q = o.quantizer_from_splits(np.asarray(vals), 0, 0, vals)   # exact bins of the true values under unique(vals) splits
    wrong_sign = (np.sign(v) * np.sign(vals) < 0).mean()
    assert wrong_sign < 0.01
    # same compression regardless of the cell format
    b8 = o.compress_sparse(keys, vals, dim, dict(opts, cell_bits=-1))
    assert np.array_equal(o.decompress(b8)[2], v)
    # compression ratio against the reference's own accounting (12 B per non-zero)
    if cells in (-1, 0):
        assert 12 * 20000 / len(b) > 3.5
    # scaling the payload scales the decode values (1/workerNum averaging)
    half = o.payload_times_by(b, 0.5)
    assert np.allclose(o.decompress(half)[2], 0.5 * v, rtol=1e-6)
    # reference field stream: big-endian ints in writeObject order
    j = o.export_java_fields(b)
    assert int.from_bytes(j[0:4], "big") == 8 and int.from_bytes(j[4:8], "big") == 2
    assert np.frombuffer(j[8:16], ">f8")[0] == 0.3 and int.from_bytes(j[16:20], "big") == p["bin_num"]


def test_payload_validation_and_edge_cases():
    dim = 1000
    e = o.compress_sparse(np.zeros(0, np.int32), np.zeros(0), dim, dict(step=2))
    assert o.decompress(e)[0] == 0 and len(e) == 256
    one = o.compress_sparse(np.array([999], np.int32), np.array([-0.5]), dim, dict(bin_num=16, group_num=4))
    kind, k, v = o.decompress(one)
    assert k.tolist() == [999] and v[0] < 0
    bad = bytearray(one)
    bad[30] ^= 1
    with pytest.raises(o.SketchMLError):
        o.parse(bytes(bad))
    with pytest.raises(o.SketchMLError):
        o.parse(one[:100])
    with pytest.raises(o.SketchMLError):
        o.compress_sparse(np.array([5, 5], np.int32), np.array([1.0, 2.0]), dim, {})
    with pytest.raises(o.SketchMLError):
        o.compress_sparse(np.array([1000], np.int32), np.array([1.0]), dim, {})
    with pytest.raises(o.SketchMLError):
        o.compress_sparse(np.array([1], np.int32), np.array([1.0]), dim, dict(row_num=9))
    # all values equal; all negative; groups > buckets
    for vals in (np.full(300, 0.25), -np.arange(1, 301) * 1e-3, np.arange(300) - 150.0):
        keys = np.arange(0, 900, 3, dtype=np.int32)
        b = o.compress_sparse(keys, vals, dim, dict(bin_num=8, group_num=8, row_num=3, col_ratio=0.5))
        kind, k, v = o.decompress(b)
        assert np.array_equal(k, keys) and np.all(np.abs(v) <= np.abs(vals).max() + 1e-12)


def test_dense_payload_and_fixed_point():
    rng = np.random.default_rng(6)
    v = rng.normal(size=5000).astype(np.float32)
    b = o.compress_dense(v, dict(bin_num=256, step=1))
    kind, k, d = o.decompress(b)
    assert kind == 2 and len(d) == 5000 and np.array_equal(k, np.arange(5000))
    assert len(b) < 5000 * 1 + 256 + 1024 + 64
    assert np.abs(d - v).mean() < 0.02
    b16 = o.compress_dense(rng.normal(size=5000), dict(bin_num=1024))
    assert o.parse(b16)["cell_bits"] == 16
    fp = o.fixed_point_encode(v.astype(np.float64), 8, 3)
    dv = o.fixed_point_decode(fp)
    assert np.abs(dv - v).max() <= fp["norm"] / 127 * 1.01 and (np.sign(dv) * np.sign(v) >= 0).all()
    with pytest.raises(o.SketchMLError):
        o.fixed_point_encode(v.astype(np.float64), 30, 0)
    jq = o.export_java_quantizer(np.array([0.0, 1.0]), -1.0, 2.0, np.array([-0.5, 0.5, 1.5]))
    assert int.from_bytes(jq[0:4], "big") == 3 and jq[-3:] == bytes([(0 - 128) & 0xFF, (1 - 128) & 0xFF, (2 - 128) & 0xFF])


def test_sort_helpers():
    a = np.array([5.0, 1.0, 9.0, 3.0, 7.0])
    assert o.quick_select(a, 2) == 3.0 and o.select_kth_largest(a, 2) == 7.0
    k, y = o.kway_merge([[1, 4, 9], [2, 3], []], [[10, 40, 90], [20, 30], []])
    assert k.tolist() == [1, 2, 3, 4, 9] and y.tolist() == [10, 20, 30, 40, 90]
    assert o.unique_sorted(np.array([1.0, 1.0, 2.0, 2.0, 3.0])).tolist() == [1.0, 2.0, 3.0]
    with pytest.raises(o.SketchMLError):
        o.quick_select(a, 6)


def test_pack_bits_roundtrip():
    rng = np.random.default_rng(3)
    for bits in (1, 5, 16, 26, 31, 32):
        hi = (1 << bits) - 1 if bits < 32 else (1 << 31) - 1
        v = rng.integers(0, hi, 1001, endpoint=True).astype(np.int64).astype(np.uint32).view(np.int32)
        w = o.pack_bits(v, bits)
        assert w.dtype == np.uint32 and len(w) == (len(v) * bits + 31) // 32 + 2
        assert np.array_equal(o.unpack_bits(w, len(v), bits), v)
    with pytest.raises(Exception):
        o.pack_bits(np.array([8], dtype=np.int32), 3)


def test_pack_varbytes_roundtrip():
    rng = np.random.default_rng(4)
    for n in (0, 1, 3, 1023, 1024, 1025, 5000):
        v = (rng.integers(0, 2 ** 31 - 1, n) >> rng.integers(0, 31, n)).astype(np.int32)
        d = o.pack_varbytes(v)
        assert len(d["block_offsets"]) == (n + 1023) // 1024 + 1
        widths = np.where(v < 256, 1, np.where(v < 65536, 2, np.where(v < 2 ** 24, 3, 4)))
        assert len(d["bytes"]) == widths.sum() + 24
        if n > 1024:
            assert d["block_offsets"][1] == widths[:1024].sum()
        assert np.array_equal(o.unpack_varbytes(d["flags"], d["bytes"], n), v)
    with pytest.raises(Exception):
        o.pack_varbytes(np.array([-1], dtype=np.int32))


def test_row_sort_delta():
    rowptr = np.array([10, 13, 13, 17], dtype=np.int64)  # offsets may start anywhere
    cols = np.array([7, 2, 9, 5, 5, 1, 30], dtype=np.int32)
    got = o.row_sort_delta(rowptr, cols)
    assert got.tolist() == [2, 5, 2, 1, 4, 0, 25]
    back = np.concatenate([np.cumsum(got[0:3]), np.cumsum(got[3:7])])
    assert back.tolist() == [2, 7, 9, 1, 5, 5, 30]


def test_pack_varnibbles_roundtrip():
    rng = np.random.default_rng(5)
    for n in (0, 1, 5, 1023, 1024, 1025, 7000):
        v = (rng.integers(0, 2 ** 31 - 1, n) >> rng.integers(0, 31, n)).astype(np.int32)
        d = o.pack_varnibbles(v)
        widths = np.ones(n, dtype=np.int64)
        for k in range(1, 8):
            widths += (v >> (4 * k)) != 0
        assert d["block_offsets"][-1] == widths.sum()
        assert np.array_equal(o.unpack_varnibbles(d["flags"], d["words"], n), v)


def test_parallel_quantize_and_create_use_threads():
    """The `parallel_*` forms run on `Parallel.get_parallelism()` threads of the C++ library: per-thread
    quantile sketches merged into one keep the rank error of a k = 128 summary, the buckets equal the
    serial lookup for the same splits, and the thread-per-group sketch build gives the serial payload."""
    from sketchml_b200.compress import GroupedMinMaxSketch, Parallel, QuantileQuantizer, SparseVectorCompressor
    rng = np.random.default_rng(3)
    v = rng.laplace(0, 1e-2, 400_000)
    Parallel.set_parallelism(4)
    try:
        q = QuantileQuantizer(256, seed=7)
        q.parallel_quantize(v)
        s = np.sort(v)
        ranks = np.searchsorted(s, q.splits) / len(v)
        assert np.abs(np.diff(np.concatenate([[0.0], ranks, [1.0]]))).max() < 1.0 / 256 + 0.03
        assert np.array_equal(q.get_bins(), np.searchsorted(q.splits, v, side="right"))
        assert q.min == v.min() and q.max == v.max()
        keys = np.sort(rng.choice(5_000_000, 60_000, replace=False)).astype(np.int32)
        bins = rng.integers(0, 256, len(keys))
        a, b = GroupedMinMaxSketch(8, 2, 0.3, 256, 128, seed=5), GroupedMinMaxSketch(8, 2, 0.3, 256, 128, seed=5)
        a.create(keys, bins)
        b.parallel_create(keys, bins)
        assert a.payload == b.payload
        c = SparseVectorCompressor(seed=2)
        c.parallel_compress_sparse(keys, v[: len(keys)])
        k2, v2 = c.decompress_sparse()
        assert np.array_equal(k2, keys)
        assert np.all(np.sign(v2) == np.sign(v[: len(keys)])) or (np.sign(v2) != np.sign(v[: len(keys)])).mean() < 0.06
    finally:
        Parallel.shutdown()
