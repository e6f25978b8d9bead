"""GPU compress / decode kernels against the C++ CPU oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _sparse_grad(n, dim, seed, scale=1e-3, positive_only=False):
    rng = np.random.default_rng(seed)
    if dim <= 4 * n or dim < 10_000_000:
        keys = np.sort(rng.choice(dim, n, replace=False)).astype(np.int32)
    else:
        keys = np.unique(rng.integers(0, dim, size=2 * n + 16))
        keys = np.sort(rng.permutation(keys)[:n]).astype(np.int32)
    vals = rng.laplace(0, scale, n).astype(np.float32)
    if positive_only:
        vals = np.abs(vals) + 1e-6
    vals[vals == 0] = 1e-6
    return keys, vals


def _sections(p):
    out = []
    for g in p["groups"]:
        out.append((g["n"], g["col_num"], tuple(g["hash_ids"]), g["table"].tolist() if g["n"] else None,
                    (g["keys"]["num_intervals"], g["keys"]["flag_kind"]) if g["n"] else None,
                    g["keys"]["flag_words"].tolist() if g["n"] else None,
                    g["keys"]["delta_words"].tolist() if g["n"] else None,
                    g.get("restart_raw").tolist() if g["n"] else None))
    return out


@pytest.mark.parametrize("encoder", ["delta_binary", "delta_adaptive"])
@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("n,dim,q,G,rows,ratio", [
    (5000, 200000, 256, 8, 2, 0.3), (1, 1000, 64, 8, 3, 0.2), (2049, 100000000, 128, 1, 3, 0.2),
    (70000, 80000, 256, 8, 2, 0.3), (3000, 2 ** 31 - 2, 300, 4, 1, 0.5), (40000, 5000000, 64, 2, 8, 0.1),
    (300000, 3000000, 256, 8, 3, 0.2)])
def test_payload_bit_exact_with_given_splits(encoder, fused, n, dim, q, G, rows, ratio):
    """Everything downstream of the split points equals the CPU oracle bit for bit, with both key
    encoders (delta_adaptive: the groups' interval counts and flag kinds, the two bit streams and
    the restart points)."""
    from sketchml_b200.compress import oracle
    from sketchml_b200.ops import GpuCompressor
    keys, vals = _sparse_grad(n, dim, seed=n)
    qz = oracle.quantile_quantize(vals, q, 128, 1, 2, False)
    splits = qz["splits"].astype(np.float32)
    opts = dict(bin_num=q, group_num=G, row_num=rows, col_ratio=ratio, seed=11, step=7, rank=2, world=4, tie_mode=1,
                key_encoder=1 if encoder == "delta_adaptive" else 0)
    ref = oracle.compress_sparse(keys, vals, dim, opts, splits, float(qz["min"]), float(qz["max"]))
    comp = GpuCompressor(dim, n, q, G, rows, ratio, seed=11, fused=fused, key_encoder=encoder)
    buf = comp.compress_local(torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda(), step=7, rank=2, world=4,
                              given=(torch.from_numpy(splits).cuda(), qz["min"], qz["max"]))
    got = comp.payload_bytes(buf)
    pg, pr = oracle.parse(got), oracle.parse(ref)
    for k in ("kind", "step", "rank", "world", "dim", "nnz", "bin_num", "zero_idx", "group_num", "row_num", "col_ratio",
              "key_encoder", "cell_bits", "seed", "restart_interval"):
        assert pg[k] == pr[k], k
    assert np.array_equal(pg["bucket_values"], pr["bucket_values"])
    sg, sr = _sections(pg), _sections(pr)
    for gi, (a, b) in enumerate(zip(sg, sr)):
        for fi, (x, y) in enumerate(zip(a, b)):
            assert x == y, f"group {gi} field {fi} differs"
    kind, k2, v2 = oracle.decompress(got)
    _, k3, v3 = oracle.decompress(ref)
    assert np.array_equal(k2, keys) and np.array_equal(v2, v3)


@pytest.mark.parametrize("encoder", ["delta_binary", "delta_adaptive"])
@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("n,dim,q,G,rows,ratio", [
    (5000, 200000, 256, 8, 2, 0.3), (1, 1000, 64, 8, 3, 0.2), (2049, 100000000, 128, 1, 3, 0.2),
    (3000, 2 ** 31 - 2, 300, 4, 1, 0.5), (300000, 3000000, 256, 8, 3, 0.2)])
def test_huffman_coded_tables(encoder, fused, n, dim, q, G, rows, ratio):
    """cell_bits = 0: the tables travel Huffman-coded. The device's code is canonical and carries restart
    offsets, so its bytes differ from the CPU oracle's tree-walk code; the decoded tables, every other
    section and the decoded gradient are the oracle's bit for bit. The GPU decoder reads both forms."""
    from sketchml_b200.compress import oracle
    from sketchml_b200.ops import GpuCompressor, GpuDecoder
    keys, vals = _sparse_grad(n, dim, seed=n + 3)
    qz = oracle.quantile_quantize(vals, q, 128, 1, 2, False)
    splits = qz["splits"].astype(np.float32)
    opts = dict(bin_num=q, group_num=G, row_num=rows, col_ratio=ratio, seed=11, step=7, rank=0, world=1, tie_mode=1,
                key_encoder=1 if encoder == "delta_adaptive" else 0, cell_bits=0)
    ref = oracle.compress_sparse(keys, vals, dim, opts, splits, float(qz["min"]), float(qz["max"]))
    comp = GpuCompressor(dim, n, q, G, rows, ratio, seed=11, fused=fused, key_encoder=encoder, cell_bits=0)
    buf = comp.compress_local(torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda(), step=7, rank=0, world=1,
                              given=(torch.from_numpy(splits).cuda(), qz["min"], qz["max"]))
    got = comp.payload_bytes(buf)
    pg, pr = oracle.parse(got), oracle.parse(ref)
    assert pg["cell_bits"] == pr["cell_bits"] == 0
    for gi, (a, b) in enumerate(zip(_sections(pg), _sections(pr))):
        for fi, (x, y) in enumerate(zip(a, b)):
            assert x == y, f"group {gi} field {fi} differs"
    _, k2, v2 = oracle.decompress(got)
    _, k3, v3 = oracle.decompress(ref)
    assert np.array_equal(k2, keys) and np.array_equal(v2, v3)
    # with enough cells per group to pay for the code books, the Huffman-coded payload is the smaller one
    plain = GpuCompressor(dim, n, q, G, rows, ratio, seed=11, fused=fused, key_encoder=encoder)
    pb = plain.compress_local(torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda(), step=7, rank=0, world=1,
                              given=(torch.from_numpy(splits).cuda(), qz["min"], qz["max"]))
    if n >= 100000:
        assert len(got) < len(plain.payload_bytes(pb))
    # both the device-made and the oracle-made payload decode on the GPU to the oracle's values
    want = np.zeros(dim if dim <= 10 ** 8 else 1)
    if dim <= 10 ** 8:
        want[k3] = v3
        dec = GpuDecoder(dim, n, fused=fused)
        out = dec.decode_sum([buf], step=7).cpu().numpy()
        assert np.array_equal(out[k3], v3.astype(np.float32)) and np.count_nonzero(out) <= n
        rb = torch.zeros(max(buf.numel(), len(ref) + 256), dtype=torch.uint8, device="cuda")
        rb[:len(ref)] = torch.frombuffer(bytearray(ref), dtype=torch.uint8).cuda()
        out2 = dec.decode_sum([rb], step=7).cpu().numpy()
        assert np.array_equal(out2, out)


@pytest.mark.parametrize("summary", ["sample", "sketch"])
@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("n", [100, 255, 256, 257, 2047, 2048, 2049, 4096, 4097, 30000, 1000003])
def test_quantile_splits_rank_error(fused, n, summary):
    from sketchml_b200.compress import oracle
    from sketchml_b200.ops import GpuCompressor
    dim = max(4 * n, 1000)
    keys, vals = _sparse_grad(n, dim, seed=n + 1)
    q = 256
    comp = GpuCompressor(dim, n, q, 8, 2, 0.3, seed=3, fused=fused, quantile_summary=summary)
    buf = comp.compress_local(torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda())
    p = oracle.parse(comp.payload_bytes(buf))
    bv = p["bucket_values"]
    assert p["nnz"] == n and 2 <= p["bin_num"] <= q
    assert abs(p["min_value"] - vals.min()) < 1e-12 and abs(p["max_value"] - vals.max()) < 1e-12
    assert np.all(np.diff(bv) > 0)
    # recover the splits from the midpoints and measure their rank error
    splits = np.empty(p["bin_num"] - 1)
    prev = p["min_value"]
    for i in range(p["bin_num"] - 1):
        splits[i] = 2 * float(bv[i]) - prev
        prev = splits[i]
    s = np.sort(vals.astype(np.float64))
    ranks = np.searchsorted(s, splits, side="left") / n
    if n <= 128:
        assert p["bin_num"] >= min(q, n) // 2
    # every split is an order statistic near an even quantile: gaps between consecutive
    # split ranks stay within the k = 128 sketch's error band
    err = np.abs(np.diff(np.concatenate([[0.0], ranks, [1.0]]))).max()
    assert err < 1.0 / q + 0.03, err
    if summary == "sample" and q <= n <= 2048:
        # every value is in the sample: the splits are exact order statistics (the test recovers them from
        # the bucket midpoints in float arithmetic, which can move a rank by one or two)
        assert err <= 1.0 / q + 3.0 / n, err
    kind, k2, v2 = oracle.decompress(comp.payload_bytes(buf))
    assert np.array_equal(k2, keys)
    assert np.all(np.sign(v2) == np.sign(vals)) or (np.sign(v2) != np.sign(vals)).mean() < 0.06


DECODE_MODES = {"staged": dict(fused=False), "fused": dict(fused=True)}


@pytest.mark.parametrize("cell_bits", [-1, 0])
@pytest.mark.parametrize("encoder", ["delta_binary", "delta_adaptive"])
@pytest.mark.parametrize("mode", list(DECODE_MODES))
def test_decode_sum_matches_oracle(mode, encoder, cell_bits):
    from sketchml_b200.compress import oracle
    from sketchml_b200.ops import GpuCompressor, GpuDecoder
    dim, world = 300000, 3
    fused = mode != "staged"
    comp = GpuCompressor(dim, 20000, 128, 8, 3, 0.2, seed=5, fused=fused, key_encoder=encoder, cell_bits=cell_bits)
    bufs, ref = [], np.zeros(dim)
    for r in range(world):
        keys, vals = _sparse_grad(15000 + 1000 * r, dim, seed=100 + r)
        b = comp.compress_local(torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda(), step=4, rank=r, world=world)
        bufs.append(b.clone())
        _, k, v = oracle.decompress(comp.payload_bytes(b))
        ref[k] += v.astype(np.float64) / world
    dec = GpuDecoder(dim, 20000 * world, **DECODE_MODES[mode])
    out = dec.decode_sum(bufs, step=4).cpu().numpy().astype(np.float64)
    assert np.abs(out - ref).max() <= 1e-6 * np.abs(ref).max()
    assert int(dec.acc.abs().max()) == 0
    # a second call gives the same bits (accumulators were left clean, sums are order independent)
    out2 = dec.decode_sum(bufs, step=4).cpu().numpy()
    assert np.array_equal(out2.astype(np.float64), out)


def test_dense_kind_roundtrip_and_mixed_decode():
    from sketchml_b200.compress import oracle
    from sketchml_b200.ops import GpuCompressor, GpuDecoder
    dim = 50000
    rng = np.random.default_rng(1)
    dense = rng.normal(0, 1e-2, dim).astype(np.float32)
    comp = GpuCompressor(dim, dim, 256, 8, 2, 0.3, seed=1)
    qz = oracle.quantile_quantize(dense, 256, 128, 1, 2, False)
    splits = torch.from_numpy(qz["splits"].astype(np.float32)).cuda()
    b0 = comp.compress_local(None, torch.from_numpy(dense).cuda(), step=2, rank=0, world=2, dense=True,
                             given=(splits, qz["min"], qz["max"])).clone()
    ref0 = oracle.compress_dense(dense, dict(bin_num=256, step=2, rank=0, world=2, seed=1), qz["splits"].astype(np.float32),
                                 float(qz["min"]), float(qz["max"]))
    k0, kk, v0 = oracle.decompress(comp.payload_bytes(b0))
    _, _, vr = oracle.decompress(ref0)
    assert k0 == 2 and np.array_equal(v0, vr)
    # sketch-built splits (no given): decode error bounded by bucket width
    b0s = comp.compress_local(None, torch.from_numpy(dense).cuda(), step=2, rank=0, world=2, dense=True).clone()
    _, _, v0s = oracle.decompress(comp.payload_bytes(b0s))
    assert np.abs(v0s - dense).mean() < 2e-3
    keys, vals = _sparse_grad(4000, dim, seed=8)
    b1 = comp.compress_local(torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda(), step=2, rank=1, world=2).clone()
    _, k1, v1 = oracle.decompress(comp.payload_bytes(b1))
    ref = v0s.astype(np.float64) / 2
    ref[k1] += v1.astype(np.float64) / 2
    out = GpuDecoder(dim, dim).decode_sum([b0s, b1], step=2).cpu().numpy()
    assert np.abs(out - ref).max() <= 1e-6 * np.abs(ref).max()


def test_empty_gradient_and_updates():
    from sketchml_b200.compress import oracle
    from sketchml_b200.ops import GpuCompressor, GpuDecoder
    dim = 10000
    comp = GpuCompressor(dim, 1000, 64, 8, 2, 0.3, seed=2)
    e = comp.compress_local(torch.zeros(0, dtype=torch.int32, device="cuda"), torch.zeros(0, device="cuda"), step=1,
                            rank=0, world=2).clone()
    assert oracle.parse(comp.payload_bytes(e))["kind"] == 0
    keys, vals = _sparse_grad(900, dim, seed=4, scale=1e-1)
    b = comp.compress_local(torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda(), step=1, rank=1, world=2).clone()
    _, k, v = oracle.decompress(comp.payload_bytes(b))
    g = np.zeros(dim)
    g[k] = v.astype(np.float64) / 2
    dec = GpuDecoder(dim, 2000)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cap = min(e.numel(), b.numel())
    # SGD
    w = torch.ones(dim, device="cuda")
    dec.decode_update([e.data_ptr(), b.data_ptr()], [None, None], cap, 1, status, w=w, lr=0.5)
    assert int(status.item()) == 0
    assert np.abs(w.cpu().numpy() - (1 - 0.5 * g)).max() < 1e-6
    # lazy Adam: only touched coordinates move
    w = torch.ones(dim, device="cuda")
    m = torch.zeros(dim, device="cuda")
    vv = torch.zeros(dim, device="cuda")
    scale = np.sqrt(1 - 0.999) / (1 - 0.9)
    dec.decode_update([e.data_ptr(), b.data_ptr()], [None, None], cap, 1, status, w=w, lr=0.1, adam_m=m, adam_v=vv,
                      adam_scale=scale)
    mt, vt = 0.1 * g, 0.001 * g * g
    ref = 1 - 0.1 * scale * mt / (np.sqrt(vt) + 1e-8)
    assert np.abs(w.cpu().numpy() - ref).max() < 1e-4
    assert np.abs(m.cpu().numpy() - mt).max() < 1e-7
    untouched = np.ones(dim, bool)
    untouched[k] = False
    assert (w.cpu().numpy()[untouched] == 1).all()


def test_bad_header_and_timeout_are_reported_not_fatal():
    from sketchml_b200.ops import GpuCompressor, GpuDecoder
    from sketchml_b200.parallel.failure import PayloadError, StepTimeout, check_status
    dim = 10000
    comp = GpuCompressor(dim, 1000, 64, 8, 2, 0.3, seed=2)
    keys, vals = _sparse_grad(500, dim, seed=4)
    b = comp.compress_local(torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda(), step=3).clone()
    dec = GpuDecoder(dim, 1000, budget_s=0.05)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    w = torch.zeros(dim, device="cuda")
    # stale step: the header says 3, the decoder expects 4
    dec.decode_update([b.data_ptr()], [None], b.numel(), 4, status, w=w, lr=1.0)
    with pytest.raises(PayloadError):
        check_status(int(status.item()))
    status.zero_()
    # corrupted header byte -> checksum mismatch
    bad = b.clone()
    bad[40] ^= 0x11
    dec.decode_update([bad.data_ptr()], [None], bad.numel(), 3, status, w=w, lr=1.0)
    with pytest.raises(PayloadError):
        check_status(int(status.item()))
    status.zero_()
    # an arrival flag that nothing sets: the bounded wait gives up and the context stays usable
    flag = torch.zeros(4, dtype=torch.int64, device="cuda")
    dec.decode_update([b.data_ptr()], [flag.data_ptr()], b.numel(), 3, status, w=w, lr=1.0)
    with pytest.raises(StepTimeout):
        check_status(int(status.item()))
    status.zero_()
    dec.reset()
    assert float(w.abs().max()) == 0.0
    flag[0] = 4  # step + 1
    dec.decode_update([b.data_ptr()], [flag.data_ptr()], b.numel(), 3, status, w=w, lr=1.0)
    assert int(status.item()) == 0 and float(w.abs().max()) > 0


def test_non_finite_values_are_reported():
    from sketchml_b200.ops import GpuCompressor
    keys, vals = _sparse_grad(5000, 100000, seed=3)
    vals[17] = -np.inf
    comp = GpuCompressor(100000, 5000, 64, 8, 2, 0.3, seed=1)
    with pytest.raises(RuntimeError, match="invalid kernel input"):
        comp.compress_local(torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda())
    # the compressor stays usable afterwards
    vals[17] = 1e-3
    comp.compress_local(torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda())


@pytest.mark.parametrize("bits", [8, 5, 13, 16])
def test_fixed_point_pack_matches_oracle(bits):
    """The pack kernel's code stream against the CPU oracle's BitSet words, and the unpack kernel
    against the oracle's decode (the two norms differ in summation order, so a code may differ by
    one where |v| / norm * max sits on an integer)."""
    from sketchml_b200.compress import oracle
    from sketchml_b200.ops.baseline_quant import FixedPointCodec
    n, n_max, seed = 100003, 120000, 991
    g = torch.Generator().manual_seed(bits)
    vals = (torch.randn(n_max, generator=g) * 0.01).float()
    keys = torch.sort(torch.randperm(1_000_000, generator=g)[:n_max]).values.int()
    dv, dk = vals.cuda(), keys.cuda()
    cnt = torch.tensor([n], dtype=torch.int64, device="cuda")
    fp = FixedPointCodec(n_max, bits, 1, "cuda")
    fp.pack(dv, cnt, seed)
    out = torch.zeros(n_max, dtype=torch.float32, device="cuda")
    acc = torch.zeros(1_000_000, dtype=torch.float32, device="cuda")
    fp.unpack(dk, fp.codes, fp.norm, cnt, 1, acc=acc, vals_out=out)
    torch.cuda.synchronize()
    code = oracle.fixed_point_encode(vals[:n].double().numpy(), bits, seed)
    assert abs(float(fp.norm.item()) - code["norm"]) <= 1e-12 * code["norm"]
    want = np.asarray(code["words"], dtype=np.uint64).view(np.uint8)
    nbytes = (n * bits + 7) // 8
    got = fp.codes[:nbytes].cpu().numpy()
    assert (got != want[:nbytes]).mean() < 1e-4
    dec = oracle.fixed_point_decode(code)
    step = code["norm"] / ((1 << (bits - 1)) - 1)
    diff = np.abs(out[:n].cpu().numpy().astype(np.float64) - dec)
    assert diff.max() <= step * 1.0001 and (diff > 1e-7 * code["norm"]).mean() < 1e-4
    ref = torch.zeros(1_000_000, dtype=torch.float64)
    ref[keys[:n].long()] = torch.from_numpy(dec)
    assert float((acc.cpu().double() - ref).abs().max()) <= step * 1.0001
    assert float(out[n:].abs().max()) == 0.0


@pytest.mark.parametrize("mode", list(DECODE_MODES))
def test_several_overlapping_payloads_sgd_and_adam(mode):
    """Four payloads with many shared keys: the key-range-owned apply must equal the oracle's
    decoded mean for SGD and one lazy-Adam step on exactly the touched coordinates."""
    from sketchml_b200.compress import oracle
    from sketchml_b200.ops import GpuCompressor, GpuDecoder
    dim, P, n = 60000, 4, 9000
    comp = GpuCompressor(dim, n, 128, 8, 3, 0.3, seed=5)
    bufs, g = [], np.zeros(dim)
    for r in range(P):
        keys, vals = _sparse_grad(n - 500 * r, dim // 3, seed=20 + r, scale=1e-2)  # keys crowd the low third: overlaps
        b = comp.compress_local(torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda(), step=7, rank=r, world=P).clone()
        _, k, v = oracle.decompress(comp.payload_bytes(b))
        g[k] += v.astype(np.float32).astype(np.float64) / P
        bufs.append(b)
    cap = min(b.numel() for b in bufs)
    ptrs = [b.data_ptr() for b in bufs]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    dec = GpuDecoder(dim, P * n, **DECODE_MODES[mode])
    w = torch.ones(dim, device="cuda")
    dec.decode_update(ptrs, [None] * P, cap, 7, status, w=w, lr=0.5)
    assert int(status.item()) == 0
    assert np.abs(w.cpu().numpy() - (1 - 0.5 * g)).max() < 2e-6
    w = torch.ones(dim, device="cuda")
    m = torch.zeros(dim, device="cuda")
    vv = torch.zeros(dim, device="cuda")
    scale = np.sqrt(1 - 0.999) / (1 - 0.9)
    dec.decode_update(ptrs, [None] * P, cap, 7, status, w=w, lr=0.1, adam_m=m, adam_v=vv, adam_scale=scale)
    assert int(status.item()) == 0
    mt, vt = 0.1 * g, 0.001 * g * g
    ref = 1 - 0.1 * scale * mt / (np.sqrt(vt) + 1e-8)
    touched = g != 0
    assert np.abs(w.cpu().numpy() - ref)[touched].max() < 2e-4
    assert (w.cpu().numpy()[~touched] == 1).all()
    assert np.abs(m.cpu().numpy() - mt).max() < 1e-6
    assert float(dec.acc.abs().max()) == 0  # the accumulators are clean for the next step
    # a second, identical call gives bit-identical results (no order dependence)
    w2 = torch.ones(dim, device="cuda")
    m2 = torch.zeros(dim, device="cuda")
    v2 = torch.zeros(dim, device="cuda")
    dec.decode_update(ptrs, [None] * P, cap, 7, status, w=w2, lr=0.1, adam_m=m2, adam_v=v2, adam_scale=scale)
    assert torch.equal(w, w2) and torch.equal(m, m2) and torch.equal(vv, v2)
    # the packed state layout ({m, v, sum, -} per coordinate) gives the same bits and leaves its sums clean
    quad = torch.zeros((dim, 4), device="cuda")
    w3 = torch.ones(dim, device="cuda")
    dec.decode_update(ptrs, [None] * P, cap, 7, status, w=w3, lr=0.1, adam_m=quad[:, 0], adam_v=quad[:, 1], adam_scale=scale)
    assert int(status.item()) == 0
    assert torch.equal(w, w3) and torch.equal(m, quad[:, 0]) and torch.equal(vv, quad[:, 1])
    assert float(quad[:, 2:].abs().max()) == 0 and float(dec.acc.abs().max()) == 0


@pytest.mark.parametrize("encoder", ["delta_binary", "delta_adaptive"])
def test_decode_skewed_keys_many_ranks(encoder):
    """Eight payloads with Zipf-like keys (many shared coordinates, one nearly empty payload): the fused
    launch must give the bits of the staged launches, which apply the ranks in the same order per
    coordinate, for SGD and for lazy Adam, and the same bits on every repetition."""
    from sketchml_b200.ops import GpuCompressor, GpuDecoder
    dim, P, n = 3_000_000, 8, 40000
    comp = GpuCompressor(dim, n, 256, 8, 3, 0.2, seed=9, key_encoder=encoder)
    rng = np.random.default_rng(5)
    bufs = []
    for r in range(P):
        keys = np.unique(np.minimum(rng.zipf(1.2, 3 * n), dim - 1))[: n - 1000 * r].astype(np.int32)
        if r == 5:
            keys = keys[:3]   # a payload whose groups are nearly all empty
        vals = rng.laplace(0, 1e-2, len(keys)).astype(np.float32)
        bufs.append(comp.compress_local(torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda(), step=3, rank=r, world=P).clone())
    cap = min(b.numel() for b in bufs)
    ptrs = [b.data_ptr() for b in bufs]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref_dec = GpuDecoder(dim, P * n, fused=False)
    w_ref = torch.ones(dim, device="cuda")
    ref_dec.decode_update(ptrs, [None] * P, cap, 3, status, w=w_ref, lr=0.5)
    assert int(status.item()) == 0
    dec = GpuDecoder(dim, P * n, max_groups=8)
    for _ in range(3):
        w = torch.ones(dim, device="cuda")
        dec.decode_update(ptrs, [None] * P, cap, 3, status, w=w, lr=0.5)
        assert int(status.item()) == 0
        assert torch.equal(w, w_ref)

    def adam(d):
        w, m, v = torch.ones(dim, device="cuda"), torch.zeros(dim, device="cuda"), torch.zeros(dim, device="cuda")
        d.decode_update(ptrs, [None] * P, cap, 3, status, w=w, lr=0.1, adam_m=m, adam_v=v, adam_scale=0.3)
        assert int(status.item()) == 0
        return w, m, v
    for a, b in zip(adam(dec), adam(ref_dec)):
        assert torch.equal(a, b)
    quad = torch.zeros((dim, 4), device="cuda")
    wq = torch.ones(dim, device="cuda")
    dec.decode_update(ptrs, [None] * P, cap, 3, status, w=wq, lr=0.1, adam_m=quad[:, 0], adam_v=quad[:, 1], adam_scale=0.3)
    assert int(status.item()) == 0
    for a, b in zip((wq, quad[:, 0], quad[:, 1]), adam(ref_dec)):
        assert torch.equal(a, b)
    assert float(quad[:, 2].abs().max()) == 0
    assert float(dec.acc.abs().max()) == 0


def _key_sets():
    rng = np.random.default_rng(11)
    yield "empty", np.zeros(0, dtype=np.int32)
    yield "single zero", np.array([0], dtype=np.int32)
    yield "single big", np.array([2 ** 31 - 1], dtype=np.int32)
    yield "consecutive", np.arange(5000, dtype=np.int32)
    yield "small gaps", np.cumsum(rng.integers(1, 4, 70001)).astype(np.int32)
    yield "byte gaps", np.cumsum(rng.integers(1, 300, 33333)).astype(np.int32)
    yield "wide gaps", np.sort(rng.choice(2 ** 31 - 2, 20000, replace=False)).astype(np.int32)
    yield "mixed", np.unique(np.concatenate([rng.integers(0, 5000, 3000), rng.integers(0, 2 ** 30, 3000)])).astype(np.int32)
    yield "zipf", np.unique(np.minimum(rng.zipf(1.1, 200000), 50_000_000 - 1)).astype(np.int32)


@pytest.mark.parametrize("name,keys", list(_key_sets()), ids=[n for n, _ in _key_sets()])
def test_delta_adaptive_device_codec_is_bit_exact(name, keys):
    """Device DeltaAdaptive encode equals the CPU oracle word for word; device decode inverts both."""
    from sketchml_b200.compress import oracle
    from sketchml_b200.ops import keys as K
    ref = oracle.delta_adaptive_encode(keys)
    got = K.encode(torch.from_numpy(keys).cuda())
    assert (got.size, got.num_intervals, got.flag_kind) == (ref["size"], ref["num_intervals"], ref["flag_kind"])
    assert (got.flag_bits, got.delta_bits) == (ref["flag_bits"], ref["delta_bits"])
    d = got.to_oracle_dict()
    assert np.array_equal(d["flag_words"], np.asarray(ref["flag_words"], dtype=np.uint64))
    assert np.array_equal(d["delta_words"], np.asarray(ref["delta_words"], dtype=np.uint64))
    assert np.array_equal(oracle.delta_adaptive_decode(d), keys)
    assert np.array_equal(K.decode(got).cpu().numpy(), keys)


def test_delta_adaptive_device_codec_rejects_unsorted_keys():
    from sketchml_b200.ops import keys as K
    with pytest.raises(ValueError):
        K.encode(torch.tensor([1, 5, 5, 9], dtype=torch.int32, device="cuda"))


def _zip_pack(vals, bins):
    from sketchml_b200.ops.baseline_quant import ZipCodec
    n = len(vals)
    zc = ZipCodec(max(n, 1) + 37, bins, 1, "cuda")   # a capacity above n: the padding must not disturb the search
    v = torch.zeros(zc.n_max, device="cuda")
    v[:n] = torch.from_numpy(vals).cuda()
    cnt = torch.tensor([n], dtype=torch.int64, device="cuda")
    zc.pack(v, cnt)
    nb, zero, rounds = (int(x) for x in zc.meta[:3].cpu())
    codes = zc.codes.cpu().numpy()
    codes = codes[:n] if zc.code_bytes == 1 else codes[:2 * n].view(np.uint16)
    return zc, v, cnt, nb, zero, rounds, zc.splits[:max(nb - 1, 0)].cpu().numpy(), zc.mids[:nb].cpu().numpy(), codes.astype(np.int64)


@pytest.mark.parametrize("n,bins", [(1, 16), (2, 2), (3, 2), (77, 8), (1000, 256), (4097, 33), (50001, 256), (300000, 300)])
def test_zipml_device_quantizer_equals_oracle_on_exact_sums(n, bins):
    """Values on a dyadic grid make every prefix sum exact in double, whatever the order of the adds,
    so the device search must pick the very split points of the CPU oracle, round by round."""
    from sketchml_b200.compress import oracle
    rng = np.random.default_rng(n + bins)
    vals = (rng.integers(-2000, 2000, n) / 1024.0).astype(np.float32)
    ref = oracle.zipml_quantize(vals.astype(np.float64), bins)
    zc, v, cnt, nb, zero, rounds, splits, mids, codes = _zip_pack(vals, bins)
    assert nb == ref["bin_num"] and zero == ref["zero_idx"]
    assert np.array_equal(splits.astype(np.float64), ref["splits"])
    assert np.array_equal(mids, ref["values"].astype(np.float32))
    assert np.array_equal(codes, ref["bins"])
    # decode: every value becomes its bucket's midpoint; the accumulating form adds them at the keys
    out = torch.zeros_like(v)
    zc.unpack(None, zc.codes, zc.mids, cnt, 1, vals_out=out)
    assert np.array_equal(out[:n].cpu().numpy(), ref["values"].astype(np.float32)[ref["bins"]])
    keys = torch.from_numpy(np.sort(rng.choice(4 * n + 8, n, replace=False)).astype(np.int32)).cuda()
    kfull = torch.zeros(zc.n_max, dtype=torch.int32, device="cuda")
    kfull[:n] = keys
    acc = torch.zeros(4 * n + 8, device="cuda")
    zc.unpack(kfull, zc.codes, zc.mids, cnt, 1, acc=acc)
    assert torch.equal(acc[keys.long()], out[:n]) and int(torch.count_nonzero(acc)) <= n


@pytest.mark.parametrize("bins", [16, 256])
def test_zipml_device_quantizer_quality_and_empty_input(bins):
    """Real-valued input: the order of the prefix-sum adds differs from the sequential oracle, so near
    ties may fall the other way; the quantization error must still match the oracle's closely."""
    from sketchml_b200.compress import oracle
    _, vals = _sparse_grad(120000, 10 ** 6, seed=5)
    ref = oracle.zipml_quantize(vals.astype(np.float64), bins)
    zc, v, cnt, nb, zero, rounds, splits, mids, codes = _zip_pack(vals, bins)
    assert 2 <= nb <= bins and rounds >= 8 and np.all(np.diff(splits) > 0)
    err_dev = np.mean((mids[codes].astype(np.float64) - vals) ** 2)
    err_ref = np.mean((ref["values"][ref["bins"]] - vals) ** 2)
    assert err_dev <= err_ref * 1.02 + 1e-18, (err_dev, err_ref)
    assert np.all(vals >= np.concatenate([[vals.min()], splits])[codes]) and np.all(vals <= np.concatenate([splits, [vals.max()]])[codes])
    cnt.zero_()
    zc.pack(v, cnt)
    assert int(zc.meta[0]) == 0
