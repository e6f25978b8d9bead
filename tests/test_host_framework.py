"""Host framework on CPU: config, parsers, data set cursor, losses, gradient kinds,
optimizers, compression API, trainer (single process), checkpoints and export."""
import argparse
import math
import os

import numpy as np
import pytest
import torch

from sketchml_b200 import config as C
from sketchml_b200.config import MLConf


def test_conf_defaults_and_spark_pairs():
    c = MLConf()
    assert (c.valid_ratio, c.epoch_num, c.batch_sample_ratio, c.learn_rate, c.learn_decay) == (0.25, 100, 0.1, 0.1, 0.9)
    assert (c.l1_reg, c.l2_reg, c.compressor, c.quant_bin_num) == (0.1, 0.1, "Sketch", 256)
    assert (c.sketch_group_num, c.sketch_row_num, c.sketch_col_ratio, c.fixed_point_bit_num) == (8, 2, 0.3, 8)
    c = MLConf.from_spark_pairs(["spark.sketchml.algo=SupportVectorMachine", "spark.sketchml.feature.num=100",
                                 "spark.sketchml.minmaxsketch.row.num=3", "spark.sketchml.batch.sample.ratio=0.3",
                                 "spark.sketchml.gradient.compressor=Zip", "spark.sketchml.input.format=dummy"])
    assert c.algo == C.ML_SUPPORT_VECTOR_MACHINE and c.feature_num == 100 and c.sketch_row_num == 3
    assert c.batch_num == 4 and c.compressor == "Zip" and c.format == "dummy"
    for bad in (dict(algo="Tree"), dict(format="parquet"), dict(compressor="Gzip"), dict(sketch_row_num=9),
                dict(fixed_point_bit_num=30), dict(sketch_k=100), dict(batch_sample_ratio=0.0)):
        with pytest.raises(ValueError):
            MLConf(**bad)
    with pytest.raises(KeyError):
        MLConf.from_spark_pairs(["spark.sketchml.nope=1"])
    p = argparse.ArgumentParser()
    C.add_arguments(p)
    ns = p.parse_args(["--algo", "lr", "--feature-num", "77", "--quantization-bin-num", "64", "--conf",
                       "spark.sketchml.learn.rate=0.5", "--optimizer", "adam"])
    c = C.conf_from_args(ns)
    assert (c.feature_num, c.quant_bin_num, c.learn_rate, c.optimizer) == (77, 64, 0.5, "adam")
    assert MLConf(algo="linreg").use_neg_y is False and MLConf(algo="lr").use_neg_y is True
    assert MLConf.from_dict(c.to_dict()).to_dict() == c.to_dict()


def test_parsers_and_dataset(tmp_path):
    from sketchml_b200.data import DataSet, load_data, parse_lines, shard_rows, split_train_valid
    m = parse_lines(["1 3:0.5 1:2.0", "0 2:1.5", "", "-1 0:1 4:1"], "libsvm", 5)
    assert m.rows == 3 and m.cols.tolist() == [1, 3, 2, 0, 4] and m.values.tolist() == [2.0, 0.5, 1.5, 1.0, 1.0]
    assert m.labels.tolist() == [1.0, -1.0, -1.0]
    assert parse_lines(["0.7 1:1"], "libsvm", 5, neg_y=False).labels.tolist() == [pytest.approx(0.7)]
    c = parse_lines(["1,0.5,0,2"], "csv", 3)
    assert c.cols.tolist() == [0, 1, 2] and c.values.tolist() == [0.5, 0.0, 2.0]
    d = parse_lines(["1,4,2", "0,1"], "dummy", 5)
    assert d.values is None and d.cols.tolist() == [2, 4, 1] and d.dense_values(torch.float32).tolist() == [1, 1, 1]
    with pytest.raises(ValueError):
        parse_lines(["1 9:1"], "libsvm", 5)
    with pytest.raises(ValueError):
        parse_lines(["1 1:1"], "arff", 5)
    f = tmp_path / "d.libsvm"
    f.write_text("\n".join(f"{i % 2} {i % 7}:1 {7 + i % 3}:0.5" for i in range(10)))
    a, off_a, total = load_data(str(f), "libsvm", 10, 0, 3)
    b, off_b, _ = load_data(str(f), "libsvm", 10, 2, 3)
    assert total == 10 and a.rows == 4 and b.rows == 3 and (off_a, off_b) == (0, 7)
    assert [shard_rows(10, r, 3) for r in range(3)] == [(0, 4), (4, 7), (7, 10)]
    ds = DataSet(a)
    assert ds.batch_size(0.6) == 2 and ds.looping_segments(3) == [(0, 3)] and ds.looping_segments(3) == [(3, 4), (0, 2)]
    assert ds.read_index == 2 and ds.looping_read(4).rows == 4
    big = parse_lines([f"1 {i % 50}:1" for i in range(2000)], "libsvm", 50)
    tr, va = split_train_valid(big, 0.25, seed=3, global_offset=100)
    tr2, va2 = split_train_valid(big, 0.25, seed=3, global_offset=100)
    assert tr.rows + va.rows == 2000 and abs(va.rows / 2000 - 0.25) < 0.04 and tr.rows == tr2.rows
    assert split_train_valid(big, 0.0, 0)[1].rows == 0


def test_native_parser_matches_python_parser():
    from sketchml_b200.data import parse_lines, parse_text_native
    rng = np.random.default_rng(0)
    lines = []
    for i in range(300):
        idx = rng.choice(500, rng.integers(1, 30), replace=True)
        lines.append(f"{rng.choice([0, 1, -1, 0.5])} " + " ".join(f"{j}:{rng.normal():.6g}" for j in idx))
    for neg in (True, False):
        a = parse_lines(lines, "libsvm", 500, neg, torch.float64)
        b = parse_text_native("\n".join(lines) + "\n", "libsvm", 500, neg, torch.float64)
        assert torch.equal(a.rowptr, b.rowptr) and torch.equal(a.cols, b.cols) and torch.equal(a.labels, b.labels)
        assert torch.allclose(a.values, b.values, rtol=0, atol=1e-12)
    d = ["1,5,3,9", "0,2", "", "1,7,7"]
    a, b = parse_lines(d, "dummy", 10), parse_text_native("\n".join(d), "dummy", 10)
    assert torch.equal(a.cols, b.cols) and torch.equal(a.values, b.values)
    c = ["1,0.5,0,2", "0, 1.5 ,2,3"]
    a, b = parse_lines(c, "csv", 3), parse_text_native("\n".join(c), "csv", 3)
    assert torch.equal(a.cols, b.cols) and torch.equal(a.values, b.values) and torch.equal(a.labels, b.labels)
    assert parse_text_native("1,4,2\n", "dummy", 5).values is None
    with pytest.raises(ValueError):
        parse_text_native("1 9:1\n", "libsvm", 5)
    with pytest.raises(ValueError):
        parse_text_native("1 a:1\n", "libsvm", 5)


def test_losses_match_reference_formulas():
    from sketchml_b200.models.loss import L2HingeLoss, L2LogLoss, L2SquareLoss
    pre = torch.tensor([-30.0, -2.0, 0.0, 0.5, 1.0, 3.0, 25.0], dtype=torch.float64)
    for yv in (1.0, -1.0):
        y = torch.full_like(pre, yv)
        z = pre * y
        lg = L2LogLoss(0.1)
        ref_loss = [math.exp(-v) if v > 18 else (-v if v < -18 else math.log(1 + math.exp(-v))) for v in z.tolist()]
        ref_grad = [yv * math.exp(-v) if v > 18 else (yv if v < -18 else yv / (1 + math.exp(v))) for v in z.tolist()]
        assert torch.allclose(lg.loss(pre, y), torch.tensor(ref_loss, dtype=torch.float64))
        assert torch.allclose(lg.grad(pre, y), torch.tensor(ref_grad, dtype=torch.float64))
        h = L2HingeLoss(0.1)
        assert h.loss(pre, y).tolist() == [max(0.0, 1 - v) for v in z.tolist()]
        assert h.grad(pre, y).tolist() == [yv if v <= 1 else 0.0 for v in z.tolist()]
    s = L2SquareLoss(0.0)
    y = torch.tensor([1.0, 0.0, 2.0, 0.5, 1.0, -1.0, 0.0], dtype=torch.float64)
    assert torch.allclose(s.loss(pre, y), 0.5 * (pre - y) ** 2) and torch.allclose(s.grad(pre, y), y - pre)
    w = torch.tensor([3.0, 4.0])
    assert L2LogLoss(0.5).get_reg(w) == pytest.approx(2.5) and not L2LogLoss(1e-9).is_l2_reg and s.get_reg(w) == 0.0


def test_gradient_kinds_and_compress_factory():
    from sketchml_b200.gradient import (DenseDoubleGradient, Kind, SparseDoubleGradient, ZeroGradient, compress,
                                        evaluate_compression, sum_gradients)
    d = DenseDoubleGradient(9, torch.tensor([0, 1e-9, 2.0, 0, 0, -3.0, 0, 0, 0]))
    assert d.count_nnz() == 2 and d.to_auto().kind is Kind.SparseDouble
    sp = d.to_sparse()
    assert sp.indices.tolist() == [2, 5] and sp.values.tolist() == [2.0, -3.0]
    dense7 = DenseDoubleGradient(9, torch.arange(9.0) + 1)
    assert dense7.to_auto().kind is Kind.DenseDouble
    with pytest.raises(ValueError):
        SparseDoubleGradient(9, torch.tensor([3, 2]), torch.tensor([1.0, 1.0]))
    with pytest.raises(ValueError):
        SparseDoubleGradient(9, torch.tensor([9]), torch.tensor([1.0]))
    assert ZeroGradient.plus_by(sp) is sp
    total = sum_gradients(9, [sp, ZeroGradient, sp])
    assert total.to_dense().values.tolist() == [0, 0, 4.0, 0, 0, -6.0, 0, 0, 0]
    rng = np.random.default_rng(0)
    dim, n = 200000, 5000
    keys = torch.from_numpy(np.sort(rng.choice(dim, n, replace=False)).astype(np.int32))
    g = SparseDoubleGradient(dim, keys, torch.from_numpy(rng.laplace(0, 1e-3, n)))
    for name, tol in (("Sketch", 0.8), ("FixedPoint", 0.9), ("Zip", 0.05), ("Float", 1e-6), ("None", 0.0)):
        conf = MLConf(feature_num=dim, compressor=name, dtype="float64")
        c = compress(g, conf, step=2, rank=0, world=1)
        ev = evaluate_compression(g, c)
        assert ev["rel_l2"] <= tol, name
        back = c.to_auto()
        assert back.kind in (Kind.SparseDouble, Kind.SparseFloat)
        assert back.to_sparse().indices.tolist() == keys.tolist()
        if name in ("Sketch", "Zip", "FixedPoint"):
            before = c.to_dense().values.clone()
            c.times_by(0.5)
            assert torch.allclose(c.to_dense().values, 0.5 * before, rtol=1e-5, atol=1e-12)
            assert c.nbytes() < g.nbytes()
    dg = DenseDoubleGradient(3000, torch.from_numpy(rng.normal(size=3000)))
    cd = compress(dg, MLConf(feature_num=3000, dtype="float64"))
    assert cd.kind is Kind.Sketch and cd.to_auto().kind is Kind.DenseDouble and cd.nbytes() < 3000 * 2


def test_optimizers_follow_reference_rules():
    from sketchml_b200.gradient import DenseDoubleGradient, SparseDoubleGradient
    from sketchml_b200.optim import Adam, GradientDescent
    sgd = GradientDescent(4, 0.1, 0.9, 0.5)
    assert sgd.batch_num == 2
    w = torch.zeros(4, dtype=torch.float64)
    sgd.update(SparseDoubleGradient(4, torch.tensor([1, 3]), torch.tensor([1.0, -2.0])), w)
    assert w.tolist() == [0, -0.1, 0, 0.2]
    sgd.advance(); sgd.advance()
    assert sgd.epoch == 1 and sgd.learning_rate() == pytest.approx(0.1 / math.sqrt(1.9))
    ad = Adam(4, 0.1, 0.9, 0.5)
    w = torch.zeros(4, dtype=torch.float64)
    g = SparseDoubleGradient(4, torch.tensor([2]), torch.tensor([0.5]))
    ad.update(g, w)
    m, v = 0.1 * 0.5, 0.001 * 0.25
    step = 0.1 * math.sqrt(1 - 0.999) * m / ((1 - 0.9) * (math.sqrt(v) + 1e-8))
    assert w[2].item() == pytest.approx(-step) and w[0].item() == 0 and ad.m[2].item() == pytest.approx(m)
    ad.advance(); ad.advance()                 # epoch 1, batch 0 -> beta powers advance on the next update
    ad.update(DenseDoubleGradient(4, torch.zeros(4)), w)
    assert ad.beta1_t == pytest.approx(0.81) and ad.beta2_t == pytest.approx(0.999 ** 2)
    ad.advance()
    ad.update(DenseDoubleGradient(4, torch.zeros(4)), w)
    assert ad.beta1_t == pytest.approx(0.81)
    sd = ad.state_dict()
    ad2 = Adam(4, 0.1, 0.9, 0.5)
    ad2.load_state_dict(sd)
    assert torch.equal(ad2.m, ad.m) and ad2.beta2_t == ad.beta2_t and (ad2.epoch, ad2.batch) == (ad.epoch, ad.batch)
    # L2 on the gradient's own coordinates only; L1 truncation
    w = torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=torch.float64)
    g = SparseDoubleGradient(4, torch.tensor([0, 2]), torch.tensor([0.5, 0.5]))
    GradientDescent.l2_reg(g, w, 0.1)
    assert g.values.tolist() == pytest.approx([0.6, 0.8])
    d = DenseDoubleGradient(3, torch.tensor([0.05, -0.05, 0.5]))
    GradientDescent.l1_reg(d, 0.1, 0.1)
    assert d.values.tolist() == pytest.approx([0.0, -0.15, 0.5])


def test_compress_api_and_demo(capsys):
    from sketchml_b200 import compress as K
    rng = np.random.default_rng(1)
    q = K.Quantizer.new_quantizer(K.QuantizationType.QUANTILE, 64)
    v = rng.normal(size=5000)
    q.quantize(v)
    assert q.get_bin_num() <= 64 and q.index_of(v[0]) == q.get_bins()[0] and len(q.to_java_stream()) > 5000
    sk = K.HeapQuantileSketch()
    sk.update(v)
    assert abs(sk.get_quantile(0.5)) < 0.1 and sk.get_quantile(0.0) == v.min() and sk.get_quantile(1.0) == v.max()
    mm = K.MinMaxSketch(2, 100, 10, seed=3)
    mm.insert([5, 6], [12, 20])
    assert mm.query(5) in (12, 20) and abs(mm.query(6) - 10) <= 10
    for enc in (K.DeltaBinaryEncoder(), K.DeltaAdaptiveEncoder()):
        enc.encode([1, 5, 900, 70000])
        assert enc.decode().tolist() == [1, 5, 900, 70000] and enc.nbytes_wire() > 0
    h = K.HuffmanEncoder()
    h.encode([1, 1, 1, 2, 3])
    assert h.decode().tolist() == [1, 1, 1, 2, 3]
    sc = K.SparseVectorCompressor(quant_bin_num=64)
    keys = np.sort(rng.choice(100000, 3000, replace=False))
    vals = rng.normal(size=3000)
    sc.parallel_compress_sparse(keys, vals)
    k2, v2 = sc.decompress_sparse()
    assert np.array_equal(k2, keys) and sc.size() == 3000 and 12 * 3000 / sc.memory_bytes() > 3 and len(sc.to_java_stream()) > 0
    sc.times_by(2.0)
    assert np.allclose(sc.decompress_sparse()[1], 2 * v2)
    with pytest.raises(K.oracle.SketchMLError):
        sc.compress_sparse([1, 2], [1.0])
    dc = K.DenseVectorCompressor(K.QuantizationType.UNIFORM, 32)
    dc.compress_dense(vals)
    assert np.abs(dc.decompress_dense() - vals).max() <= (vals.max() - vals.min()) / 32 and 8 * 3000 / dc.memory_bytes() > 4
    dc.compress_sparse([0, 4], [1.0, 2.0])
    assert len(dc.decompress_dense()) == 5            # maxKey + 1 (the reference allocates one short)
    K.Parallel.set_parallelism(4)
    assert K.Parallel.get_parallelism() == 4
    from sketchml_b200.compress import app
    d, s = app.main(400000, 0)
    assert d["rate"] > 5 and s["rate"] > 2.5 and "compression rate" in capsys.readouterr().out


def _conf(**kw):
    base = dict(algo="lr", format="synthetic", feature_num=3000, syn_rows=3000, syn_nnz_per_row=10, epoch_num=3,
                learn_rate=0.5, l2_reg=1e-4, valid_ratio=0.2, batch_sample_ratio=0.25, device="cpu", dtype="float64",
                quant_bin_num=64, sketch_row_num=3, sketch_col_ratio=0.5, seed=2)
    base.update(kw)
    return MLConf(**base)


@pytest.mark.parametrize("algo", ["lr", "svm", "linreg"])
@pytest.mark.parametrize("compressor", ["Sketch", "None", "Zip", "FixedPoint", "Float"])
def test_trainer_single_process(algo, compressor):
    from sketchml_b200.trainer import Trainer
    kw = {}
    if algo == "linreg":
        kw = dict(syn_values="normal", learn_rate=0.05, syn_noise=0.1)
    t = Trainer(_conf(algo=algo, compressor=compressor, **kw))
    t.load_data()
    h = t.train()
    assert len(h["train_loss"]) == 3 and all(np.isfinite(h["train_loss"])) and h["train_loss"][-1] < h["train_loss"][0]
    assert t.metrics.of("validate")[-1]["valid_num"] > 0 and t.metrics.of("epoch")[-1]["samples_per_s"] > 0
    if compressor == "Sketch":
        ex = t.metrics.of("exchange")
        assert ex and ex[-1]["ratio_vs_12B"] > 2
    if algo == "linreg":
        assert set(t.train_data.matrix.labels.tolist()) != {-1.0, 1.0}     # raw targets are kept for regression
    t.close()


def test_adam_and_recompress_options():
    from sketchml_b200.trainer import Trainer
    t = Trainer(_conf(optimizer="adam", learn_rate=0.01, recompress_sum=True, key_encoder="delta_adaptive", cell_bits=0,
                      extras={"eval_compression": True}))
    t.load_data()
    h = t.train()
    assert h["train_loss"][-1] < h["train_loss"][0] and t.metrics.of("exchange")[-1]["cosine"] > 0.5


def test_checkpoint_resume_and_export(tmp_path):
    from sketchml_b200.trainer import Trainer
    from sketchml_b200.utils import export_model, import_model, load_checkpoint
    full = Trainer(_conf(epoch_num=4, compressor="None"))
    full.load_data()
    full.train()
    a = Trainer(_conf(epoch_num=2, compressor="None", checkpoint_dir=str(tmp_path), checkpoint_every=2,
                      export_path=str(tmp_path / "model.txt")))
    a.load_data()
    a.train()
    ck = tmp_path / "epoch_0002.ckpt"
    blob = load_checkpoint(str(ck))
    assert blob["epoch"] == 2 and blob["step"] == 8
    b = Trainer(_conf(epoch_num=4, compressor="None", resume=str(ck)))
    b.load_data()
    h = b.train()
    assert len(h["train_loss"]) == 2 and torch.allclose(b.model.weights, full.model.weights, atol=1e-12)
    w = import_model(str(tmp_path / "model.txt"), torch.float64)
    assert torch.allclose(w, a.model.weights) and torch.equal(import_model(str(tmp_path / "model.txt.pt")), a.model.weights.float())
    bad = tmp_path / "bad.ckpt"
    blob["model"]["weights"][0] += 1
    torch.save(blob, bad)
    with pytest.raises(ValueError):
        load_checkpoint(str(bad))
    from sketchml_b200 import cli
    assert cli.main(["export", str(ck), str(tmp_path / "m2.txt")]) == 0 and os.path.exists(tmp_path / "m2.txt.pt")


def test_rank_sum_auc_matches_pair_counting():
    """The rank-sum AUC (ValidationUtil.scala:69-82) against the definition: the fraction of
    (positive, negative) pairs ranked correctly; the reference's 0-based variant is 1 / N lower."""
    import numpy as np
    from sketchml_b200.utils import rank_sum_auc
    rng = np.random.default_rng(0)
    y = np.where(rng.random(400) < 0.3, 1.0, -1.0)
    s = rng.normal(size=400) + 0.8 * (y == 1)
    pos, neg = s[y == 1], s[y != 1]
    want = (pos[:, None] > neg[None, :]).mean()
    assert abs(rank_sum_auc(s, y) - want) < 1e-12
    assert abs(rank_sum_auc(s, y, java_compat=True) - (want - 1.0 / len(neg))) < 1e-12


def test_trainer_reports_auc_when_asked():
    from sketchml_b200.config import MLConf
    from sketchml_b200.trainer import Trainer
    conf = MLConf(algo="lr", format="synthetic", feature_num=2000, syn_rows=4000, syn_nnz_per_row=10, epoch_num=2,
                  batch_sample_ratio=0.25, learn_rate=0.5, l2_reg=1e-5, valid_ratio=0.25, device="cpu", dtype="float64",
                  compressor="None", extras={"auc": True})
    t = Trainer(conf)
    t.load_data()
    t.train()
    v = t.validate(99)
    assert 0.5 < v["auc"] <= 1.0


def test_batch_index_builders_describe_the_same_column_sums(monkeypatch):
    """Both forms of the prepared batch index (per-column lists; row tiles with (tile, column) pairs and
    16-bit local rows) are built with plain tensor ops, so their structure is checked here without a GPU:
    walking either one reproduces the column sums of the batch."""
    import types
    import numpy as np
    from sketchml_b200.ops import transposed as T
    rng = np.random.default_rng(4)
    rows, dim, lo, hi = 900, 400, 100, 800
    counts = rng.integers(1, 12, rows)
    rowptr = np.concatenate([[0], np.cumsum(counts)])
    cols = np.concatenate([np.sort(rng.choice(dim, c, replace=False)) for c in counts]).astype(np.int32)
    cols[rowptr[lo]:rowptr[lo] + 1] = 0
    vals = rng.normal(size=len(cols)).astype(np.float32)
    csr = types.SimpleNamespace(rowptr=torch.from_numpy(rowptr), cols=torch.from_numpy(cols), values=torch.from_numpy(vals))
    coef = rng.normal(size=hi - lo)
    e0, e1 = rowptr[lo], rowptr[hi]
    want = np.zeros(dim)
    r_of = np.repeat(np.arange(rows), counts)[e0:e1] - lo
    np.add.at(want, cols[e0:e1], coef[r_of] * vals[e0:e1])
    plain = T.build_batch_index(csr, lo, hi)
    got = np.zeros(dim)
    cp, ri, sv, uc = plain.colptr.numpy(), plain.rowidx.numpy(), plain.svals.numpy(), plain.ucols.numpy()
    for i, c in enumerate(uc):
        got[c] = np.sum(coef[ri[cp[i]:cp[i + 1]]] * sv[cp[i]:cp[i + 1]])
    assert np.allclose(got, want) and np.all(np.diff(uc) > 0)
    assert plain.n_short + plain.n_medium + len(np.unique(plain.long_col.numpy())) == plain.n_cols
    monkeypatch.setattr(T, "TILE_ROWS_MAX", 96)
    monkeypatch.setattr(T, "PAIR_SEGMENT", 4)
    tiled = T.build_batch_index(csr, lo, hi, tiled=True)
    tp = tiled.tiled
    assert tp.n_tiles == -(-(hi - lo) // 96) and tp.tile_rows % 4 == 0 and tp.n_tiles * tp.tile_rows >= hi - lo
    assert np.array_equal(tiled.ucols.numpy(), uc)
    pair_ptr, lrow = tp.pair_ptr.numpy(), tp.lrow.numpy().astype(np.int64) & 0xFFFF
    tptr, dst, cptr = tp.tile_pair_ptr.numpy(), tp.pair_dst.numpy(), tp.col_pair_ptr.numpy()
    assert np.all(np.diff(pair_ptr) >= 1) and np.all(np.diff(pair_ptr) <= 4) and pair_ptr[-1] == e1 - e0
    assert sorted(dst.tolist()) == list(range(tp.n_pairs)) and cptr[-1] == tp.n_pairs
    partial = np.zeros(tp.n_pairs)
    tv = tiled.svals.numpy()
    for t in range(tp.n_tiles):
        for p in range(tptr[t], tptr[t + 1]):
            e = slice(pair_ptr[p], pair_ptr[p + 1])
            assert np.all(lrow[e] < min(tp.tile_rows, hi - lo - t * tp.tile_rows))
            partial[dst[p]] = np.sum(coef[t * tp.tile_rows + lrow[e]] * tv[e])
    got2 = np.zeros(dim)
    for i, c in enumerate(tiled.ucols.numpy()):
        got2[c] = partial[cptr[i]:cptr[i + 1]].sum()
    assert np.allclose(got2, want)


def test_adam_moment_layouts_are_checked():
    from sketchml_b200.ops.glm import moment_stride
    quad = torch.zeros((10, 4))
    assert moment_stride(None, None) == 1
    assert moment_stride(torch.zeros(10), torch.zeros(10)) == 1
    assert moment_stride(quad[:, 0], quad[:, 1]) == 4
    with pytest.raises(ValueError):
        moment_stride(quad[:, 0], quad[:, 2])
    with pytest.raises(ValueError):
        moment_stride(torch.zeros(10), quad[:, 1])

