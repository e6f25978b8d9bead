"""GPU numerics of the GLM kernels against plain PyTorch fp32/fp64 references."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _random_csr(rows, dim, nnz_lo, nnz_hi, seed, binary=False, zipf=True):
    from sketchml_b200.data import CSRMatrix
    rng = np.random.default_rng(seed)
    counts = rng.integers(nnz_lo, nnz_hi + 1, rows)
    rowptr = np.zeros(rows + 1, np.int64)
    rowptr[1:] = np.cumsum(counts)
    cols = np.empty(rowptr[-1], np.int32)
    for r in range(rows):
        if zipf:
            p = 1.0 / np.arange(1, dim + 1) ** 1.1
            c = rng.choice(dim, counts[r], replace=False, p=p / p.sum())
        else:
            c = rng.choice(dim, counts[r], replace=False)
        cols[rowptr[r]:rowptr[r + 1]] = np.sort(c)
    vals = None if binary else torch.from_numpy(rng.normal(size=rowptr[-1]).astype(np.float32))
    labels = torch.from_numpy(np.where(rng.random(rows) < 0.5, 1.0, -1.0).astype(np.float32))
    return CSRMatrix(torch.from_numpy(rowptr), torch.from_numpy(cols), vals, labels, dim)


def _ref_grad(m, w, loss, lo, hi, lam):
    b = m.slice_rows(lo, hi)
    w64 = w.double().cpu()
    pre = loss.predict(w64, b)
    y = b.labels.double()
    coef = -loss.grad(pre, y) / (hi - lo)
    g = torch.zeros(m.dim, dtype=torch.float64)
    g.index_add_(0, b.cols.long(), coef[b.row_ids()] * b.dense_values(torch.float64))
    touched = g.abs() > 0
    full = g + lam * w64 * touched
    keep = touched & (full.abs() > 1e-8)
    return full, keep, float(loss.loss(pre, y).sum())


@pytest.mark.parametrize("loss_name,binary,nnz", [("log", True, (20, 20)), ("hinge", False, (1, 70)), ("square", False, (150, 260))])
def test_grad_compact_matches_reference(loss_name, binary, nnz):
    from sketchml_b200.models.loss import L2HingeLoss, L2LogLoss, L2SquareLoss
    from sketchml_b200.ops import DeviceCSR, GlmState, compact_gradient, glm_grad
    dev = torch.device("cuda")
    loss = {"log": L2LogLoss, "hinge": L2HingeLoss, "square": L2SquareLoss}[loss_name](1e-3)
    dim, rows = 20000, 700
    m = _random_csr(rows, dim, nnz[0], nnz[1], seed=nnz[0], binary=binary)
    csr = DeviceCSR(m, dev)
    w = (torch.randn(dim) * 0.3).float()
    wd = w.to(dev)
    st = GlmState.create(dim, dim, dev)
    lo, hi = 37, 650
    st.partials.zero_()
    glm_grad(csr, [(lo, hi)], wd, st, loss.loss_id, hi - lo, hot=4096)
    compact_gradient(st, wd, loss.lam)
    torch.cuda.synchronize()
    assert int(st.status.item()) == 0
    n = int(st.meta[0])
    keys = st.keys[:n].cpu().long()
    vals = st.vals[:n].cpu().double()
    full, keep, ref_loss = _ref_grad(m, w, loss, lo, hi, loss.lam)
    ref_keys = torch.nonzero(keep).flatten()
    # coordinates whose magnitude sits at the 1e-8 filter may differ; compare as dense vectors
    got = torch.zeros(dim, dtype=torch.float64)
    got[keys] = vals
    ref = torch.where(keep, full, torch.zeros_like(full))
    assert torch.all(keys[1:] > keys[:-1])
    assert abs(n - ref_keys.numel()) <= max(2, ref_keys.numel() // 1000)
    scale = float(ref.abs().max())
    assert float((got - ref).abs().max()) <= 2e-5 * max(scale, 1.0) + 1e-7
    assert abs(float(st.partials[1]) - ref_loss) <= 1e-3 * max(1.0, abs(ref_loss))
    # accumulator and bitmap are clean for the next step
    assert float(st.g.abs().max()) == 0.0 and int(st.bitmap.abs().max()) == 0


def test_wraparound_segments_and_validation():
    from sketchml_b200.models.loss import L2LogLoss
    from sketchml_b200.ops import DeviceCSR, GlmState, compact_gradient, glm_grad, glm_validate
    from sketchml_b200.trainer import validation_counts
    dev = torch.device("cuda")
    loss = L2LogLoss(0.0)
    dim, rows = 5000, 300
    m = _random_csr(rows, dim, 5, 40, seed=3)
    csr = DeviceCSR(m, dev)
    w = (torch.randn(dim) * 0.5).float()
    wd = w.to(dev)
    st = GlmState.create(dim, dim, dev)
    st.partials.zero_()
    glm_grad(csr, [(250, 300), (0, 70)], wd, st, loss.loss_id, 120, hot=1024)
    compact_gradient(st, wd, 0.0)
    n = int(st.meta[0])
    got = torch.zeros(dim, dtype=torch.float64)
    got[st.keys[:n].cpu().long()] = st.vals[:n].cpu().double()
    f1, k1, _ = _ref_grad(m, w, loss, 250, 300, 0.0)
    f2, k2, _ = _ref_grad(m, w, loss, 0, 70, 0.0)
    ref = f1 * 50 / 120 + f2 * 70 / 120
    ref = torch.where(ref.abs() > 1e-8, ref, torch.zeros_like(ref))
    assert float((got - ref).abs().max()) < 1e-5
    acc = glm_validate(csr, wd, loss.loss_id, st.status).cpu()
    pre = loss.predict(w.double(), m)
    refc = validation_counts(pre, m.labels.double(), loss)
    assert abs(acc[0] - refc[0]) < 1e-3 * refc[0]
    assert [int(x) for x in acc[1:6]] == [int(x) for x in refc[1:6]]


def test_dense_kind_decision_and_values():
    from sketchml_b200.models.loss import L2SquareLoss
    from sketchml_b200.ops import DeviceCSR, GlmState, compact_gradient, glm_grad
    dev = torch.device("cuda")
    loss = L2SquareLoss(1e-2)
    dim, rows = 600, 200
    m = _random_csr(rows, dim, 100, 200, seed=9, zipf=False)
    csr = DeviceCSR(m, dev)
    w = torch.randn(dim).float()
    wd = w.to(dev)
    st = GlmState.create(dim, dim, dev, allow_dense=True)
    st.partials.zero_()
    glm_grad(csr, [(0, rows)], wd, st, loss.loss_id, rows, hot=256)
    compact_gradient(st, wd, loss.lam)
    assert int(st.meta[1]) == 2
    full, keep, _ = _ref_grad(m, w, loss, 0, rows, 0.0)
    ref = full + loss.lam * w.double()
    assert float((st.dense_vals.cpu().double() - ref).abs().max()) < 1e-4 * float(ref.abs().max())


def test_device_generator_statistics():
    from sketchml_b200.data.synthetic import SyntheticSpec, zipf_inverse_cdf
    from sketchml_b200.ops import generate_gpu
    spec = SyntheticSpec(rows=20000, dim=100000, nnz_per_row=20, zipf_s=1.1, values="binary", task="logistic", seed=5)
    csr, w = generate_gpu(spec, 0, spec.rows, "cuda")
    cols = csr.cols[:csr.nnz].cpu().numpy().reshape(spec.rows, 20)
    assert cols.min() >= 0 and cols.max() < spec.dim
    srt = np.sort(cols, axis=1)
    assert (srt[:, 1:] != srt[:, :-1]).all(), "columns repeat inside a row"
    # head mass of the Zipf law: column 0 is in most rows, and rank frequencies decay
    f0 = (cols == 0).any(axis=1).mean()
    exp = zipf_inverse_cdf(np.random.default_rng(0).random(400000), spec.dim, 1.1)
    p0 = (exp == 0).mean()
    assert abs(f0 - (1 - (1 - p0) ** 20)) < 0.08
    lab = csr.labels.cpu().numpy()
    assert set(np.unique(lab)) <= {-1.0, 1.0} and 0.2 < (lab > 0).mean() < 0.8
    wn = w.cpu().numpy()
    assert abs((wn != 0).mean() - 0.1) < 0.01
    spec2 = SyntheticSpec(rows=2000, dim=5000, nnz_per_row=200, zipf_s=0.0, values="uniform_l2", task="svm", seed=6)
    c2, _ = generate_gpu(spec2, 100, 2000, "cuda")
    v = c2.values[:c2.nnz].cpu().numpy().reshape(2000, 200)
    assert np.allclose((v ** 2).sum(axis=1), 1.0, atol=1e-4)


@pytest.mark.parametrize("binary", [True, False])
def test_transposed_index_gradient_matches_scatter_path(binary):
    from sketchml_b200.models.loss import L2LogLoss
    from sketchml_b200.ops import DeviceCSR, GlmState, compact_gradient, glm_grad
    from sketchml_b200.ops.transposed import build_batch_index, glm_grad_transposed
    dev = torch.device("cuda")
    loss = L2LogLoss(1e-3)
    dim, rows = 30000, 6000
    m = _random_csr(rows, dim, 1, 60, seed=21, binary=binary)
    csr = DeviceCSR(m, dev)
    w = (torch.randn(dim) * 0.3).float().to(dev)
    st = GlmState.create(dim, dim, dev)
    lo, hi = 2000, 4000
    st.partials.zero_()
    glm_grad(csr, [(lo, hi)], w, st, loss.loss_id, hi - lo, hot=2048)
    compact_gradient(st, w, loss.lam)
    n = int(st.meta[0])
    ref = torch.zeros(dim, dtype=torch.float64)
    ref[st.keys[:n].cpu().long()] = st.vals[:n].cpu().double()
    ref_loss = float(st.partials[1])
    bi = build_batch_index(csr, lo, hi)
    assert bi.n_short + bi.n_medium + len(torch.unique(bi.long_col)) == bi.n_cols
    assert torch.all(bi.ucols[1:] > bi.ucols[:-1]) and int(bi.colptr[-1]) == int(csr.rowptr[hi] - csr.rowptr[lo])
    coef = torch.zeros(hi - lo, device=dev)
    out = torch.zeros(dim, device=dev)
    st.partials.zero_()
    glm_grad_transposed(csr, bi, w, coef, out, st.partials, st.status, loss.loss_id, loss.lam)
    got = torch.zeros(dim, dtype=torch.float64)
    got[bi.ucols.cpu().long()] = out[:bi.n_cols].cpu().double()
    assert int(st.status.item()) == 0
    assert abs(float(st.partials[1]) - ref_loss) < 1e-3 * abs(ref_loss)
    assert abs(bi.n_cols - n) <= 3          # the scatter path drops |v| <= 1e-8, this one keeps them
    assert float((got - ref).abs().max()) < 2e-6 * max(1.0, float(ref.abs().max())) + 2e-8


@pytest.mark.parametrize("binary", [True, False])
@pytest.mark.parametrize("tile_rows_max,rows", [(49152, 2000), (512, 2000), (1000, 5003), (49152, 60000)])
def test_row_tiled_index_matches_the_per_column_form(binary, tile_rows_max, rows, monkeypatch):
    """The row-tiled index (tile coefficients in shared memory, partial sums per (tile, column) pair added in
    tile order) gives the gradient of the per-column form up to the order of the float adds, the same keys,
    and the same bits on every repetition."""
    from sketchml_b200.models.loss import L2LogLoss
    from sketchml_b200.ops import DeviceCSR, GlmState
    from sketchml_b200.ops import transposed as T
    monkeypatch.setattr(T, "TILE_ROWS_MAX", tile_rows_max)
    dev = torch.device("cuda")
    loss = L2LogLoss(1e-3)
    dim = 30000
    m = _random_csr(rows + 500, dim, 1, 40, seed=33, binary=binary)
    csr = DeviceCSR(m, dev)
    w = (torch.randn(dim) * 0.3).float().to(dev)
    st = GlmState.create(dim, dim, dev)
    lo, hi = 250, 250 + rows
    plain, tiled = T.build_batch_index(csr, lo, hi), T.build_batch_index(csr, lo, hi, tiled=True)
    assert tiled.tiled is not None and tiled.tiled.n_tiles == -(-rows // tile_rows_max)
    assert torch.equal(plain.ucols, tiled.ucols) and int(tiled.tiled.pair_ptr[-1]) == int(csr.rowptr[hi] - csr.rowptr[lo])
    assert int(tiled.tiled.col_pair_ptr[-1]) == tiled.tiled.n_pairs
    coef = torch.zeros((rows + 3) // 4 * 4, device=dev)
    outs = []
    for bi in (plain, tiled, tiled):
        out = torch.full((dim,), 7.0, device=dev)
        st.partials.zero_()
        T.glm_grad_transposed(csr, bi, w, coef, out, st.partials, st.status, loss.loss_id, loss.lam)
        assert int(st.status.item()) == 0
        outs.append(out[:bi.n_cols].clone())
    assert torch.equal(outs[1], outs[2])
    assert float((outs[0].double() - outs[1].double()).abs().max()) < 2e-6 * max(1.0, float(outs[0].abs().max()))

