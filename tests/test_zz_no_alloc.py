"""skml_compact_noalloc (the compaction entry point that allocates nothing) against the
regular skml_compact, through the exported C symbol.

Some callers of this library cannot create GPU buffers at the point where they need the
compaction (they run inside another framework's callback, or under a frozen memory pool),
so one entry point keeps its scratch inside the library. This test calls it twice in a row
with different gradients and demands the same keys, values, count and clean-up as the
regular entry point, which uses a caller-owned scratch buffer. The second call runs over
the leftovers of the first one in the shared scratch array."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _load():
    from sketchml_b200 import build
    path = build.CUDA_SO
    if not path.exists():
        build.build_cuda()
    lib = C.CDLL(str(path))
    vp, ll = C.c_void_p, C.c_longlong
    lib.skml_compact_noalloc.restype = C.c_int
    lib.skml_compact_noalloc.argtypes = [vp, vp, vp, C.c_int, C.c_float, vp, vp, vp, ll, vp, vp]
    lib.skml_compact.restype = C.c_int
    lib.skml_compact.argtypes = [vp, vp, vp, C.c_int, C.c_float, vp, vp, vp, vp, vp, ll, vp, vp]
    lib.skml_compact_blocks.restype = ll
    lib.skml_compact_blocks.argtypes = [C.c_int]
    return lib


def _case(dim, nnz, seed, dev):
    rng = np.random.default_rng(seed)
    idx = np.sort(rng.choice(dim, nnz, replace=False))
    g = np.zeros(dim, np.float32)
    g[idx] = rng.normal(0, 1e-2, nnz).astype(np.float32)
    g[idx[::7]] = 5e-9                       # below the 1e-8 filter once lambda * w is tiny
    bitmap = np.zeros((dim + 31) // 32 + 4, np.uint32)
    np.bitwise_or.at(bitmap, idx // 32, (1 << (idx % 32)).astype(np.uint32))
    w = (rng.normal(0, 1e-7, dim)).astype(np.float32)
    return (torch.from_numpy(g).to(dev), torch.from_numpy(w).to(dev),
            torch.from_numpy(bitmap.view(np.int32)).to(dev))


def test_noalloc_compaction_matches_regular_entry_point_twice():
    lib = _load()
    dev = torch.device("cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for call, (dim, nnz, seed) in enumerate([(3_000_017, 200_000, 1), (777_777, 350_000, 2)]):
        g, w, bm = _case(dim, nnz, seed, dev)
        g2, bm2 = g.clone(), bm.clone()
        lam = 1e-3
        meta_a = torch.zeros(4, dtype=torch.int64, device=dev)
        meta_b = torch.zeros(4, dtype=torch.int64, device=dev)
        keys_a = torch.full((nnz,), -1, dtype=torch.int32, device=dev)
        keys_b = torch.full((nnz,), -1, dtype=torch.int32, device=dev)
        vals_a = torch.zeros(nnz, dtype=torch.float32, device=dev)
        vals_b = torch.zeros(nnz, dtype=torch.float32, device=dev)
        st_a = torch.zeros(1, dtype=torch.int32, device=dev)
        st_b = torch.zeros(1, dtype=torch.int32, device=dev)
        counts = torch.zeros(int(lib.skml_compact_blocks(dim)) + 1, dtype=torch.int32, device=dev)
        rc = lib.skml_compact(g.data_ptr(), w.data_ptr(), bm.data_ptr(), dim, lam, counts.data_ptr(), meta_a.data_ptr(),
                              keys_a.data_ptr(), vals_a.data_ptr(), None, nnz, st_a.data_ptr(), stream)
        assert rc == 0
        rc = lib.skml_compact_noalloc(g2.data_ptr(), w.data_ptr(), bm2.data_ptr(), dim, lam, meta_b.data_ptr(),
                                      keys_b.data_ptr(), vals_b.data_ptr(), nnz, st_b.data_ptr(), stream)
        assert rc == 0, f"call {call}: rc {rc}"
        torch.cuda.synchronize()
        assert int(st_a.item()) == 0 and int(st_b.item()) == 0
        n = int(meta_a[0])
        assert n == int(meta_b[0]) and 0 < n < nnz
        assert int(meta_b[1]) == 1
        assert torch.equal(keys_a[:n], keys_b[:n])
        assert torch.allclose(vals_a[:n], vals_b[:n], rtol=2e-5, atol=1e-7)   # tolerance of the GLM tests
        assert torch.equal(vals_a[:n], vals_b[:n])                            # and in fact the same bits
        assert float(g2.abs().max()) == 0.0 and int(bm2.abs().max()) == 0


def test_noalloc_rejects_oversized_and_bad_arguments():
    lib = _load()
    dev = torch.device("cuda")
    t = torch.zeros(64, dtype=torch.float32, device=dev)
    i = torch.zeros(64, dtype=torch.int32, device=dev)
    m = torch.zeros(4, dtype=torch.int64, device=dev)
    too_big = 4096 * 4096 * 32 + 1
    rc = lib.skml_compact_noalloc(t.data_ptr(), t.data_ptr(), i.data_ptr(), too_big, 0.0, m.data_ptr(), i.data_ptr(),
                                  t.data_ptr(), 64, i.data_ptr(), None)
    assert rc == -2
    rc = lib.skml_compact_noalloc(None, t.data_ptr(), i.data_ptr(), 64, 0.0, m.data_ptr(), i.data_ptr(), t.data_ptr(),
                                  64, i.data_ptr(), None)
    assert rc == -1
    torch.cuda.synchronize()
