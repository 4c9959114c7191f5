"""The plain-C routing oracle against the fixtures made from the reference and against the torch oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import build as oracle_build
from oracle import moe_oracle as O


@pytest.fixture(scope="module")
def clib():
    lib = C.CDLL(str(oracle_build.build()))
    lib.oracle_topk_indices.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p]
    lib.oracle_softmax_selected.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]
    lib.oracle_route_histogram.argtypes = [C.c_void_p, C.c_int64, C.c_int] + [C.c_void_p] * 4
    lib.oracle_route_histogram.restype = C.c_int64
    return lib


def _topk(clib, x, k):
    x = np.ascontiguousarray(x, dtype=np.float32)
    M, N = x.shape
    idx = np.zeros((M, k), dtype=np.int64)
    assert clib.oracle_topk_indices(x.ctypes.data, M, N, N, k, idx.ctypes.data) == 0
    sc = np.zeros((M, k), dtype=np.float32)
    clib.oracle_softmax_selected(x.ctypes.data, M, N, k, idx.ctypes.data, sc.ctypes.data)
    return sc, idx


def test_topk_fixtures(clib):
    g = np.load(GOLDEN / "topk_c1.npz")
    sc, idx = _topk(clib, g["logits"], 6)
    assert np.array_equal(idx, g["idx_B"].astype(np.int64))
    np.testing.assert_allclose(sc, g["scores_B"], rtol=1e-6, atol=0)
    t = np.load(GOLDEN / "topk_ties.npz")
    sc, idx = _topk(clib, t["logits"], 8)
    assert np.array_equal(idx, t["idx_stable"].astype(np.int64))
    np.testing.assert_allclose(sc, t["scores_ref"], rtol=1e-6, atol=0)
    c4 = np.load(GOLDEN / "topk_c4_rows8.npz")
    big = torch.randn(64, 32768, generator=torch.Generator().manual_seed(0))[:2].numpy()
    _, idx = _topk(clib, big, 2048)
    assert np.array_equal(idx, c4["idx_stable"][:2].astype(np.int64))


def test_topk_special_values_and_random_agreement(clib):
    x = np.array([[0.0, -0.0, 1.0, np.nan, -0.0, 0.0, -np.inf, np.inf]], dtype=np.float32)
    _, idx = _topk(clib, x, 8)
    assert idx.tolist() == [[3, 7, 2, 0, 1, 4, 5, 6]]
    g = torch.Generator().manual_seed(4)
    for M, N, k in ((50, 33, 5), (20, 257, 64), (7, 1000, 1000)):
        q = torch.round(torch.randn(M, N, generator=g) * 3) / 3
        _, idx = _topk(clib, q.numpy(), k)
        assert np.array_equal(idx, O.stable_topk(q, k)[1].numpy())


def test_histogram_fixture_and_random(clib):
    g = np.load(GOLDEN / "histogram.npz")
    ids = np.ascontiguousarray(g["topk_idx"].reshape(-1), dtype=np.int32)
    E = int(g["E"])
    counts, offsets = np.zeros(E, np.int32), np.zeros(E + 1, np.int32)
    perm, inv = np.zeros(ids.size, np.int32), np.zeros(ids.size, np.int32)
    bad = clib.oracle_route_histogram(ids.ctypes.data, ids.size, E, counts.ctypes.data, offsets.ctypes.data,
                                      perm.ctypes.data, inv.ctypes.data)
    assert bad == 0
    assert np.array_equal(counts, g["counts"]) and np.array_equal(offsets[1:], g["offsets_inclusive"])
    assert np.array_equal(perm, g["perm_stable"]) and np.array_equal(inv, g["inv"])
    rnd = torch.randint(0, 37, (5000,), generator=torch.Generator().manual_seed(8), dtype=torch.int32)
    c, o, p, i = O.route_histogram(rnd.view(-1, 1), 37)
    counts, offsets = np.zeros(37, np.int32), np.zeros(38, np.int32)
    perm, inv = np.zeros(5000, np.int32), np.zeros(5000, np.int32)
    ids = rnd.numpy()
    clib.oracle_route_histogram(ids.ctypes.data, 5000, 37, counts.ctypes.data, offsets.ctypes.data, perm.ctypes.data,
                                inv.ctypes.data)
    assert np.array_equal(counts, c.numpy()) and np.array_equal(offsets, o.numpy())
    assert np.array_equal(perm, p.numpy()) and np.array_equal(inv, i.numpy())
