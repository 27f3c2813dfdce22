"""Odd small shapes through every scan: row counts around a warp and a tile edge, dimensions around the vector width and
the 128-wide k-block, k from one to all rows.  Run under the normal library for parity with the CPU oracle and, from
tests/test_gpu_checked.py, under the checked build variant, where every global access of every kernel is range-tested."""
import numpy as np
import pytest

import oracle
from parity import assert_topk_parity

pytestmark = pytest.mark.gpu
NAMES = ["euclidean", "cosine", "dotProduct", "manhattan"]
ROWS = [1, 31, 32, 33, 255, 257]
DIMS = [1, 3, 4, 127, 128, 129]


@pytest.fixture(scope="module")
def vsk():
    import vectorstorekit_b200 as v
    return v


@pytest.fixture(scope="module")
def dev(vsk):
    d = vsk.CUDAAcceleratorStrategy(0).initialize()
    yield d
    d.close()


def _data(n, d, nq, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, d)).astype(np.float32)
    q = rng.standard_normal((nq, d)).astype(np.float32)
    if d == 1:
        x += np.float32(3.0)       # keep cosine away from the 0/0 corner the reference guards with 1e-8
        q += np.float32(3.0)
    return x, q


@pytest.mark.parametrize("metric", NAMES)
@pytest.mark.parametrize("d", DIMS)
def test_flat_search_odd_rows_and_k(vsk, dev, cpu_oracle, metric, d):
    mid = oracle.METRIC_IDS[metric]
    for n in ROWS:
        for nq in (1, 9, 40):                                   # streaming scan, fp32 tile, tensor path
            x, q = _data(n, d, nq, 1000 * n + d)
            ix = vsk.FlatIndex(dev, d, metric)
            ix.add(x)
            for k in sorted({1, min(10, n), n}):
                gd, gi = ix.batchSearch(q, k)
                rd, ri = cpu_oracle.flat_search(mid, q, x, k)
                # a dot product of N(0,1) vectors sits near zero, where "relative" has nothing to hold on to: the
                # scale of the comparison is floored at 0.1 there (sums of d products of magnitude one, rounded in
                # a different order, differ by a few 1e-6)
                assert_topk_parity(gd, gi, rd, ri, dist_rtol=2e-4 if metric == "cosine" and d <= 4 else 1e-4,
                                   atol=1e-5 if metric == "dotProduct" else 1e-6)
            ix.close()


@pytest.mark.parametrize("metric", NAMES)
def test_batch_distances_odd_shapes(vsk, dev, cpu_oracle, metric):
    eng = vsk.CUDAAccelerationEngine(dev)
    mid = oracle.METRIC_IDS[metric]
    for n in ROWS:
        for d in DIMS:
            x, q = _data(n, d, 5, 77 * n + d)
            got = eng.computeDistanceMatrix(q, x, metric)
            ref = cpu_oracle.batch_distances(mid, q, x)
            assert got.shape == (5, n) and np.allclose(got, ref, rtol=2e-4, atol=2e-5)


@pytest.mark.parametrize("d", [3, 128, 129])
def test_filtered_search_odd_shapes(vsk, dev, cpu_oracle, d):
    rng = np.random.default_rng(5 + d)
    for n in (33, 257):
        x, q = _data(n, d, 12, 9 * n + d)
        rm = rng.integers(0, 2 ** 64, n, dtype=np.uint64)
        qm = np.uint64(1) << rng.integers(0, 64, 12).astype(np.uint64)
        for metric in ("euclidean", "manhattan"):
            ix = vsk.FlatIndex(dev, d, metric)
            ix.add(x, rm)
            gd, gi = ix.batchSearch(q, 5, qm)
            rd, ri = cpu_oracle.flat_search(oracle.METRIC_IDS[metric], q, x, 5, rm, qm)
            assert_topk_parity(gd, gi, rd, ri)
            ix.close()


@pytest.mark.parametrize("d", [4, 127, 128])
def test_int8_and_kmeans_odd_shapes(vsk, dev, cpu_oracle, d):
    rng = np.random.default_rng(11 + d)
    n = 257
    x = rng.standard_normal((n, d)).astype(np.float32)
    q = rng.standard_normal((7, d)).astype(np.float32)
    sq = vsk.ScalarQuantizer(dev, per_dim=True)
    scale, offset = sq.train(x)
    rs, ro = cpu_oracle.sq8_train(x, True)
    assert np.array_equal(scale, rs) and np.array_equal(offset, ro)
    codes = sq.quantizeBatch(x)
    rcodes = cpu_oracle.sq8_encode(x, rs, ro)
    assert np.array_equal(codes, rcodes)
    ix = vsk.QuantizedFlatIndex(dev, d, "dotProduct", scale, offset)
    ix.add(codes)
    gd, gi = ix.batchSearch(q, 10)
    ix.close()
    rd, ri = cpu_oracle.sq8_search(oracle.DOT, q, rcodes, rs, ro, 10)
    assert_topk_parity(gd, gi, rd, ri)
    k = 31
    km = vsk.KMeansClustering(dev, maxIterations=3, tolerance=-1.0)
    cent, asg, it, inertia = km.cluster(x, k, x[:k].copy())
    rc, ra, rin, rit = cpu_oracle.kmeans(x, x[:k].copy(), 3)
    assert np.array_equal(np.asarray(asg), ra)
    assert np.max(np.abs(cent - rc)) < 1e-4
