"""The few-query fp32 scan (``csrc/stream_scan.cu``: a batch of at most eight queries streams every row from
HBM once) against the CPU oracle, through the C ABI: ``VectorStore.search`` is the one-query case of it."""
import numpy as np
import pytest

import oracle
from parity import assert_topk_parity

pytestmark = pytest.mark.gpu
NAMES = ["euclidean", "cosine", "dotProduct", "manhattan"]


@pytest.fixture(scope="module")
def vsk():
    import vectorstorekit_b200 as v
    return v


@pytest.fixture(scope="module")
def dev(vsk):
    return vsk.CUDAAcceleratorStrategy(0).initialize()


def _search(vsk, dev, metric, x, q, k, rm=None, qm=None, path=1):
    dev.set_search_path(path)
    ix = vsk.FlatIndex(dev, x.shape[1], metric)
    ix.add(x, rm)
    try:
        return ix.batchSearch(q, k, qm) if qm is not None else ix.batchSearch(q, k)
    finally:
        ix.close()
        dev.set_search_path(0)


# odd row counts leave the two-row step a ragged end; 130 and 7 are not multiples of 4 (scalar loads);
# 30 001 rows make the schedule run a dense chunk and several thresholded ones
@pytest.mark.parametrize("mid", range(4))
@pytest.mark.parametrize("nq", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("n,d,k", [(30_001, 256, 50), (9_999, 130, 10), (1_500, 7, 3), (20_000, 768, 100)])
def test_few_queries_fp32_path_vs_oracle(vsk, dev, cpu_oracle, mid, nq, n, d, k):
    rng = np.random.default_rng(100 * mid + nq + n + d)
    x = rng.standard_normal((n, d)).astype(np.float32)
    q = rng.standard_normal((nq, d)).astype(np.float32)
    gd, gi = _search(vsk, dev, NAMES[mid], x, q, k, path=1)
    rd, ri = cpu_oracle.flat_search(mid, q, x, k)
    assert_topk_parity(gd, gi, rd, ri)


@pytest.mark.parametrize("nq", [1, 4, 7])
def test_single_query_manhattan_on_the_default_path(vsk, dev, cpu_oracle, nq):
    """Manhattan has no tensor-core form: the default search path sends it to the fp32 scan as well."""
    rng = np.random.default_rng(5 + nq)
    x = rng.uniform(-1, 1, (50_000, 256)).astype(np.float32)
    q = rng.uniform(-1, 1, (nq, 256)).astype(np.float32)
    gd, gi = _search(vsk, dev, "manhattan", x, q, 50, path=0)
    rd, ri = cpu_oracle.flat_search(oracle.MANHATTAN, q, x, 50)
    assert_topk_parity(gd, gi, rd, ri)


@pytest.mark.parametrize("metric", ["manhattan", "cosine", "euclidean"])
@pytest.mark.parametrize("same_mask", [True, False])
def test_few_filtered_queries(vsk, dev, cpu_oracle, metric, same_mask):
    """Row masks with Bernoulli(0.5) bits.  One shared one-hot mask: the batch scans the list of eligible rows
    (row numbers through an index list).  Different masks: one pass over all rows, rows that no query of the
    batch may see are skipped, the others are filtered per query."""
    rng = np.random.default_rng(77)
    n, d = 40_003, 64
    x = rng.uniform(-1, 1, (n, d)).astype(np.float32)
    rm = rng.integers(0, 2 ** 64, n, dtype=np.uint64)
    rm[rng.integers(0, n, n // 4)] = 0                         # rows no query may see
    nq = 6
    bits = np.full(nq, 17) if same_mask else rng.integers(0, 64, nq)
    qm = np.uint64(1) << bits.astype(np.uint64)
    q = rng.uniform(-1, 1, (nq, d)).astype(np.float32)
    gd, gi = _search(vsk, dev, metric, x, q, 20, rm, qm)
    rd, ri = cpu_oracle.flat_search(oracle.METRIC_IDS[metric], q, x, 20, rm, qm)
    assert_topk_parity(gd, gi, rd, ri)
    assert np.all((rm[gi] & qm[:, None]) != 0)


def test_filter_that_matches_almost_nothing(vsk, dev, cpu_oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5_000, 32)).astype(np.float32)
    rm = np.zeros(5_000, np.uint64)
    rm[[11, 4_999]] = 4
    q = rng.standard_normal((2, 32)).astype(np.float32)
    qm = np.array([4, 8], np.uint64)                           # second query: nothing passes
    gd, gi = _search(vsk, dev, "euclidean", x, q, 5, rm, qm)
    rd, ri = cpu_oracle.flat_search(oracle.EUCLIDEAN, q, x, 5, rm, qm)
    assert_topk_parity(gd, gi, rd, ri)
    assert sorted(gi[0][gi[0] >= 0].tolist()) == [11, 4_999] and np.all(gi[1] == -1)


def _mixture(rng, n, d, centres, sigma=0.1):
    c = rng.integers(0, centres.shape[0], n)
    return (centres[c] + sigma * rng.standard_normal((n, d))).astype(np.float32)


@pytest.mark.parametrize("cfg", [(60_000, 128, 256, 16, 10), (20_000, 32, 64, 8, 10), (3_000, 17, 10, 10, 25),
                                 (40_000, 130, 40, 3, 100)])
@pytest.mark.parametrize("nq", [1, 2, 7, 16, 17])
def test_ivf_search_of_a_few_queries(vsk, dev, cpu_oracle, cfg, nq):
    """``IVFIndex.search`` is a one-query call: a handful of queries stream the rows of their own probed lists
    (per-query slices of one row list) instead of going through the list-major tiles.  Parity on shared state,
    as for the batch search: the GPU's centroids and list membership are handed to the oracle."""
    n, d, nlist, nprobe, k = cfg
    rng = np.random.default_rng(n + nlist)
    centres = rng.standard_normal((max(nlist, 4), d)).astype(np.float32)
    x = _mixture(rng, n, d, centres)
    q = _mixture(rng, nq, d, centres)
    ix = vsk.IVFIndex(dev, d, numberOfCentroids=nlist, numberOfProbes=nprobe, maxIterations=4, tolerance=-1.0)
    try:
        ix.train(x)
        ix.insert(x)
        asg = ix.assignments()
        gd, gi = ix.batchSearch(q, k)
        rd, ri = cpu_oracle.ivf_search(q, x, ix.centroids, asg, nprobe, k)
        assert_topk_parity(gd, gi, rd, ri)
        if nq <= 7:
            # `.exact` probes every list and equals the flat search (IVFIndexTests.swift:203-260)
            ed, ei = ix.batchSearch(q, k, vsk.SearchStrategy.exact)
            fd, fi = cpu_oracle.flat_search(oracle.EUCLIDEAN, q, x, k)
            assert_topk_parity(ed, ei, fd, fi)
    finally:
        ix.close()


def test_ivf_few_queries_with_id_base_and_short_lists(vsk, dev, cpu_oracle):
    """Fewer rows in the probed lists than k: the tail of a result row is (+inf, -1); ids carry the index's
    id base (a shard's first global row)."""
    rng = np.random.default_rng(8)
    centres = (10.0 * rng.standard_normal((50, 8))).astype(np.float32)
    x = _mixture(rng, 400, 8, centres)
    q = _mixture(rng, 3, 8, centres)
    ix = vsk.IVFIndex(dev, 8, numberOfCentroids=50, numberOfProbes=2, maxIterations=3, tolerance=-1.0)
    try:
        ix.train(x)
        ix.insert(x)
        ix.set_id_base(1_000_000)
        asg = ix.assignments()
        gd, gi = ix.batchSearch(q, 40)
        rd, ri = cpu_oracle.ivf_search(q, x, ix.centroids, asg, 2, 40)
        ri = np.where(ri >= 0, ri + 1_000_000, ri)
        assert_topk_parity(gd, gi, rd, ri)
        assert np.any(gi < 0)
    finally:
        ix.close()


def test_ivf_few_queries_adversarial_row_order(vsk, dev, cpu_oracle):
    """Rows stored so that, inside a list, every next row is nearer to queries 0 and 2 than all rows before it: the
    threshold never filters, their candidate lists overflow and the two are re-run with smaller chunks (a subset
    of the batch whose list positions differ from its query numbers), while query 1 finishes at the first try."""
    n, d = 60_000, 8
    rng = np.random.default_rng(12)
    x = (1e-3 * rng.standard_normal((n, d))).astype(np.float32)
    x[:, 0] += (2.0 - np.arange(n) / n).astype(np.float32)
    q = np.zeros((3, d), np.float32)
    q[1] = x[n // 3] + 0.01
    q[2, 1] = 1e-3
    ix = vsk.IVFIndex(dev, d, numberOfCentroids=4, numberOfProbes=4, maxIterations=5, tolerance=-1.0)
    try:
        ix.train(x)
        ix.insert(x)
        asg = ix.assignments()
        before = dev.stats()["fallback_queries"]
        gd, gi = ix.batchSearch(q, 10)
        assert dev.stats()["fallback_queries"] - before >= 2
        rd, ri = cpu_oracle.ivf_search(q, x, ix.centroids, asg, 4, 10)
        assert_topk_parity(gd, gi, rd, ri)
    finally:
        ix.close()


@pytest.mark.parametrize("nq,d", [(1, 1536), (4, 1536), (8, 1536), (8, 1500), (3, 3000)])
def test_few_queries_at_the_shared_memory_limit(vsk, dev, cpu_oracle, nq, d):
    """The staged queries must fit 48 KB of shared memory next to the kernel's static words: eight queries of
    1 536 dimensions are exactly 48 KB and go to the tile instead; four of them, or eight of 1 500, stream."""
    rng = np.random.default_rng(nq + d)
    x = rng.standard_normal((3_000, d)).astype(np.float32)
    q = rng.standard_normal((nq, d)).astype(np.float32)
    gd, gi = _search(vsk, dev, "cosine", x, q, 10, path=1)
    rd, ri = cpu_oracle.flat_search(oracle.COSINE, q, x, 10)
    assert_topk_parity(gd, gi, rd, ri)
