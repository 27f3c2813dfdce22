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
