"""GPU parity of distances and flat exact k-NN against the CPU oracle, through the C ABI."""
import math
import os

import numpy as np
import pytest

import oracle
from parity import assert_topk_parity

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "metal_shader_vectors.npz"))
NAMES = ["euclidean", "cosine", "dotProduct", "manhattan"]


@pytest.fixture(scope="module")
def vsk():
    import vectorstorekit_b200 as v
    return v


@pytest.fixture(scope="module")
def dev(vsk):
    return vsk.CUDAAcceleratorStrategy(0).initialize()


@pytest.fixture(scope="module")
def engine(vsk, dev):
    return vsk.CUDAAccelerationEngine(dev)


def test_device_is_b200(dev):
    info = dev.info()
    assert info["compute_capability"][0] == 10 and info["sm_count"] > 0


# known answers of the reference's tests, through the library
def test_kat(engine):
    e = engine
    f = lambda *a: np.array(a, np.float32)
    assert abs(e.computeDistances(f(1, 0, 0, 0), f(0, 1, 0, 0)[None], "euclidean")[0] - math.sqrt(2)) < 1e-4
    assert abs(e.computeDistances(f(1, 0, 0, 0), f(0, 1, 0, 0)[None], "cosine")[0] - 1.0) < 1e-4
    assert abs(e.computeDistances(f(1, 0, 0, 0), f(1, 1, 1, 1)[None], "manhattan")[0] - 3.0) < 1e-4
    z = np.zeros(512, np.float32)
    assert abs(e.computeDistances(z, np.ones((1, 512), np.float32), "euclidean")[0] - math.sqrt(512)) < 1e-3
    q = np.stack([np.full(512, float(i), np.float32) for i in range(10)])
    c = np.stack([np.full(512, float(j), np.float32) for j in range(100)])
    dm = e.batchComputeDistances(q, c, "euclidean")
    exp = np.sqrt(512.0 * (np.arange(10)[:, None] - np.arange(100)[None, :]) ** 2)
    assert np.max(np.abs(dm - exp)) < 1e-2
    one, two = np.ones((1, 512), np.float32), 2 * np.ones((1, 512), np.float32)
    assert abs(e.batchComputeDistances(one, two, "manhattan")[0, 0] - 512.0) < 1e-2
    assert abs(e.batchComputeDistances(one, two, "cosine")[0, 0]) < 1e-2
    # Phase1ValidationTests.swift:117-140: 100 queries x 1000 candidates, d = 256, k = 10 -> 100 rows of 10
    rng = np.random.default_rng(0)
    r = e.batchComputeDistances(rng.standard_normal((100, 256)).astype(np.float32),
                                rng.standard_normal((1000, 256)).astype(np.float32), "cosine", topK=10)
    assert r.shape == (100, 10) and np.all(np.diff(r, axis=1) >= 0)


@pytest.mark.parametrize("mid", range(4))
def test_golden_shader_vectors(engine, mid):
    got = engine.batchComputeDistances(GOLD["dist_q"], GOLD["dist_x"], NAMES[mid])
    ref = GOLD[f"dist_{NAMES[mid]}"]
    assert np.allclose(got, ref, rtol=1e-4, atol=1e-5)
    got1 = engine.computeDistances(GOLD["single_q"], GOLD["single_x"], NAMES[mid])
    assert np.allclose(got1, GOLD[f"single_{NAMES[mid]}"], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("mid", range(4))
@pytest.mark.parametrize("shape", [(1, 1, 1), (3, 31, 3), (33, 257, 127), (130, 129, 128), (5, 300, 129), (64, 1000, 768)])
def test_batch_distances_vs_oracle(engine, cpu_oracle, mid, shape):
    nq, nx, d = shape
    rng = np.random.default_rng(1000 * mid + nq + nx + d)
    q = rng.standard_normal((nq, d)).astype(np.float32)
    x = rng.standard_normal((nx, d)).astype(np.float32)
    got = engine.batchComputeDistances(q, x, NAMES[mid])
    ref = cpu_oracle.batch_distances(mid, q, x)
    assert np.allclose(got, ref, rtol=1e-4, atol=1e-4)


def _flat(vsk, dev, metric, x, masks=None):
    ix = vsk.FlatIndex(dev, x.shape[1], metric)
    ix.add(x, masks)
    return ix


@pytest.mark.parametrize("path", [1, 0])
@pytest.mark.parametrize("mid", range(4))
@pytest.mark.parametrize("shape", [(1, 1, 1, 1), (7, 31, 3, 5), (33, 255, 127, 10), (130, 5000, 128, 10),
                                   (257, 20000, 64, 100), (16, 9000, 129, 33)])
def test_flat_search_vs_oracle(vsk, dev, cpu_oracle, path, mid, shape):
    nq, nx, d, k = shape
    dev.set_search_path(path)
    rng = np.random.default_rng(77 * mid + nx + d)
    q = rng.standard_normal((nq, d)).astype(np.float32)
    x = rng.standard_normal((nx, d)).astype(np.float32)
    ix = _flat(vsk, dev, NAMES[mid], x)
    try:
        gd, gi = ix.batchSearch(q, min(k, nx))
    finally:
        ix.close()
        dev.set_search_path(0)
    rd, ri = cpu_oracle.flat_search(mid, q, x, min(k, nx))
    assert_topk_parity(gd, gi, rd, ri)


@pytest.mark.parametrize("path", [1, 0])
def test_config1_flat_euclidean_100k(vsk, dev, cpu_oracle, path):
    """Flat exact k-NN, Euclidean: N = 100 000 x d = 128, 1 000 queries, k = 10, i.i.d. N(0,1)."""
    rng = np.random.default_rng(202611251)
    x = rng.standard_normal((100_000, 128)).astype(np.float32)
    q = rng.standard_normal((1000, 128)).astype(np.float32)
    dev.set_search_path(path)
    ix = _flat(vsk, dev, "euclidean", x)
    try:
        gd, gi = ix.batchSearch(q, 10)
    finally:
        ix.close()
        dev.set_search_path(0)
    rd, ri = cpu_oracle.flat_search(oracle.EUCLIDEAN, q, x, 10, nthreads=0)
    assert_topk_parity(gd, gi, rd, ri)


@pytest.mark.parametrize("path", [1, 0])
def test_config2_shape_cosine_reduced(vsk, dev, cpu_oracle, path):
    """Cosine, d = 768, k = 100, rows and queries L2-normalised (the headline configuration at
    reduced N so that the CPU oracle finishes in seconds)."""
    rng = np.random.default_rng(202611252)
    x = cpu_oracle.normalize_rows(rng.standard_normal((30_000, 768)).astype(np.float32))
    q = cpu_oracle.normalize_rows(rng.standard_normal((256, 768)).astype(np.float32))
    dev.set_search_path(path)
    ix = _flat(vsk, dev, "cosine", x)
    try:
        gd, gi = ix.batchSearch(q, 100)
    finally:
        ix.close()
        dev.set_search_path(0)
    rd, ri = cpu_oracle.flat_search(oracle.COSINE, q, x, 100)
    assert_topk_parity(gd, gi, rd, ri)


@pytest.mark.parametrize("path", [1, 0])
@pytest.mark.parametrize("k", [1000, 2048])
def test_large_k(vsk, dev, cpu_oracle, path, k):
    """k near the limits of the candidate lists (k = 2048 is the largest accepted)."""
    rng = np.random.default_rng(31)
    x = rng.standard_normal((30_000, 40)).astype(np.float32)
    q = rng.standard_normal((20, 40)).astype(np.float32)
    dev.set_search_path(path)
    ix = _flat(vsk, dev, "euclidean", x)
    try:
        gd, gi = ix.batchSearch(q, k)
        with pytest.raises(vsk.InvalidInput):
            ix.batchSearch(q, 2049)
    finally:
        ix.close()
        dev.set_search_path(0)
    rd, ri = cpu_oracle.flat_search(oracle.EUCLIDEAN, q, x, k)
    assert_topk_parity(gd, gi, rd, ri)


def test_filtered_manhattan(vsk, dev, cpu_oracle):
    """Filtered flat search, Manhattan, uniform [-1,1], uint64 row masks with Bernoulli(0.5) bits,
    one-hot query masks (about half the rows pass), k = 50."""
    rng = np.random.default_rng(202611255)
    x = rng.uniform(-1, 1, (30_000, 256)).astype(np.float32)
    q = rng.uniform(-1, 1, (200, 256)).astype(np.float32)
    rm = rng.integers(0, 2 ** 64, 30_000, dtype=np.uint64)
    qm = (np.uint64(1) << rng.integers(0, 64, 200).astype(np.uint64))
    ix = _flat(vsk, dev, "manhattan", x, rm)
    try:
        gd, gi = ix.batchSearch(q, 50, qm)
        ud, ui = ix.batchSearch(q, 50)          # same index, unfiltered
    finally:
        ix.close()
    rd, ri = cpu_oracle.flat_search(oracle.MANHATTAN, q, x, 50, rm, qm)
    assert_topk_parity(gd, gi, rd, ri)
    assert np.all((rm[gi] & qm[:, None]) != 0)
    rd2, ri2 = cpu_oracle.flat_search(oracle.MANHATTAN, q, x, 50)
    assert_topk_parity(ud, ui, rd2, ri2)


@pytest.mark.parametrize("metric", ["manhattan", "euclidean", "cosine"])
def test_filtered_search_grouped_by_mask(vsk, dev, cpu_oracle, metric):
    """Few distinct query masks: each group of queries is scanned only against its eligible rows (row lists,
    narrow query tiles for small groups).  Group sizes 130 / 70 / 40 / 33 / 9, one mask that matches nothing,
    one that combines two bits."""
    rng = np.random.default_rng(21)
    n, d = 40_000, 48
    x = rng.uniform(-1, 1, (n, d)).astype(np.float32)
    rm = rng.integers(0, 2 ** 16, n, dtype=np.uint64)          # bits 0..15 set at random, higher bits clear
    masks = [1 << 2, 1 << 9, (1 << 3) | (1 << 4), 1 << 40, 1 << 15]
    sizes = [130, 70, 40, 33, 9]
    qm = np.concatenate([np.full(s, m, np.uint64) for m, s in zip(masks, sizes)])
    perm = rng.permutation(qm.size)
    qm = qm[perm]                                               # groups interleaved in the batch
    q = rng.uniform(-1, 1, (qm.size, d)).astype(np.float32)
    ix = _flat(vsk, dev, metric, x, rm)
    try:
        gd, gi = ix.batchSearch(q, 20, qm)
    finally:
        ix.close()
    rd, ri = cpu_oracle.flat_search(oracle.METRIC_IDS[metric], q, x, 20, rm, qm)
    assert_topk_parity(gd, gi, rd, ri)
    none = qm == np.uint64(1 << 40)
    assert none.sum() == 33 and np.all(gi[none] == -1) and np.all(np.isinf(gd[none]))
    ok = ~none
    assert np.all((rm[gi[ok]] & qm[ok][:, None]) != 0)


def test_selective_filter_and_short_results(vsk, dev, cpu_oracle):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((6000, 16)).astype(np.float32)
    q = rng.standard_normal((5, 16)).astype(np.float32)
    rm = np.zeros(6000, np.uint64)
    rm[::500] = 1          # 12 rows pass bit 0
    rm[7] |= 2             # one row passes bit 1
    qm = np.array([1, 2, 4, 3, 1], np.uint64)   # bit 2: nothing passes
    ix = _flat(vsk, dev, "euclidean", x, rm)
    try:
        gd, gi = ix.batchSearch(q, 20, qm)
    finally:
        ix.close()
    rd, ri = cpu_oracle.flat_search(oracle.EUCLIDEAN, q, x, 20, rm, qm)
    assert_topk_parity(gd, gi, rd, ri)
    assert np.all(gi[2] == -1) and np.all(np.isinf(gd[2]))
    assert (gi[1] >= 0).sum() == 1 and gi[1, 0] == 7


@pytest.mark.parametrize("path", [1, 0])
def test_adversarial_order_overflows_lists_and_is_still_exact(vsk, dev, cpu_oracle, path):
    """Rows sorted farthest-first make every later row beat the running threshold, so the candidate
    lists overflow and the flagged queries take the non-overflowing re-run."""
    rng = np.random.default_rng(11)
    x = rng.standard_normal((40_000, 32)).astype(np.float32)
    q = np.zeros((3, 32), np.float32)
    q[1] += 0.01
    q[2] -= 0.01
    order = np.argsort(-np.linalg.norm(x, axis=1))
    x = np.ascontiguousarray(x[order])
    dev.set_search_path(path)
    before = dev.stats()["fallback_queries"]
    ix = _flat(vsk, dev, "euclidean", x)
    try:
        gd, gi = ix.batchSearch(q, 10)
    finally:
        ix.close()
        dev.set_search_path(0)
    rd, ri = cpu_oracle.flat_search(oracle.EUCLIDEAN, q, x, 10)
    assert_topk_parity(gd, gi, rd, ri)
    assert dev.stats()["fallback_queries"] > before


def test_incremental_add_and_id_base(vsk, dev, cpu_oracle):
    rng = np.random.default_rng(12)
    x = rng.standard_normal((3000, 24)).astype(np.float32)
    q = rng.standard_normal((9, 24)).astype(np.float32)
    ix = vsk.FlatIndex(dev, 24, "dotProduct")
    try:
        ix.add(x[:1000]); ix.add(x[1000:1001]); ix.add(x[1001:])
        assert ix.count == 3000
        ix.set_id_base(5_000_000_000)
        gd, gi = ix.batchSearch(q, 7)
    finally:
        ix.close()
    rd, ri = cpu_oracle.flat_search(oracle.DOT, q, x, 7)
    assert_topk_parity(gd, gi - 5_000_000_000, rd, ri)


def test_device_pointers_and_merge(vsk, dev, engine, cpu_oracle):
    import torch
    rng = np.random.default_rng(13)
    x = rng.standard_normal((8000, 48)).astype(np.float32)
    q = rng.standard_normal((70, 48)).astype(np.float32)
    xd, qd = torch.from_numpy(x).cuda(), torch.from_numpy(q).cuda()
    parts_d, parts_i = [], []
    for s in range(4):
        ix = vsk.FlatIndex(dev, 48, "euclidean")
        ix.add(xd[s * 2000:(s + 1) * 2000])
        ix.set_id_base(s * 2000)
        d, i = ix.batchSearch(qd, 10)
        assert d.is_cuda and i.dtype == torch.int64
        parts_d.append(d); parts_i.append(i)
        ix.close()
    md, mi = engine.mergeTopK(torch.stack(parts_d), torch.stack(parts_i))
    rd, ri = cpu_oracle.flat_search(oracle.EUCLIDEAN, q, x, 10)
    assert_topk_parity(md.cpu().numpy(), mi.cpu().numpy(), rd, ri)
    od, oi = cpu_oracle.merge_topk(torch.stack(parts_d).cpu().numpy(), torch.stack(parts_i).cpu().numpy())
    assert np.array_equal(mi.cpu().numpy(), oi) and np.array_equal(md.cpu().numpy(), od)


@pytest.mark.parametrize("metric,shards,k", [("euclidean", 3, 20), ("cosine", 4, 100), ("dotProduct", 2, 1),
                                             ("euclidean", 8, 5)])
def test_two_half_shard_search(vsk, engine, cpu_oracle, metric, shards, k):
    """The search of a row shard in two halves (bound out, reduced bound in): shards emulated one after another on
    one GPU, each on its own context; their merged result equals the unsharded search, and the reduced bound drops
    most of each shard's rows before the exact re-scoring."""
    import torch
    rng = np.random.default_rng(29)
    n, d, nq = 36_000, 64, 300
    x = rng.standard_normal((n, d)).astype(np.float32)
    q = rng.standard_normal((nq, d)).astype(np.float32)
    x[20_000] = x[5]                       # an exact tie across two shards
    xd, qd = torch.from_numpy(x).cuda(), torch.from_numpy(q).cuda()
    devs, idx, bounds = [], [], []
    try:
        for s in range(shards):
            dv = vsk.CUDAAcceleratorStrategy(0).initialize()
            lo, hi = s * n // shards, (s + 1) * n // shards
            ix = vsk.FlatIndex(dv, d, metric)
            ix.add(xd[lo:hi])
            ix.set_id_base(lo)
            devs.append(dv); idx.append(ix)
            bounds.append(ix.shardSearchBegin(qd, k, shards))
        torch.cuda.synchronize()           # `begin` returns with its kernels still running on the library's stream
        g = torch.stack(bounds).max(dim=0).values
        assert bool(torch.isfinite(g).all())
        parts = [ix.shardSearchFinish(g) for ix in idx]
        reranked = sum(dv.stats()["reranked_rows"] for dv in devs)
        fallbacks = sum(dv.stats()["fallback_queries"] for dv in devs)
    finally:
        for ix in idx:
            ix.close()
    pd, pi = torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts])
    md, mi = engine.mergeTopK(pd, pi)
    rd, ri = cpu_oracle.flat_search(oracle.METRIC_IDS[metric], q, x, k)
    assert_topk_parity(md.cpu().numpy(), mi.cpu().numpy(), rd, ri)
    assert fallbacks <= nq // 20
    if shards * 4 <= k:
        # every shard alone would re-score more than k rows per query; with the bound, well under half of that
        assert reranked < 0.5 * shards * nq * k


def test_two_half_shard_search_without_split_form(vsk, cpu_oracle):
    """fp32 search path and Manhattan have no split form: `begin` reports +inf, `finish` runs the whole search."""
    import torch
    rng = np.random.default_rng(31)
    x = rng.standard_normal((5000, 32)).astype(np.float32)
    q = rng.standard_normal((40, 32)).astype(np.float32)
    dv = vsk.CUDAAcceleratorStrategy(0).initialize()
    ix = vsk.FlatIndex(dv, 32, "manhattan")
    try:
        ix.add(torch.from_numpy(x).cuda())
        with pytest.raises(vsk.InvalidInput):
            ix._pending = (torch.from_numpy(q).cuda(), 6)
            ix.shardSearchFinish(torch.zeros(40, device="cuda"))
        b = ix.shardSearchBegin(torch.from_numpy(q).cuda(), 6, 4)
        torch.cuda.synchronize()
        assert bool(torch.isinf(b).all())
        gd, gi = ix.shardSearchFinish(b)
    finally:
        ix.close()
    rd, ri = cpu_oracle.flat_search(oracle.MANHATTAN, q, x, 6)
    assert_topk_parity(gd.cpu().numpy(), gi.cpu().numpy(), rd, ri)


@pytest.mark.parametrize("d", [96, 128, 200, 320])
@pytest.mark.parametrize("case", ["unit", "tiny", "huge", "offset", "query_scale", "zero_rows"])
def test_euclidean_row_term_inside_contraction(vsk, dev, cpu_oracle, d, case):
    """Euclidean search over operand layouts with and without the |x|^2 term folded into the contraction (d <= 256
    folds, d = 320 does not), on value ranges that stress the folded term: tiny and huge norms, a common offset (|x|^2
    much larger than the differences that rank the rows), queries on another scale than the rows, zero rows."""
    rng = np.random.default_rng(1000 + d)
    n, nq, k = 20_000, 200, 10
    x = rng.standard_normal((n, d)).astype(np.float32)
    q = rng.standard_normal((nq, d)).astype(np.float32)
    if case == "tiny":
        x *= 1e-3; q *= 1e-3
    elif case == "huge":
        x *= 1e3; q *= 1e3
    elif case == "offset":
        x += 5.0; q += 5.0
    elif case == "query_scale":
        q *= 100.0
    elif case == "zero_rows":
        x[::7] = 0.0
        q[0] = 0.0
    ix = vsk.FlatIndex(dev, d, "euclidean")
    try:
        ix.add(x)
        gd, gi = ix.batchSearch(q, k)
    finally:
        ix.close()
    rd, ri = cpu_oracle.flat_search(oracle.EUCLIDEAN, q, x, k)
    assert_topk_parity(gd, gi, rd, ri)


def test_errors(vsk, dev, engine):
    x = np.zeros((4, 8), np.float32)
    with pytest.raises(vsk.EmptyInput):
        engine.batchComputeDistances(x, np.zeros((0, 8), np.float32), "euclidean")
    with pytest.raises(vsk.UnsupportedOperation):
        engine.batchComputeDistances(x, x, "hamming")
    with pytest.raises(vsk.DimensionMismatch):
        engine.batchComputeDistances(x, np.zeros((4, 9), np.float32), "euclidean")
    ix = vsk.FlatIndex(dev, 8, "euclidean")
    try:
        with pytest.raises(vsk.EmptyInput):
            ix.batchSearch(x, 3)               # empty index
        ix.add(x)
        with pytest.raises(vsk.DimensionMismatch):
            ix.batchSearch(np.zeros((1, 7), np.float32), 3)
        with pytest.raises(vsk.InvalidInput):
            ix.batchSearch(x, 0)
        with pytest.raises(vsk.InvalidInput):
            ix.batchSearch(x, 3, np.ones(4, np.uint64))   # no row masks in the index
        d, i = ix.batchSearch(x, 6)            # k > n: padded
        assert np.all(i[:, 4:] == -1) and np.all(np.isinf(d[:, 4:]))
    finally:
        ix.close()


def test_cpp_host_mirror_on_gpu(tmp_path):
    import subprocess
    from test_abi_cpu import _build_host_mirror
    out = subprocess.run([_build_host_mirror(str(tmp_path))], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip() == "ok", out


def test_two_lanes_equal_one_lane(vsk, cpu_oracle):
    """A batch large enough for the two-lane schedule (two halves on two streams) returns what the one-lane schedule
    returns, bit for bit, and both match the oracle; uneven halves and a batch just above the switch included."""
    import torch
    dev = vsk.CUDAComputeDevice(0)
    rng = np.random.default_rng(77)
    try:
        for metric, d, nq in (("cosine", 256, 2048 + 37), ("euclidean", 96, 4096), ("dotProduct", 320, 3000)):
            x = rng.standard_normal((60_000, d)).astype(np.float32)
            q = rng.standard_normal((nq, d)).astype(np.float32)
            ix = vsk.FlatIndex(dev, d, metric)
            ix.add(x)
            qd = torch.as_tensor(q, device="cuda")
            dev.set_tuning(overlap_min_queries=2048)
            d2, i2 = ix.batchSearch(qd, 20)
            dev.set_tuning(overlap_min_queries=0)
            d1, i1 = ix.batchSearch(qd, 20)
            assert torch.equal(i1, i2) and torch.equal(d1, d2)
            sub = np.arange(0, nq, 16)
            rd, ri = cpu_oracle.flat_search(oracle.METRIC_IDS[metric], q[sub], x, 20)
            assert_topk_parity(d2.cpu().numpy()[sub], i2.cpu().numpy()[sub], rd, ri)
            ix.close()
        assert dev.tuning()["overlap_min_queries"] == 0
    finally:
        dev.close()


@pytest.mark.parametrize("metric", ["euclidean", "cosine", "dotProduct"])
def test_filtered_batch_stays_on_the_tensor_path(vsk, cpu_oracle, metric):
    """A filtered batch of a tensor-path metric is filtered in the contraction's epilogue: tensor tiles are computed,
    the result equals the oracle's pre-filter + search.  One-hot masks over Bernoulli(0.5) row masks, a mask that
    matches nothing, one that matches everything, and a rare bit (1 % of the rows) that leaves fewer than k rows in
    the first chunk."""
    dev = vsk.CUDAComputeDevice(0)
    try:
        rng = np.random.default_rng(5150)
        n, d, nq, k = 50_000, 200, 700, 30
        x = rng.standard_normal((n, d)).astype(np.float32)
        q = rng.standard_normal((nq, d)).astype(np.float32)
        rm = rng.integers(0, 2 ** 62, n, dtype=np.uint64)
        rare = rng.random(n) < 0.01
        rm = (rm & ~np.uint64(1 << 62)) | (rare.astype(np.uint64) << np.uint64(62))
        qm = (np.uint64(1) << rng.integers(0, 62, nq).astype(np.uint64))
        qm[0:40] = np.uint64(1 << 63)                     # no row has bit 63
        qm[40:80] = np.uint64(2 ** 64 - 1)                # every row with any bit
        qm[80:140] = np.uint64(1 << 62)                   # the rare bit
        ix = vsk.FlatIndex(dev, d, metric)
        ix.add(x, rm)
        before = dev.stats()
        gd, gi = ix.batchSearch(q, k, qm)
        after = dev.stats()
        ix.close()
        assert after["tensor_tiles"] > before["tensor_tiles"]
        rd, ri = cpu_oracle.flat_search(oracle.METRIC_IDS[metric], q, x, k, rm, qm)
        assert_topk_parity(gd, gi, rd, ri)
        assert np.all(gi[:40] == -1)
        ok = gi >= 0
        assert np.all(((rm[np.clip(gi, 0, None)] & qm[:, None]) != 0) | ~ok)
    finally:
        dev.close()


def test_selective_filters_take_the_row_list_path(vsk, cpu_oracle):
    """When the filters leave only a few percent of the pairs eligible, scanning the eligible rows beats filtering
    the full contraction: the batch goes to the grouped fp32 scan (no tensor tiles) and is exact all the same."""
    dev = vsk.CUDAComputeDevice(0)
    try:
        rng = np.random.default_rng(61)
        n, d, nq, k = 40_000, 64, 300, 10
        x = rng.standard_normal((n, d)).astype(np.float32)
        q = rng.standard_normal((nq, d)).astype(np.float32)
        rm = (rng.random(n) < 0.01).astype(np.uint64) | ((rng.random(n) < 0.02).astype(np.uint64) << np.uint64(1))
        qm = np.where(np.arange(nq) % 2 == 0, np.uint64(1), np.uint64(2)).astype(np.uint64)
        ix = vsk.FlatIndex(dev, d, "euclidean")
        ix.add(x, rm)
        before = dev.stats()
        gd, gi = ix.batchSearch(q, k, qm)
        after = dev.stats()
        ix.close()
        assert after["tensor_tiles"] == before["tensor_tiles"]
        rd, ri = cpu_oracle.flat_search(oracle.EUCLIDEAN, q, x, k, rm, qm)
        assert_topk_parity(gd, gi, rd, ri)
    finally:
        dev.close()


def test_bounded_wait_expiry_returns_timeout_and_the_context_survives(vsk, cpu_oracle):
    """The contraction kernel's pipeline waits are bounded.  The testing switch makes CTA 0 leave one operand stage
    unfilled: the consumer's wait for it runs out (a short limit is set so that this takes milliseconds), every role
    leaves its loop, copies in flight are drained, tensor memory is released and the call returns the counterpart of
    commandBufferTimeout (MetalErrors.swift:30) - no trap, no fault.  The next search on the same context is exact."""
    dev = vsk.CUDAComputeDevice(0)
    try:
        rng = np.random.default_rng(404)
        x = rng.standard_normal((20_000, 128)).astype(np.float32)
        q = rng.standard_normal((300, 128)).astype(np.float32)
        ix = vsk.FlatIndex(dev, 128, "cosine")
        ix.add(x)
        d0, i0 = ix.batchSearch(q, 10)
        dev.set_tuning(wait_limit_log2=16, test_stall_scan=1)
        with pytest.raises(vsk.Timeout):
            ix.batchSearch(q, 10)
        assert dev.tuning()["test_stall_scan"] == 0          # one shot
        dev.set_tuning(wait_limit_log2=0)
        d1, i1 = ix.batchSearch(q, 10)
        assert np.array_equal(i1, i0) and np.array_equal(d1, d0)
        rd, ri = cpu_oracle.flat_search(oracle.COSINE, q, x, 10)
        assert_topk_parity(d1, i1, rd, ri)
        ix.close()
    finally:
        dev.close()


def test_distance_matrix_api(vsk, dev, cpu_oracle):
    """MetalDistanceMatrix.computeDistanceMatrix (MetalDistanceMatrix.swift:49-119): A x B, and A x A with the
    lower triangle mirrored from the upper one."""
    import oracle as orc
    rng = np.random.default_rng(77)
    a = rng.standard_normal((37, 512)).astype(np.float32)       # the reference's type is Vector512
    b = rng.standard_normal((53, 512)).astype(np.float32)
    eng = vsk.CUDAAccelerationEngine(dev)
    for metric in ("euclidean", "cosine", "manhattan", "dotProduct"):
        mid = orc.METRIC_IDS[metric]
        ab = eng.computeDistanceMatrix(a, b, metric)
        ref = cpu_oracle.batch_distances(mid, a, b)
        assert ab.shape == (37, 53) and np.allclose(ab, ref, rtol=1e-4, atol=1e-5)
        aa = eng.computeDistanceMatrix(a, None, metric)
        ref = cpu_oracle.batch_distances(mid, a, a)
        assert np.array_equal(aa, aa.T)
        assert np.allclose(np.triu(aa), np.triu(ref), rtol=1e-4, atol=2e-4)
    import torch
    aa = eng.computeDistanceMatrix(torch.as_tensor(a, device="cuda"), None, "euclidean")
    assert torch.equal(aa, aa.T) and float(aa.diagonal().abs().max()) == 0.0


def test_async_search_is_the_blocking_search(vsk, cpu_oracle):
    """vsk_search_async / vsk_search_dev_async (the completion-handler form, MetalAccelerationEngine.swift:444-449):
    submissions queue on the context's worker and resolve, in order, to what the blocking call returns; a failing
    call fails its future and is reported once more by wait()."""
    import torch
    dev = vsk.CUDAComputeDevice(0)
    try:
        rng = np.random.default_rng(909)
        x = rng.standard_normal((30_000, 96)).astype(np.float32)
        qs = [rng.standard_normal((n, 96)).astype(np.float32) for n in (1, 200, 1500)]
        ix = vsk.FlatIndex(dev, 96, "euclidean")
        ix.add(x)
        want = [ix.batchSearch(q, 10) for q in qs]
        futs = [ix.batchSearchAsync(q, 10) for q in qs]                  # three in the queue at once
        fdev = ix.batchSearchAsync(torch.as_tensor(qs[1], device="cuda"), 10)
        for f, (wd, wi) in zip(futs, want):
            gd, gi = f.result(timeout=120)
            assert np.array_equal(gi, wi) and np.array_equal(gd, wd)
        dd, di = fdev.result(timeout=120)                                # stream drained before the callback
        assert np.array_equal(di.cpu().numpy(), want[1][1])
        dev.wait()
        rd, ri = cpu_oracle.flat_search(oracle.EUCLIDEAN, qs[2], x, 10)
        assert_topk_parity(*futs[2].result(), rd, ri)
        bad = ix.batchSearchAsync(qs[0], 40_000)                         # k > rows of the index
        with pytest.raises(vsk.VSKError):
            bad.result(timeout=120)
        with pytest.raises(vsk.VSKError):
            dev.wait()
        dev.wait()                                                       # reported once
        gd, gi = ix.batchSearchAsync(qs[0], 10).result(timeout=120)      # the context still works
        assert np.array_equal(gi, want[0][1])
        ix.close()
    finally:
        dev.close()


@pytest.mark.parametrize("d", [96, 200, 768])
def test_ring_stage_granularity_does_not_change_results(vsk, cpu_oracle, d):
    """The contraction kernel's operand ring holds one or two K blocks per stage (vsk_tuning.stage_kblocks): the same
    MMAs in the same order either way, so the results are identical bit for bit (odd numbers of K blocks included)."""
    dev = vsk.CUDAComputeDevice(0)
    try:
        rng = np.random.default_rng(1000 + d)
        x = rng.standard_normal((30_000, d)).astype(np.float32)
        q = rng.standard_normal((600, d)).astype(np.float32)
        ix = vsk.FlatIndex(dev, d, "euclidean")
        ix.add(x)
        out = []
        for kblocks in (1, 2):
            dev.set_tuning(stage_kblocks=kblocks)
            out.append(ix.batchSearch(q, 20))
        assert np.array_equal(out[0][1], out[1][1]) and np.array_equal(out[0][0], out[1][0])
        rd, ri = cpu_oracle.flat_search(oracle.EUCLIDEAN, q, x, 20)
        assert_topk_parity(out[1][0], out[1][1], rd, ri)
        ix.close()
    finally:
        dev.close()
