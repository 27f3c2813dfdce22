"""GPU parity of k-means, IVF build/search and the int8 quantiser/scan against the CPU oracle."""
import os

import numpy as np
import pytest

import oracle
from parity import assert_topk_parity

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "metal_shader_vectors.npz"))


@pytest.fixture(scope="module")
def vsk():
    import vectorstorekit_b200 as v
    return v


@pytest.fixture(scope="module")
def dev(vsk):
    return vsk.CUDAAcceleratorStrategy(0).initialize()


def _mixture(rng, n, d, centres, sigma=0.1):
    c = rng.integers(0, centres.shape[0], n)
    return (centres[c] + sigma * rng.standard_normal((n, d))).astype(np.float32)


def test_kmeans_golden_shader_steps(vsk, dev):
    """Three Lloyd steps of the reference's shader kernels; centroid 5 starts far away, receives no
    row and keeps its value."""
    x, c0 = GOLD["km_x"], GOLD["km_c0"]
    for it in (1, 2, 3):
        km = vsk.KMeansClustering(dev, maxIterations=it, tolerance=-1.0)
        cent, asg, iters, inertia = km.cluster(x, 6, c0)
        assert iters == it
        assert np.allclose(cent, GOLD[f"km_c{it}"], rtol=1e-5, atol=1e-6)
        assert np.array_equal(cent[5], c0[5])
    assert np.array_equal(asg, GOLD["km_assign3"])


@pytest.mark.parametrize("shape", [(500, 12, 9, 4), (20_000, 128, 64, 5), (5000, 33, 300, 3), (100_000, 128, 256, 3),
                                   (60_000, 40, 100, 2)])
def test_kmeans_vs_oracle(vsk, dev, cpu_oracle, shape):
    n, d, k, iters = shape
    rng = np.random.default_rng(n + d)
    centres = rng.standard_normal((k, d)).astype(np.float32)
    x = _mixture(rng, n, d, centres, 0.3)
    km = vsk.KMeansClustering(dev, maxIterations=iters, tolerance=-1.0)
    cent, asg, it, inertia = km.cluster(x, k, x[:k])
    rc, ra, rin, rit = cpu_oracle.kmeans(x, x[:k], iters)
    assert it == rit == iters
    agree = np.mean(asg == ra)
    assert agree > 0.999, agree
    assert np.max(np.abs(cent - rc)) < 1e-3
    assert abs(inertia - rin) <= 1e-3 * abs(rin)


def test_tensor_assign_equals_fp32_assign(vsk, dev):
    """The tensor-core assignment (coarse arg-min, near-tie lists, exact decision) against the fp32 tile on the
    same inputs, including exact duplicates of centroids among the rows and duplicate centroids."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((200_000, 96), generator=g, device="cuda")
    c = torch.randn((500, 96), generator=g, device="cuda")
    c[7] = c[3]                      # duplicate centroid: the lower index must win
    x[:500] = c                      # rows that coincide with centroids
    km = vsk.KMeansClustering(dev)
    dev.set_search_path(vsk.PATH_FP32_SCAN)
    a0, d0 = km.assign(x, c)
    dev.set_search_path(vsk.PATH_TENSOR_RERANK)
    a1, d1 = km.assign(x, c)
    a0, a1, d0, d1 = (t.cpu().numpy() for t in (a0, a1, d0, d1))
    assert np.mean(a0 == a1) > 0.9999
    assert np.allclose(d0, d1, rtol=1e-4, atol=1e-4)
    assert a1[7] == 3 and a1[3] == 3 and np.array_equal(a1[:500][np.arange(500) != 7], np.arange(500)[np.arange(500) != 7])


def test_lloyd_iterations_on_the_tensor_path_equal_the_fp32_path(vsk, dev):
    """Several Lloyd iterations on clustered data, where the thresholds of the next scan come from the previous
    assignment (per row the exact value of its centroid at the new position or, where the centroid has hardly moved,
    the triangle inequality): the run ends where the fp32 tile's run ends."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(17)
    n, d, k, iters = 300_000, 64, 1024, 8
    centres = torch.randn((k, d), generator=g, device="cuda")
    x = centres[torch.randint(0, k, (n,), generator=g, device="cuda")] + 0.05 * torch.randn((n, d), generator=g, device="cuda")
    init = x[:k].contiguous()
    out = []
    for path in (vsk.PATH_FP32_SCAN, vsk.PATH_TENSOR_RERANK):
        dev.set_search_path(path)
        km = vsk.KMeansClustering(dev, maxIterations=iters, tolerance=-1.0)
        before = dev.stats()
        cent, asg, it, inertia = km.cluster(x, k, init)
        after = dev.stats()
        out.append((cent.cpu().numpy(), asg.cpu().numpy(), float(inertia), after["fallback_queries"] - before["fallback_queries"]))
    dev.set_search_path(vsk.PATH_TENSOR_RERANK)
    (c0, a0, i0, _), (c1, a1, i1, fb) = out
    assert fb < n                                        # never the whole-batch fp32 fallback
    assert np.mean(a0 == a1) > 0.999, np.mean(a0 == a1)
    assert abs(i0 - i1) <= 1e-3 * abs(i0)
    assert np.max(np.abs(c0 - c1)) < 5e-2


@pytest.mark.parametrize("d", [64, 192, 240])
@pytest.mark.parametrize("data", ["unstructured", "clustered"])
def test_every_lloyd_step_assigns_each_row_to_a_nearest_centroid(vsk, dev, data, d):
    """Step by step through the trainer (the caller hands in the centroids of each step): after every step each row's
    centroid must be a nearest one under the direct formula - checked in fp64 - whichever way the step's thresholds
    were formed.  On unstructured data (no gaps between clusters) many centroids sit inside the looser triangle
    bound; the hit log may fill, in which case the step repeats itself with exact thresholds."""
    import torch
    # d = 64 and 192: the fold columns start a K block of their own and travel as a 16-column tile (one and three
    # 64-column blocks before it); d = 240: they fill the last block's fourth K16 step, and a ring stage is one K block
    g = torch.Generator(device="cuda").manual_seed(23)
    n, k = 200_000, 1024
    if data == "unstructured":
        x = torch.randn((n, d), generator=g, device="cuda")
    else:
        centres = torch.randn((k, d), generator=g, device="cuda")
        x = centres[torch.randint(0, k, (n,), generator=g, device="cuda")] + 0.05 * torch.randn((n, d), generator=g, device="cuda")
    c = x[:k].clone()
    tr = vsk.KMeansTrainer(dev, x, k)
    sample = torch.randperm(n, generator=g, device="cuda")[:20_000]
    xs = x[sample].double()
    try:
        for step in range(7):
            sums, counts, inertia = tr.step(c)
            a = tr.assignments()[sample].long()
            dd = torch.cdist(xs, c.double())                       # [sample][k], fp64
            best = dd.min(dim=1).values
            got = dd.gather(1, a[:, None])[:, 0]
            assert bool((got <= best * (1 + 1e-5) + 1e-6).all()), (step, float((got - best).max()))
            c = tr.finish(sums, counts, c)
    finally:
        tr.close()


def test_kmeans_convergence_and_errors(vsk, dev, cpu_oracle):
    rng = np.random.default_rng(4)
    x = np.concatenate([rng.standard_normal((200, 4)) * 0.01 + 5, rng.standard_normal((200, 4)) * 0.01 - 5]).astype(np.float32)
    km = vsk.KMeansClustering(dev, maxIterations=50, tolerance=1e-4)
    cent, asg, it, inertia = km.cluster(x, 2, x[[0, 399]])
    rc, ra, rin, rit = cpu_oracle.kmeans(x, x[[0, 399]], 50, 1e-4)
    assert it == rit and it < 50 and np.array_equal(asg, ra)
    with pytest.raises(vsk.InsufficientTrainingData):
        km.cluster(x[:3], 5, x[:5])


@pytest.mark.parametrize("shape", [(30_000, 32, 64, 4), (200_000, 128, 256, 3)])
def test_kmeans_trainer_shards_equal_single_run(vsk, dev, cpu_oracle, shape):
    """The step-wise trainer that multi-GPU training uses: two shards of the rows (here on one GPU), their sums,
    counts and inertia added up by hand, give the centroids of vsk_kmeans on all rows."""
    import torch
    from vectorstorekit_b200.sharded import ShardedKMeans
    n, d, k, iters = shape
    rng = np.random.default_rng(n)
    centres = rng.standard_normal((k, d)).astype(np.float32)
    x = _mixture(rng, n, d, centres, 0.3)
    init = x[:k].copy()
    init[k - 1] = 1e3                                                     # attracts nothing: stays put
    whole = vsk.KMeansClustering(dev, maxIterations=iters, tolerance=-1.0)
    rc, ra, rit, rin = whole.cluster(x, k, init)
    xt = torch.as_tensor(x, device="cuda")
    cut = n // 3
    shards = [vsk.KMeansTrainer(dev, xt[:cut], k), vsk.KMeansTrainer(dev, xt[cut:], k)]

    def step(cent):
        parts = [t.step(cent) for t in shards]
        return tuple(sum(p[i] for p in parts) for i in range(3))           # what the all-reduce does across ranks

    cent, it, inertia = ShardedKMeans(step, shards[0].finish).cluster(torch.as_tensor(init, device="cuda"), iters, -1.0)
    assert it == rit == iters
    assert np.max(np.abs(cent.cpu().numpy() - rc)) < 1e-3
    assert abs(inertia - rin) <= 1e-3 * abs(rin)
    assert np.array_equal(cent.cpu().numpy()[k - 1], init[k - 1])
    asg = torch.cat([t.assignments() for t in shards]).cpu().numpy()
    # the trainers hold the assignment to the centroids of the LAST step's input; compare with the oracle's
    # assignment to those centroids (= the whole run's returned assignment)
    assert np.mean(asg == ra) > 0.999
    for t in shards:
        t.close()


def test_ivf_kat_and_errors(vsk, dev):
    """IVFIndexTests.swift:140-201: untrained use throws; basic search finds the inserted row."""
    ix = vsk.IVFIndex(dev, 4, numberOfCentroids=2, numberOfProbes=2, maxIterations=25)
    with pytest.raises(vsk.NotTrained):
        ix.insert(np.zeros((1, 4), np.float32))
    with pytest.raises(vsk.NotTrained):
        ix.batchSearch(np.zeros((1, 4), np.float32), 1)
    with pytest.raises(vsk.InsufficientTrainingData):
        ix.train(np.zeros((1, 4), np.float32))
    train = np.array([[1, 0, 0, 0], [0, 1, 0, 0], [0, 0, 1, 0], [0, 0, 0, 1],
                      [.9, .1, 0, 0], [.1, .9, 0, 0], [0, .1, .9, 0], [0, 0, .1, .9]], np.float32)
    ix.train(train)
    ix.insert(np.array([[1, 0, 0, 0], [0, 1, 0, 0], [0, 0, 1, 0]], np.float32))
    d, i = ix.search(np.array([.9, .1, 0, 0], np.float32), 1)
    assert i[0] == 0
    ix.close()


@pytest.mark.parametrize("cfg", [(20_000, 32, 64, 8, 10, 300), (50_000, 128, 256, 16, 10, 500),
                                 (3000, 17, 10, 10, 25, 40), (12_000, 16, 2, 1, 5, 64)])
def test_ivf_search_vs_oracle(vsk, dev, cpu_oracle, cfg):
    """Search parity on shared state: the GPU-trained centroids and list membership are handed to
    the oracle, which applies IVFIndex.search semantics to them."""
    n, d, nlist, nprobe, k, nq = cfg
    rng = np.random.default_rng(n + nlist)
    centres = rng.standard_normal((max(nlist, 4), d)).astype(np.float32)
    x = _mixture(rng, n, d, centres)
    q = _mixture(rng, nq, d, centres)
    ix = vsk.IVFIndex(dev, d, numberOfCentroids=nlist, numberOfProbes=nprobe, maxIterations=5, tolerance=-1.0)
    ix.train(x)
    ix.insert(x)
    asg = ix.assignments()
    ra, _ = cpu_oracle.assign(x, ix.centroids)
    assert np.mean(asg == ra) > 0.999
    gd, gi = ix.batchSearch(q, k)
    rd, ri = cpu_oracle.ivf_search(q, x, ix.centroids, asg, nprobe, k)
    assert_topk_parity(gd, gi, rd, ri)
    # `.exact` probes every list and equals the flat search (IVFIndexTests.swift:203-260)
    ed, ei = ix.batchSearch(q[:32], k, vsk.SearchStrategy.exact)
    fd, fi = cpu_oracle.flat_search(oracle.EUCLIDEAN, q[:32], x, k)
    assert_topk_parity(ed, ei, fd, fi)
    ix.close()


@pytest.mark.parametrize("cfg", [(200_000, 64, 512, 32, 10, 2000), (120_000, 128, 300, 20, 100, 1000),
                                 (60_000, 40, 64, 64, 10, 700)])
def test_ivf_tensor_list_scan(vsk, dev, cpu_oracle, cfg):
    """The probed lists scanned on the tensor cores (coarse fp16 values, certificate, exact rerank) against the
    oracle and against the fp32 list scan; lists are made very uneven (a few centres own most of the rows)."""
    n, d, nlist, nprobe, k, nq = cfg
    rng = np.random.default_rng(n + k)
    centres = rng.standard_normal((nlist, d)).astype(np.float32)
    w = rng.random(nlist) ** 4
    w /= w.sum()
    x = (centres[rng.choice(nlist, n, p=w)] + 0.15 * rng.standard_normal((n, d))).astype(np.float32)
    q = (centres[rng.choice(nlist, nq, p=w)] + 0.15 * rng.standard_normal((nq, d))).astype(np.float32)
    ix = vsk.IVFIndex(dev, d, numberOfCentroids=nlist, numberOfProbes=nprobe, maxIterations=4, tolerance=-1.0)
    ix.train(x, x[:nlist])
    ix.insert(x)
    asg = ix.assignments()
    sizes = np.bincount(asg, minlength=nlist)
    assert sizes.max() > 3 * max(1, int(np.median(sizes)))            # uneven on purpose
    before = dev.stats()
    gd, gi = ix.batchSearch(q, k)
    after = dev.stats()
    assert after["tensor_tiles"] > before["tensor_tiles"]              # the tensor path ran
    assert after["fallback_queries"] - before["fallback_queries"] <= nq // 10
    rd, ri = cpu_oracle.ivf_search(q, x, ix.centroids, asg, nprobe, k)
    assert_topk_parity(gd, gi, rd, ri)
    dev.set_search_path(vsk.PATH_FP32_SCAN)
    try:
        fd, fi = ix.batchSearch(q, k)
    finally:
        dev.set_search_path(vsk.PATH_TENSOR_RERANK)
    assert_topk_parity(gd, gi, fd, fi)
    # device pointers
    import torch
    td, ti = ix.batchSearch(torch.as_tensor(q, device="cuda"), k)
    assert np.array_equal(ti.cpu().numpy(), gi) and np.array_equal(td.cpu().numpy(), gd)
    ix.close()


def test_sq8_codes_bit_exact(vsk, dev, cpu_oracle):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((5000, 37)).astype(np.float32)
    for per_dim in (False, True):
        sq = vsk.ScalarQuantizer(dev, per_dim=per_dim)
        s, o = sq.train(x)
        rs, ro = cpu_oracle.sq8_train(x, per_dim)
        assert np.array_equal(s, rs) and np.array_equal(o, ro)
        codes = sq.quantizeBatch(x)
        assert np.array_equal(codes, cpu_oracle.sq8_encode(x, rs, ro))
        assert np.array_equal(sq.dequantizeBatch(codes), cpu_oracle.sq8_decode(codes, rs, ro))
    # the reference's round-trip pins (ScalarQuantizerTests.swift:55-94, VerifyComponents/main.swift:101-119)
    sq = vsk.ScalarQuantizer(dev)
    v = np.array([[-1.0, -0.5, 0.0, 0.5, 1.0]], np.float32)
    sq.train(v)
    assert np.max(np.abs(sq.dequantizeBatch(sq.quantizeBatch(v)) - v)) < 0.1
    w = (np.arange(128, dtype=np.float32) / 128.0)[None]
    sq.train(w)
    assert np.max(np.abs(sq.dequantizeBatch(sq.quantizeBatch(w)) - w)) < 0.01


@pytest.mark.parametrize("metric", ["dotProduct", "euclidean", "cosine", "manhattan"])
def test_sq8_search_vs_oracle(vsk, dev, cpu_oracle, metric):
    """Int8 scalar-quantised flat search: N(0,1) rows quantised per dimension with min/max scaling,
    fp32 queries, k = 10 (reduced N)."""
    import torch
    rng = np.random.default_rng(202611254)
    x = rng.standard_normal((20_000, 384)).astype(np.float32)
    q = rng.standard_normal((100, 384)).astype(np.float32)
    sq = vsk.ScalarQuantizer(dev, per_dim=True)
    xd = torch.from_numpy(x).cuda()
    s, o = sq.train(xd)
    codes = sq.quantizeBatch(xd)
    rs, ro = cpu_oracle.sq8_train(x, True)
    assert np.array_equal(s.cpu().numpy(), rs) and np.array_equal(o.cpu().numpy(), ro)
    rcodes = cpu_oracle.sq8_encode(x, rs, ro)
    assert np.array_equal(codes.cpu().numpy(), rcodes)
    ix = vsk.QuantizedFlatIndex(dev, 384, metric, s, o)
    ix.add(codes)
    gd, gi = ix.batchSearch(q, 10)
    ix.close()
    rd, ri = cpu_oracle.sq8_search(oracle.METRIC_IDS[metric], q, rcodes, rs, ro, 10)
    assert_topk_parity(gd, gi, rd, ri)


# ---- IVF: metadata filter, incremental insert, exact probing of many lists, k-means++ -------------------------

def _ivf_case(rng, n, d, nlist, nq):
    centres = rng.standard_normal((nlist, d)).astype(np.float32)
    x = _mixture(rng, n, d, centres, 0.25)
    q = _mixture(rng, nq, d, centres, 0.25)
    return centres, x, q


@pytest.mark.parametrize("nq", [1, 5, 40, 700])
def test_ivf_filtered_search_vs_oracle(vsk, dev, cpu_oracle, nq):
    """IVFIndex.search with a filter (IVFIndex.swift:162-165): the probed candidates are filtered first.  One query and
    a handful stream their lists, 40 take the fp32 list tiles, 700 the tensor-core tiles; every one with its own
    one-hot mask over Bernoulli(0.5) row masks, plus a rare bit and a bit no row has."""
    rng = np.random.default_rng(300 + nq)
    n, d, nlist, nprobe, k = 60_000, 64, 64, 8, 10
    centres, x, q = _ivf_case(rng, n, d, nlist, nq)
    rm = rng.integers(0, 2 ** 60, n, dtype=np.uint64) | ((rng.random(n) < 0.02).astype(np.uint64) << np.uint64(61))
    qm = (np.uint64(1) << rng.integers(0, 60, nq).astype(np.uint64))
    qm[::7] = np.uint64(1 << 61)
    if nq > 2:
        qm[2] = np.uint64(1 << 63)
    ix = vsk.IVFIndex(dev, d, numberOfCentroids=nlist, numberOfProbes=nprobe, maxIterations=4, tolerance=-1.0)
    try:
        ix.train(x, x[:nlist])
        ix.insert(x, rm)
        gd, gi = ix.batchSearch(q, k, filter_masks=qm)
        ud, ui = ix.batchSearch(q, k)
        cent, asg = np.asarray(ix.centroids), ix.assignments()
    finally:
        ix.close()
    rd, ri = cpu_oracle.ivf_search_filtered(q, x, cent, asg, nprobe, k, rm, qm)
    assert_topk_parity(gd, gi, rd, ri)
    ok = gi >= 0
    assert np.all(((rm[np.clip(gi, 0, None)] & qm[:, None]) != 0) | ~ok)
    if nq > 2:
        assert np.all(gi[2] == -1)
    rd, ri = cpu_oracle.ivf_search(q, x, cent, asg, nprobe, k)
    assert_topk_parity(ud, ui, rd, ri)


@pytest.mark.parametrize("masked", [False, True])
def test_ivf_incremental_insert_equals_one_shot_build(vsk, dev, cpu_oracle, masked):
    """Rows appended in blocks (and one block of a single row) land in the lists a one-shot build gives them: same
    assignments, same search results, ids = insertion indices."""
    rng = np.random.default_rng(17)
    n, d, nlist, nprobe, k, nq = 30_000, 48, 32, 6, 12, 300
    centres, x, q = _ivf_case(rng, n, d, nlist, nq)
    rm = rng.integers(1, 2 ** 62, n, dtype=np.uint64) if masked else None
    qm = (np.uint64(1) << rng.integers(0, 62, nq).astype(np.uint64)) if masked else None
    a = vsk.IVFIndex(dev, d, numberOfCentroids=nlist, numberOfProbes=nprobe, maxIterations=3, tolerance=-1.0)
    b = vsk.IVFIndex(dev, d, numberOfCentroids=nlist, numberOfProbes=nprobe, maxIterations=3, tolerance=-1.0)
    try:
        a.train(x[:5000], x[:nlist])
        b.centroids, b.trained = a.centroids, True
        a.insert(x, rm)
        cuts = [0, 7000, 7001, 19_000, n]
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            b.insert(x[lo:hi], rm[lo:hi] if masked else None)
        assert a.count == b.count == n
        assert np.array_equal(a.assignments(), b.assignments())
        ad, ai = a.batchSearch(q, k, filter_masks=qm)
        bd, bi = b.batchSearch(q, k, filter_masks=qm)
        assert np.array_equal(ai, bi) and np.array_equal(ad, bd)
        rd, ri = cpu_oracle.ivf_search_filtered(q, x, np.asarray(a.centroids), a.assignments(), nprobe, k, rm, qm)
        assert_topk_parity(bd, bi, rd, ri)
        # one-entry inserts are collected and appended before the next search
        extra = _mixture(rng, 3, d, centres, 0.25)
        for v in extra:
            b.insertEntry(v, mask=(2 ** 62 - 1) if masked else None)
        assert b.count == n + 3
        d1, i1 = b.batchSearch(extra, 1)
        assert np.array_equal(i1[:, 0], np.arange(n, n + 3)) and np.all(d1 < 1e-3)
    finally:
        a.close()
        b.close()


def test_ivf_exact_strategy_over_more_lists_than_a_candidate_list_holds(vsk, dev, cpu_oracle):
    """nprobe == nlist with more lists than a top-k selection can rank (4 100 > 2 048): every list is probed
    without a selection, the result is the flat exact search; a probe count between the two limits is refused."""
    rng = np.random.default_rng(4100)
    n, d, nlist, k = 9000, 8, 4100, 5
    x = rng.standard_normal((n, d)).astype(np.float32)
    q = rng.standard_normal((20, d)).astype(np.float32)
    ix = vsk.IVFIndex(dev, d, numberOfCentroids=nlist, numberOfProbes=nlist, maxIterations=1, tolerance=-1.0)
    try:
        ix.train(x, x[:nlist])
        ix.insert(x)
        gd, gi = ix.batchSearch(q, k, vsk.SearchStrategy.exact)
        rd, ri = cpu_oracle.flat_search(oracle.EUCLIDEAN, q, x, k)
        assert_topk_parity(gd, gi, rd, ri)
        ix.numberOfProbes = 3000
        with pytest.raises(vsk.InvalidInput):
            ix.batchSearch(q, k)
    finally:
        ix.close()


@pytest.mark.parametrize("case", [(4000, 16, 12, 7), (20_000, 64, 40, 123456789), (1500, 5, 30, 2 ** 63 + 11)])
def test_kmeans_plusplus_picks_match_the_cpu_restatement(vsk, dev, cpu_oracle, case):
    """k-means++ (KMeansClustering.swift:209-260) with the reference's seeded generator: the rows the GPU picks are
    the rows the CPU restatement picks, and the centroids are those rows."""
    n, d, k, seed = case
    rng = np.random.default_rng(n)
    x = (rng.standard_normal((n, d)) * 0.05).astype(np.float32)     # small spread: the weights sum to less than one at
    x[: n // 2] += 3.0                                               # first, so draws reach deep into the rows
    km = vsk.KMeansClustering(dev, seed=seed)
    cent, picked = km.initializeKMeansPlusPlus(x, k)
    rc, rp = cpu_oracle.kmeans_plusplus(x, k, seed)
    # The reference adds the weights as floats, one after the other; over thousands of rows that running sum drifts
    # from the true sum by up to ~1e-4 of it, so a draw can land a few rows away from where an exactly summed draw
    # lands (and every later draw then differs, since the chosen row feeds the next distances).  The GPU sums in
    # double precision.  Required: identical picks up to the first such draw, and that draw within 0.1 % of the rows.
    same = picked == rp
    if not same.all():
        j = int(np.argmin(same))
        assert n >= 10_000 and abs(int(picked[j]) - int(rp[j])) <= max(2, n // 1000), (j, picked[j], rp[j])
    assert np.array_equal(np.asarray(cent), x[picked]) and np.array_equal(rc, x[rp])
    # clustering from it runs and beats clustering from the first k rows on this two-blob data
    c1, _, _, inertia_pp = vsk.KMeansClustering(dev, maxIterations=5, tolerance=-1.0, seed=seed).cluster(x, k)
    assert np.isfinite(inertia_pp) and c1.shape == (k, d)


def test_kmeans_plusplus_degenerate_data_is_refused(vsk, dev):
    x = np.ones((50, 4), np.float32)
    with pytest.raises(vsk.InvalidInput):
        vsk.KMeansClustering(dev, seed=1).initializeKMeansPlusPlus(x, 3)
