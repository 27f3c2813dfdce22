"""Pins the CPU oracle: known-answer values from the reference's own tests, the committed
golden vectors produced by the reference's shader source, and (where it was built) the
shader source itself, bit for bit."""
import math
import os

import numpy as np
import pytest

import oracle
from oracle import COSINE, DOT, EUCLIDEAN, MANHATTAN

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "metal_shader_vectors.npz"))
NAMES = ["euclidean", "cosine", "dotProduct", "manhattan"]


# --- known answers: Tests/VectorStoreKitTests/ValidationTests/Phase1ValidationTests.swift:143-172
def test_kat_phase1(cpu_oracle):
    assert abs(cpu_oracle.distance(EUCLIDEAN, [1, 0, 0, 0], [0, 1, 0, 0]) - math.sqrt(2)) < 1e-4
    assert abs(cpu_oracle.distance(COSINE, [1, 0, 0, 0], [0, 1, 0, 0]) - 1.0) < 1e-4
    assert abs(cpu_oracle.distance(MANHATTAN, [1, 0, 0, 0], [1, 1, 1, 1]) - 3.0) < 1e-4


# --- Tests/VectorStoreKitTests/MetalDistance512Tests.swift:50-66,94-116,156-182
def test_kat_d512(cpu_oracle):
    z = np.zeros(512, np.float32)
    assert abs(cpu_oracle.distance(EUCLIDEAN, z, np.ones(512)) - math.sqrt(512)) < 1e-3
    assert abs(cpu_oracle.distance(EUCLIDEAN, z, 2 * np.ones(512)) - math.sqrt(2048)) < 1e-3
    cand = np.stack([np.full(512, (i % 100) / 100.0, np.float32) for i in range(1000)])
    d = cpu_oracle.batch_distances(EUCLIDEAN, z[None], cand)[0]
    exp = np.sqrt(512.0 * ((np.arange(1000) % 100) / 100.0) ** 2)
    assert np.max(np.abs(d - exp)) < 1e-2
    q = np.stack([np.full(512, float(i), np.float32) for i in range(10)])
    c = np.stack([np.full(512, float(j), np.float32) for j in range(100)])
    dm = cpu_oracle.batch_distances(EUCLIDEAN, q, c)
    exp = np.sqrt(512.0 * (np.arange(10)[:, None] - np.arange(100)[None, :]) ** 2)
    assert np.max(np.abs(dm - exp)) < 1e-2


# --- Tests/VectorStoreKitTests/MetalDistanceMatrixTests.swift:27-55,76-139
def test_kat_matrix(cpu_oracle):
    one, two = np.ones((1, 512), np.float32), 2 * np.ones((1, 512), np.float32)
    assert abs(cpu_oracle.batch_distances(MANHATTAN, one, two)[0, 0] - 512.0) < 1e-2
    assert abs(cpu_oracle.batch_distances(COSINE, one, two)[0, 0]) < 1e-2
    rng = np.random.default_rng(1)
    v = rng.uniform(-1, 1, (20, 512)).astype(np.float32)
    m = cpu_oracle.batch_distances(EUCLIDEAN, v, v)
    assert np.max(np.abs(m - m.T)) < 1e-4 and np.max(np.abs(np.diag(m))) < 1e-4


# --- Tests/VectorStoreKitTests/Vector512Tests.swift:61-101
def test_kat_vector512(cpu_oracle):
    one = np.ones(512, np.float32)
    assert abs(-cpu_oracle.distance(DOT, one, 2 * one) - 1024.0) < 1e-3
    assert abs(cpu_oracle.distance(EUCLIDEAN, one, 3 * one) ** 2 - 2048.0) < 0.5
    assert abs((1 - cpu_oracle.distance(COSINE, one, 5 * one)) - 1.0) < 1e-3
    a = np.zeros(512, np.float32); a[0] = 1
    b = np.zeros(512, np.float32); b[1] = 1
    assert abs(1 - cpu_oracle.distance(COSINE, a, b)) < 1e-3


# --- Tests/VectorStoreKitTests/MetalComputeIntegrationTests.swift:11-86
def test_kat_four_metrics_finite(cpu_oracle):
    rng = np.random.default_rng(2)
    q = rng.uniform(-1, 1, 4).astype(np.float32)
    c = rng.uniform(-1, 1, (100, 4)).astype(np.float32)
    c[0] = q
    for m in (EUCLIDEAN, COSINE, MANHATTAN, DOT):
        d = cpu_oracle.batch_distances(m, q[None], c)[0]
        assert np.all(np.isfinite(d))
        if m != DOT:
            assert np.all(d >= -1e-6) and abs(d[0]) < 1e-3


# --- Tests/VectorStoreKitTests/ScalarQuantizerTests.swift:55-94,146-168; Sources/VerifyComponents/main.swift:101-119
def test_kat_int8_round_trip(cpu_oracle):
    v = np.array([[-1.0, -0.5, 0.0, 0.5, 1.0]], np.float32)
    s, o = cpu_oracle.sq8_train(v, per_dim=False)
    assert np.all(s == s[0]) and np.all(o == o[0])          # a batch shares one scale/offset
    back = cpu_oracle.sq8_decode(cpu_oracle.sq8_encode(v, s, o), s, o)
    assert np.max(np.abs(back - v)) < 0.1
    w = (np.arange(128, dtype=np.float32) / 128.0)[None]
    s, o = cpu_oracle.sq8_train(w, per_dim=False)
    back = cpu_oracle.sq8_decode(cpu_oracle.sq8_encode(w, s, o), s, o)
    assert np.max(np.abs(back - w)) < 0.01
    # parameters: ScalarQuantizer.swift:428-431
    assert s[0] == np.float32(255.0) / (w.max() - w.min())
    assert o[0] == -w.min() * s[0] - np.float32(128.0)
    codes = cpu_oracle.sq8_encode(w, s, o)
    assert codes.dtype == np.int8 and codes.min() == -128 and codes.max() <= 127


def test_int8_truncates_toward_zero(cpu_oracle):
    x = np.array([[0.26, -0.26, 0.999, -0.999]], np.float32)
    codes = cpu_oracle.sq8_encode(x, np.full(4, 10, np.float32), np.zeros(4, np.float32))
    assert codes.tolist() == [[2, -2, 9, -9]]


# --- Tests/VectorStoreKitTests/IVFIndexTests.swift:160-201 (basic search) and :203-260 (exact finds itself)
def test_kat_ivf_basic(cpu_oracle):
    train = np.array([[1, 0, 0, 0], [0, 1, 0, 0], [0, 0, 1, 0], [0, 0, 0, 1],
                      [.9, .1, 0, 0], [.1, .9, 0, 0], [0, .1, .9, 0], [0, 0, .1, .9]], np.float32)
    cent, asg, _, _ = cpu_oracle.kmeans(train, train[:2], 25, 1e-4)
    rows = np.array([[1, 0, 0, 0], [0, 1, 0, 0], [0, 0, 1, 0]], np.float32)
    a, _ = cpu_oracle.assign(rows, cent)
    d, ids = cpu_oracle.ivf_search(np.array([[.9, .1, 0, 0]], np.float32), rows, cent, a, 2, 1)
    assert ids[0, 0] == 0
    rng = np.random.default_rng(3)
    x = rng.uniform(-1, 1, (100, 16)).astype(np.float32)
    cent, _, _, _ = cpu_oracle.kmeans(x, x[:4], 10)
    a, _ = cpu_oracle.assign(x, cent)
    d, ids = cpu_oracle.ivf_search(x[50:51], x, cent, a, 4, 5)       # .exact probes every list
    assert ids[0, 0] == 50 and d[0, 0] == 0.0
    d2, ids2 = cpu_oracle.flat_search(EUCLIDEAN, x[50:51], x, 5)
    assert np.array_equal(ids, ids2) and np.array_equal(d, d2)


# --- golden vectors produced by the reference's shader source (tests/golden/make_golden.py)
@pytest.mark.parametrize("mid", range(4))
def test_golden_batch_distances_bit_exact(cpu_oracle, mid):
    got = cpu_oracle.batch_distances(mid, GOLD["dist_q"], GOLD["dist_x"])
    assert np.array_equal(got, GOLD[f"dist_{NAMES[mid]}"])
    got1 = cpu_oracle.batch_distances(mid, GOLD["single_q"][None], GOLD["single_x"])[0]
    assert np.array_equal(got1, GOLD[f"single_{NAMES[mid]}"])


def test_golden_kmeans_steps_bit_exact(cpu_oracle):
    x, c0 = GOLD["km_x"], GOLD["km_c0"]
    for it in (1, 2, 3):
        cent, asg, inertia, iters = cpu_oracle.kmeans(x, c0, it)
        assert iters == it
        assert np.array_equal(cent, GOLD[f"km_c{it}"])
    # assignments returned are those of the last assignment step
    cent2, _, _, _ = cpu_oracle.kmeans(x, c0, 2)
    a, dist = cpu_oracle.assign(x, cent2)
    assert np.array_equal(a, GOLD["km_assign3"]) and np.array_equal(dist, GOLD["km_dist3"])
    # the far-away centroid never receives a row and keeps its value (ClusteringShaders.metal:171-176)
    assert np.array_equal(GOLD["km_c3"][5], c0[5])


def test_golden_shader_uint8_round_trip():
    assert np.max(np.abs(GOLD["q_back"] - GOLD["q_in"])) <= 0.5 / 255 + 1e-6


# --- the shader source itself, where it was built from the reference tree
@pytest.mark.parametrize("mid", range(4))
def test_restatement_equals_shader_source(cpu_oracle, metal_ref, mid):
    rng = np.random.default_rng(100 + mid)
    for (nq, nx, d) in [(3, 50, 1), (5, 33, 129), (2, 17, 768)]:
        q = rng.standard_normal((nq, d)).astype(np.float32)
        x = rng.standard_normal((nx, d)).astype(np.float32)
        assert np.array_equal(cpu_oracle.batch_distances(mid, q, x), metal_ref.batch_distances(mid, q, x))


def test_kmeans_equals_shader_source(cpu_oracle, metal_ref):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((500, 12)).astype(np.float32)
    c = x[:9].copy()
    for it in range(4):
        c, asg, dist = metal_ref.kmeans_step(x, c)
    cent, _, _, _ = cpu_oracle.kmeans(x, x[:9], 4)
    assert np.array_equal(cent, c)
    assert np.allclose(metal_ref.min_distances(x, c) ** 0.5, cpu_oracle.assign(x, c)[1], rtol=1e-6)


# --- top-k semantics
def test_flat_search_is_sorted_prefix(cpu_oracle):
    rng = np.random.default_rng(5)
    q = rng.standard_normal((6, 24)).astype(np.float32)
    x = rng.standard_normal((200, 24)).astype(np.float32)
    for mid in range(4):
        full = cpu_oracle.batch_distances(mid, q, x)
        d, ids = cpu_oracle.flat_search(mid, q, x, 10)
        order = np.lexsort((np.arange(200)[None].repeat(6, 0), full), axis=1)[:, :10]
        assert np.array_equal(ids, order)
        assert np.array_equal(d, np.take_along_axis(full, order, 1))
        df, idf = cpu_oracle.flat_search(mid, q, x, 10, fast=True)
        assert np.allclose(df, d, rtol=1e-5, atol=1e-6)


def test_flat_search_filter_and_short_lists(cpu_oracle):
    rng = np.random.default_rng(6)
    q = rng.standard_normal((4, 8)).astype(np.float32)
    x = rng.standard_normal((30, 8)).astype(np.float32)
    rm = rng.integers(0, 2 ** 63, 30, dtype=np.uint64)
    qm = np.array([1 << 3, 1 << 7, 1 << 62, 0], np.uint64)
    d, ids = cpu_oracle.flat_search(MANHATTAN, q, x, 25, rm, qm)
    for a in range(4):
        ok = np.nonzero(rm & qm[a])[0]
        n = min(25, ok.size)
        assert set(ids[a, :n]) <= set(ok) and np.all(ids[a, n:] == -1) and np.all(np.isinf(d[a, n:]))
    assert np.all(ids[3] == -1)


def test_merge_equals_unsharded(cpu_oracle):
    rng = np.random.default_rng(8)
    q = rng.standard_normal((5, 16)).astype(np.float32)
    x = rng.standard_normal((400, 16)).astype(np.float32)
    d, ids = cpu_oracle.flat_search(EUCLIDEAN, q, x, 7)
    parts = [cpu_oracle.flat_search(EUCLIDEAN, q, x[s * 100:(s + 1) * 100], 7) for s in range(4)]
    pd = np.stack([p[0] for p in parts])
    pi = np.stack([p[1] + s * 100 for s, p in enumerate(parts)])
    md, mi = cpu_oracle.merge_topk(pd, pi)
    assert np.array_equal(mi, ids) and np.array_equal(md, d)


def test_sq8_search_matches_decode_then_flat(cpu_oracle):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((300, 24)).astype(np.float32)
    q = rng.standard_normal((5, 24)).astype(np.float32)
    s, o = cpu_oracle.sq8_train(x, per_dim=True)
    codes = cpu_oracle.sq8_encode(x, s, o)
    xd = cpu_oracle.sq8_decode(codes, s, o)
    assert np.max(np.abs(xd - x)) < (x.max() - x.min()) / 255 * 1.01
    d, ids = cpu_oracle.sq8_search(DOT, q, codes, s, o, 10)
    d2, ids2 = cpu_oracle.flat_search(DOT, q, xd, 10)
    assert np.array_equal(ids, ids2) and np.array_equal(d, d2)


# ---- product quantisation ------------------------------------------------------------------------------------
def test_pq_encode_decode_equal_reference_shaders(cpu_oracle):
    """Golden outputs of the reference's productQuantize / productDequantize shaders
    (QuantizationShaders.metal:113-204); codeword 200 duplicates 17, so ties resolve to the lower code."""
    codes = cpu_oracle.pq_encode(GOLD["pq_x"], GOLD["pq_cb"])
    assert np.array_equal(codes, GOLD["pq_codes"])
    assert not np.any(codes == 200) and np.any(codes == 17)
    assert np.array_equal(cpu_oracle.pq_decode(codes, GOLD["pq_cb"]), GOLD["pq_back"])


def test_pq_shaders_live(cpu_oracle, metal_ref):
    rng = np.random.default_rng(12)
    x = rng.standard_normal((150, 32)).astype(np.float32)
    cb = rng.standard_normal((8, 256, 4)).astype(np.float32)
    codes = metal_ref.product_quantize(x, cb)
    assert np.array_equal(cpu_oracle.pq_encode(x, cb), codes)
    assert np.array_equal(cpu_oracle.pq_decode(codes, cb), metal_ref.product_dequantize(codes, cb))


def test_pq_tables_and_distance_by_hand(cpu_oracle):
    """ProductQuantizer.precomputeDistanceTables (:205-233) and DistanceTables.computeDistance
    (ProductQuantizerTypes.swift:14-20) on numbers worked out by hand: 2 segments of 2 dimensions, 2 codewords."""
    cb = np.array([[[0, 0], [1, 1]], [[2, 0], [0, 3]]], np.float32)
    q = np.array([[1, 0, 0, 0]], np.float32)
    t = cpu_oracle.pq_tables(q, cb)
    assert np.array_equal(t[0], np.array([[1, 1], [4, 9]], np.float32))
    codes = np.array([[0, 0], [1, 1], [0, 1], [1, 0]], np.uint8)
    d, ids = cpu_oracle.pq_search(q, codes, cb, 4)
    # sums 5, 10, 10, 5 -> sqrt; ties keep row order
    assert np.array_equal(ids[0], [0, 3, 1, 2])
    assert np.allclose(d[0], np.sqrt(np.array([5, 5, 10, 10], np.float32)))
    # asymmetric distance == distance to the decoded row when the per-segment sums add exactly
    back = cpu_oracle.pq_decode(codes, cb)
    assert np.allclose(d[0], np.sort(np.sqrt(((q - back) ** 2).sum(1))))


def test_pq_search_equals_table_sums(cpu_oracle):
    rng = np.random.default_rng(13)
    x = rng.standard_normal((500, 16)).astype(np.float32)
    q = rng.standard_normal((6, 16)).astype(np.float32)
    init = np.stack([x[:16, s * 4:(s + 1) * 4] for s in range(4)])
    cb = cpu_oracle.pq_train(x, init, 4)
    codes = cpu_oracle.pq_encode(x, cb)
    t = cpu_oracle.pq_tables(q, cb)
    d, ids = cpu_oracle.pq_search(q, codes, cb, 9)
    for a in range(6):
        s = np.zeros(500, np.float32)
        for seg in range(4):
            s = s + t[a, seg, codes[:, seg]]            # fp32 adds in segment order
        full = np.sqrt(s)
        order = np.lexsort((np.arange(500), full))[:9]
        assert np.array_equal(ids[a], order) and np.array_equal(d[a], full[order])
    # training moved the codewords to the means of their cells
    asg = cpu_oracle.pq_encode(x, cb)
    assert len(np.unique(asg[:, 0])) > 8
