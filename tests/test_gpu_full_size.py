"""The benchmark configurations at FULL size.

* the CPU oracle runs at full N on a fixed subset of 64 queries (seconds on the host cores) and the GPU result of
  those queries must match it under the acceptance rule (ids identical except ties within 1e-5 relative distance,
  distances within 1e-4 relative).  The IVF case hands the GPU-trained centroids and list membership to the oracle,
  so that the search is compared on shared state (20 Lloyd iterations amplify summation-order differences);
* the tensor-core path and the fp32 direct-formula path are two independent implementations inside the library: on a
  larger sample of the queries the two must agree as well;
* planted rows: queries that ARE database rows must find that row first, at distance 0;
* every result row is ascending, its ids are distinct and inside the index;
* the accumulation term of the tensor path's error bound is measured against fp64 on exact fp16 operands.
"""
import numpy as np
import pytest

import oracle
from parity import assert_topk_parity

pytestmark = pytest.mark.gpu

ORACLE_QUERIES = 64


@pytest.fixture(scope="module")
def vsk():
    import vectorstorekit_b200 as v
    return v


@pytest.fixture(scope="module")
def dev(vsk):
    return vsk.CUDAAcceleratorStrategy(0).initialize()


def _check_rows(d, i, n):
    assert np.all(np.diff(d, axis=1) >= 0)
    assert i.min() >= 0 and i.max() < n
    s = np.sort(i, axis=1)
    assert np.all(s[:, 1:] != s[:, :-1])


def _subset(nq):
    return np.arange(25, nq, nq // ORACLE_QUERIES)[:ORACLE_QUERIES]


def test_flat_cosine_1m_d768_q10000_k100(vsk, dev, cpu_oracle):
    """Flat cosine, 1 000 000 x 768, 10 000 queries, k = 100 (rows and queries L2-normalised)."""
    import torch
    n, d, nq, k = 1_000_000, 768, 10_000, 100
    g = torch.Generator(device="cuda").manual_seed(7)
    ix = vsk.FlatIndex(dev, d, "cosine")
    xh = np.empty((n, d), np.float32)                      # the same bytes for the oracle
    try:
        for lo in range(0, n, 250_000):
            x = torch.randn((250_000, d), generator=g, device="cuda")
            x /= x.norm(dim=1, keepdim=True)
            ix.add(x)
            xh[lo:lo + 250_000] = x.cpu().numpy()
            if lo == 0:
                planted = x[:50].clone()
        q = torch.randn((nq, d), generator=g, device="cuda")
        q /= q.norm(dim=1, keepdim=True)
        q[:50] = planted                                   # queries 0..49 are rows 0..49
        before = dev.stats()
        td, ti = ix.batchSearch(q, k)
        after = dev.stats()
        assert after["tensor_tiles"] > before["tensor_tiles"]
        assert after["fallback_queries"] - before["fallback_queries"] <= nq // 100
        gd, gi = td.cpu().numpy(), ti.cpu().numpy()
        _check_rows(gd, gi, n)
        assert np.array_equal(gi[:50, 0], np.arange(50)) and np.all(np.abs(gd[:50, 0]) < 1e-6)
        # CPU oracle, all rows, 64 fixed queries
        sub = _subset(nq)
        rd, ri = cpu_oracle.flat_search(oracle.COSINE, q.cpu().numpy()[sub], xh, k)
        assert_topk_parity(gd[sub], gi[sub], rd, ri)
        del xh
        sample = torch.arange(0, nq, nq // 100, device="cuda")
        dev.set_search_path(vsk.PATH_FP32_SCAN)
        try:
            fd, fi = ix.batchSearch(q[sample].contiguous(), k)
        finally:
            dev.set_search_path(vsk.PATH_TENSOR_RERANK)
        s = sample.cpu().numpy()
        assert_topk_parity(gd[s], gi[s], fd.cpu().numpy(), fi.cpu().numpy())
    finally:
        ix.close()


def test_ivf_euclidean_10m_d128_nlist4096_nprobe32(vsk, dev, cpu_oracle):
    """IVF, 10 000 000 x 128 from a mixture of 4 096 centres (noise 0.1), nlist 4 096, 20 Lloyd iterations,
    10 000 queries, nprobe 32, k = 10."""
    import torch
    n, d, nlist, nprobe, nq, k = 10_000_000, 128, 4096, 32, 10_000, 10
    g = torch.Generator(device="cuda").manual_seed(11)
    centres = torch.randn((nlist, d), generator=g, device="cuda")
    x = torch.empty((n, d), device="cuda")
    for lo in range(0, n, 1_000_000):
        c = torch.randint(0, nlist, (1_000_000,), generator=g, device="cuda")
        x[lo:lo + 1_000_000] = centres[c] + 0.1 * torch.randn((1_000_000, d), generator=g, device="cuda")
    c = torch.randint(0, nlist, (nq,), generator=g, device="cuda")
    q = centres[c] + 0.1 * torch.randn((nq, d), generator=g, device="cuda")
    q[:50] = x[:50]
    ix = vsk.IVFIndex(dev, d, numberOfCentroids=nlist, numberOfProbes=nprobe, maxIterations=20, tolerance=-1.0)
    try:
        ix.train(x, x[:nlist].contiguous())
        ix.insert(x)
        assert ix.count == n
        before = dev.stats()
        td, ti = ix.batchSearch(q, k)
        after = dev.stats()
        assert after["tensor_tiles"] > before["tensor_tiles"]
        assert after["fallback_queries"] - before["fallback_queries"] <= nq // 100
        gd, gi = td.cpu().numpy(), ti.cpu().numpy()
        _check_rows(gd, gi, n)
        assert np.array_equal(gi[:50, 0], np.arange(50)) and np.all(gd[:50, 0] < 1e-3)
        # CPU oracle on shared state: the GPU's centroids and list membership, IVFIndex.search semantics
        sub = _subset(nq)
        cent = ix.centroids.cpu().numpy() if hasattr(ix.centroids, "cpu") else np.asarray(ix.centroids)
        rd, ri = cpu_oracle.ivf_search(q.cpu().numpy()[sub], x.cpu().numpy(), cent, ix.assignments(), nprobe, k)
        assert_topk_parity(gd[sub], gi[sub], rd, ri)
        sample = torch.arange(0, nq, nq // 200, device="cuda")
        dev.set_search_path(vsk.PATH_FP32_SCAN)
        try:
            fd, fi = ix.batchSearch(q[sample].contiguous(), k)
        finally:
            dev.set_search_path(vsk.PATH_TENSOR_RERANK)
        s = sample.cpu().numpy()
        assert_topk_parity(gd[s], gi[s], fd.cpu().numpy(), fi.cpu().numpy())
    finally:
        ix.close()


def test_filtered_manhattan_5m_d256_q10000_k50(vsk, dev, cpu_oracle):
    """Filtered flat search, Manhattan: 5 000 000 x 256 uniform in [-1, 1], a uint64 mask per row with Bernoulli(0.5)
    bits, 10 000 queries each with a one-hot mask (about half the rows pass), k = 50."""
    import torch
    n, d, nq, k = 5_000_000, 256, 10_000, 50
    g = torch.Generator(device="cuda").manual_seed(13)
    ix = vsk.FlatIndex(dev, d, "manhattan")
    xh = np.empty((n, d), np.float32)
    mh = np.empty(n, np.uint64)
    try:
        for lo in range(0, n, 1_000_000):
            x = torch.rand((1_000_000, d), generator=g, device="cuda") * 2 - 1
            a = torch.randint(0, 2 ** 31, (1_000_000, 2), generator=g, device="cuda", dtype=torch.int64)
            b = torch.randint(0, 4, (1_000_000,), generator=g, device="cuda", dtype=torch.int64)
            m = (a[:, 0] | (a[:, 1] << 31) | (b << 62)).contiguous()
            ix.add(x, m)
            xh[lo:lo + 1_000_000] = x.cpu().numpy()
            mh[lo:lo + 1_000_000] = m.cpu().numpy().view(np.uint64)
        q = torch.rand((nq, d), generator=g, device="cuda") * 2 - 1
        qm = (torch.ones(nq, dtype=torch.int64, device="cuda")
              << torch.randint(0, 64, (nq,), generator=g, device="cuda")).contiguous()
        td, ti = ix.batchSearch(q, k, qm)
        gd, gi = td.cpu().numpy(), ti.cpu().numpy()
        _check_rows(gd, gi, n)
        qmh = qm.cpu().numpy().view(np.uint64)
        assert np.all((mh[gi] & qmh[:, None]) != 0)
        sub = _subset(nq)
        rd, ri = cpu_oracle.flat_search(oracle.MANHATTAN, q.cpu().numpy()[sub], xh, k, mh, qmh[sub])
        assert_topk_parity(gd[sub], gi[sub], rd, ri)
    finally:
        ix.close()


def test_int8_dot_shard_6m25_d384_q10000_k10(vsk, dev, cpu_oracle):
    """One rank's shard of the int8 workload: 6 250 000 x 384 N(0,1) rows quantised per dimension to int8 (min/max
    scaling over the shard), 10 000 fp32 queries, dot product against the dequantised rows, k = 10.  Rows are
    generated and encoded slab by slab; the fp32 source is dropped after encoding."""
    import torch
    n, d, nq, k = 6_250_000, 384, 10_000, 10
    step = 1_250_000
    sq = vsk.ScalarQuantizer(dev, per_dim=True)
    mn = mx = None
    for s in range(n // step):
        g = torch.Generator(device="cuda").manual_seed(1700 + s)
        x = torch.randn((step, d), generator=g, device="cuda")
        a, c = sq.minmax(x)
        mn = a if mn is None else torch.minimum(mn, a)
        mx = c if mx is None else torch.maximum(mx, c)
    scale, offset = sq.set_range(mn, mx)
    ix = vsk.QuantizedFlatIndex(dev, d, "dotProduct", scale, offset)
    codes_h = np.empty((n, d), np.int8)
    try:
        for s in range(n // step):
            g = torch.Generator(device="cuda").manual_seed(1700 + s)
            x = torch.randn((step, d), generator=g, device="cuda")
            codes = sq.quantizeBatch(x)
            ix.add(codes)
            codes_h[s * step:(s + 1) * step] = codes.cpu().numpy()
        g = torch.Generator(device="cuda").manual_seed(1799)
        q = torch.randn((nq, d), generator=g, device="cuda")
        before = dev.stats()
        td, ti = ix.batchSearch(q, k)
        after = dev.stats()
        assert after["tensor_tiles"] > before["tensor_tiles"]
        gd, gi = td.cpu().numpy(), ti.cpu().numpy()
        _check_rows(gd, gi, n)
        sub = _subset(nq)[:32]
        rd, ri = cpu_oracle.sq8_search(oracle.DOT, q.cpu().numpy()[sub], codes_h, scale.cpu().numpy(), offset.cpu().numpy(), k)
        assert_topk_parity(gd[sub], gi[sub], rd, ri)
    finally:
        ix.close()


@pytest.mark.parametrize("d", [768, 1536, 4096])
def test_tensor_accumulation_error_is_inside_the_certificate_term(vsk, dev, d):
    """The certificate charges dim16 * 2^-22 * |q'| * |x'| for fp32 accumulation inside the tensor cores.  With
    operands that ARE fp16 numbers (so no operand rounding happens) the contraction's raw result is compared with
    the fp64 dot product of the same numbers: the observed error must stay inside that term (headroom printed), and
    the full per-query bound eps must cover it as well."""
    import torch
    n, nq = 4096, 512
    g = torch.Generator(device="cuda").manual_seed(900 + d)
    # N(0,1) rounded to fp16: full 11-bit significands, and still fp16 numbers after any power-of-two operand scale
    # the library may choose (|values| stay far inside fp16's range), so the operands carry no rounding of their own
    x = torch.randn((n, d), generator=g, device="cuda").half().float().contiguous()
    q = torch.randn((nq, d), generator=g, device="cuda").half().float().contiguous()
    ix = vsk.FlatIndex(dev, d, "dotProduct")
    try:
        ix.add(x)
        coarse, eps = ix.coarseValues(q, n)               # coarse = -(q.x) as the contraction computed it
    finally:
        ix.close()
    exact = -(q.double() @ x.double().T)
    err = (coarse.double() - exact).abs()
    qn = q.double().norm(dim=1)
    xn = x.double().norm(dim=1)
    dim16 = -(-d // 64) * 64
    term = dim16 * 2.0 ** -22 * qn[:, None] * xn[None, :]
    ratio = float((err / term).max())
    print(f"d={d}: max |acc - exact| / (dim16 * 2^-22 * |q||x|) = {ratio:.4f}  (max abs err {float(err.max()):.3e})")
    assert ratio <= 1.0
    assert bool((err <= eps.double()[:, None]).all())


@pytest.mark.parametrize("metric", ["euclidean", "cosine", "dotProduct"])
def test_coarse_values_stay_within_eps_of_the_exact_values(vsk, dev, metric):
    """On ordinary fp32 data the coarse value of every (query, row) pair lies within the query's eps of the exact
    value (fp64 of the reference's formula; squared form for euclidean, without |q|^2; cosine without its 1): the inequality the
    certificate rests on."""
    import torch
    rng = np.random.default_rng(31)
    n, d, nq = 4096, 200, 256
    x = rng.standard_normal((n, d)).astype(np.float32) * 3.0
    q = rng.standard_normal((nq, d)).astype(np.float32)
    ix = vsk.FlatIndex(dev, d, metric)
    try:
        ix.add(x)
        coarse, eps = ix.coarseValues(torch.as_tensor(q, device="cuda"), n)
    finally:
        ix.close()
    coarse, eps = coarse.cpu().numpy().astype(np.float64), eps.cpu().numpy().astype(np.float64)
    q64, x64 = q.astype(np.float64), x.astype(np.float64)
    dot = q64 @ x64.T
    if metric == "euclidean":
        ref = (x64 ** 2).sum(1)[None, :] - 2.0 * dot                     # |x|^2 - 2 q.x
    elif metric == "cosine":
        # the scan ranks by -cos; the row-independent "1 +" is added when the distance is formed
        ref = -dot / (np.linalg.norm(q64, axis=1)[:, None] * np.linalg.norm(x64, axis=1)[None, :] + 1e-8)
    else:
        ref = -dot
    excess = np.abs(coarse - ref) - eps[:, None]
    print(f"{metric}: max |coarse - exact| / eps = {float((np.abs(coarse - ref) / eps[:, None]).max()):.4f}")
    assert np.all(excess <= 0.0)
