"""The headline configurations at FULL size, checked through properties that need no CPU oracle run:

* the tensor-core path and the fp32 direct-formula path are two independent implementations inside the library; the
  fp32 path is checked against the CPU oracle at reduced sizes (test_gpu_flat.py, test_gpu_ivf_sq8.py), so on a sample
  of the queries of the full-size run the two must agree under the acceptance rule;
* planted rows: queries that ARE database rows must find that row first, at distance 0;
* every result row is ascending, its ids are distinct and inside the index.
"""
import numpy as np
import pytest

from parity import assert_topk_parity

pytestmark = pytest.mark.gpu


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


def test_flat_cosine_1m_d768_q10000_k100(vsk, dev):
    """Flat cosine, 1 000 000 x 768, 10 000 queries, k = 100 (rows and queries L2-normalised)."""
    import torch
    n, d, nq, k = 1_000_000, 768, 10_000, 100
    g = torch.Generator(device="cuda").manual_seed(7)
    ix = vsk.FlatIndex(dev, d, "cosine")
    try:
        for lo in range(0, n, 250_000):
            x = torch.randn((250_000, d), generator=g, device="cuda")
            x /= x.norm(dim=1, keepdim=True)
            ix.add(x)
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


def test_ivf_euclidean_10m_d128_nlist4096_nprobe32(vsk, dev):
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
