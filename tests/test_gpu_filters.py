"""Metadata filters end to end on the GPU: row masks compiled at insert time + per-query masks give the same top-k
as the reference's order of operations — filter the candidates, then distances, then sort
(Indexes/IVFIndex.swift:163-176) — evaluated by the CPU restatements."""
import json

import numpy as np
import pytest

import oracle
from oracle import filter_ref as fr
from parity import assert_topk_parity
from test_filters_cpu import FILTERS, _random_rows, _to_ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def vsk():
    import vectorstorekit_b200 as v
    return v


@pytest.fixture(scope="module")
def dev(vsk):
    return vsk.CUDAAcceleratorStrategy(0).initialize()


@pytest.mark.parametrize("metric", ["euclidean", "cosine", "manhattan", "dotProduct"])
def test_filtered_search_equals_prefilter_then_search(vsk, dev, cpu_oracle, metric):
    rng = np.random.default_rng(21)
    n, d, nq, k = 4000, 24, 60, 15
    md, x = _random_rows(rng, n, d)
    q = rng.standard_normal((nq, d)).astype(np.float32)
    comp = vsk.FilterBitmaskCompiler()
    for f in FILTERS:
        comp.register(f)
    masks = comp.row_masks(md, x)
    ix = vsk.FlatIndex(dev, d, metric)
    ix.add(x, masks=masks)
    # each query carries one of the registered filters, or a union of two
    per_query = [FILTERS[i % len(FILTERS)] for i in range(nq - 2)]
    per_query += [vsk.CompositeFilter(vsk.LogicalOperation.or_, (FILTERS[0], FILTERS[3])),
                  vsk.CompositeFilter(vsk.LogicalOperation.or_, (FILTERS[4], FILTERS[6], FILTERS[1]))]
    qm = comp.query_masks(per_query)
    dist, ids = ix.batchSearch(q, k, filter_masks=qm)
    mid = oracle.METRIC_IDS[metric]
    for a, f in enumerate(per_query):
        ok = np.nonzero(fr.eligible_rows(_to_ref(f), md, x))[0]            # the reference's pre-filter
        rd, ri = cpu_oracle.flat_search(mid, q[a:a + 1], x[ok], k)          # distances + sort on what is left
        want_ids = np.where(ri[0] >= 0, ok[np.clip(ri[0], 0, None)], -1) if ok.size else np.full(k, -1)
        assert_topk_parity(dist[a:a + 1], ids[a:a + 1], rd, want_ids[None])
        kk = min(k, ok.size)
        assert np.all(ids[a, kk:] == -1) and np.all(np.isin(ids[a, :kk], ok))
