"""The caller-side layer (string ids, metadata, SearchResult, SearchFilter) end to end on the GPU, with the reference's
own filter tests as known answers (Tests/VectorStoreKitTests/IVFIndexTests.swift:536-678): category == "A" leaves
{v1, v3}; magnitude in 1...3 leaves {medium, large}; category == "A" AND value >= "15" leaves {v2}."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def vsk():
    import vectorstorekit_b200 as v
    return v


@pytest.fixture(scope="module")
def dev(vsk):
    return vsk.CUDAAcceleratorStrategy(0).initialize()


UNIT = [[1, 0, 0, 0], [0, 1, 0, 0], [0, 0, 1, 0], [0, 0, 0, 1]]


def _ivf(vsk, dev, training):
    ix = vsk.IVFVectorIndex(dev, 4, numberOfCentroids=2, numberOfProbes=2, seed=5)
    ix.train(np.array(training, np.float32))
    return ix


def test_reference_metadata_filter_kat(vsk, dev):
    ix = _ivf(vsk, dev, UNIT)
    for i, (cat, val) in enumerate([("A", 10), ("B", 20), ("A", 30), ("B", 40)]):
        r = ix.insert(vsk.VectorEntry(f"v{i + 1}", UNIT[i], {"category": cat, "value": val}))
        assert r.success
    flt = vsk.MetadataFilter("category", vsk.FilterOperation.equals, "A")
    res = ix.search([0.5, 0.5, 0.5, 0.5], 10, vsk.SearchStrategy.exact, flt)
    assert len(res) == 2 and {r.id for r in res} == {"v1", "v3"}
    assert all(r.metadata["category"] == "A" for r in res)
    assert all(abs(r.distance - 1.0) < 1e-6 for r in res)          # |(0.5,0.5,0.5,0.5) - e_i| = 1
    # no filter: all four, every distance 1, ids in insertion order on the tie
    res = ix.search([0.5, 0.5, 0.5, 0.5], 10, vsk.SearchStrategy.exact)
    assert [r.id for r in res] == ["v1", "v2", "v3", "v4"]
    ix.close()


def test_reference_vector_magnitude_filter_kat(vsk, dev):
    ix = _ivf(vsk, dev, [[1, 0, 0, 0], [0, 1, 0, 0], [2, 2, 0, 0], [0, 0, 3, 3]])
    for name, v in (("small", [0.5, 0.5, 0, 0]), ("medium", [1, 1, 0, 0]), ("large", [2, 2, 0, 0])):
        ix.insert(vsk.VectorEntry(name, v, {"label": name}))
    flt = vsk.VectorFilter(("magnitude", 1.0, 3.0))
    res = ix.search([1, 1, 0, 0], 10, vsk.SearchStrategy.exact, flt)
    assert [r.id for r in res] == ["medium", "large"]
    assert res[0].distance == 0.0 and abs(res[1].distance - np.sqrt(2.0)) < 1e-6
    ix.close()


def test_reference_composite_filter_kat(vsk, dev):
    ix = _ivf(vsk, dev, UNIT)
    for i, (cat, val) in enumerate([("A", 10), ("A", 20), ("B", 30), ("B", 40)]):
        ix.insert(vsk.VectorEntry(f"v{i + 1}", UNIT[i], {"category": cat, "value": val}))
    flt = vsk.CompositeFilter(vsk.LogicalOperation.and_, (
        vsk.MetadataFilter("category", vsk.FilterOperation.equals, "A"),
        vsk.MetadataFilter("value", vsk.FilterOperation.greaterThanOrEqual, "15")))
    res = ix.search([0.5, 0.5, 0.5, 0.5], 10, vsk.SearchStrategy.exact, flt)
    assert len(res) == 1 and res[0].id == "v2"
    # a second filter registered after the rows were stored: the masks are recomputed, and inserts keep working
    ix.insert(vsk.VectorEntry("v5", [0.9, 0.1, 0, 0], {"category": "A", "value": 50}))
    only_b = vsk.MetadataFilter("category", vsk.FilterOperation.equals, "B")
    assert {r.id for r in ix.search([0.5, 0.5, 0.5, 0.5], 10, vsk.SearchStrategy.exact, only_b)} == {"v3", "v4"}
    assert {r.id for r in ix.search([0.5, 0.5, 0.5, 0.5], 10, vsk.SearchStrategy.exact, flt)} == {"v2", "v5"}
    ix.close()


def test_flat_vector_store_ids_metadata_and_filters(vsk, dev, cpu_oracle):
    import oracle
    rng = np.random.default_rng(12)
    n, d = 3000, 24
    x = rng.standard_normal((n, d)).astype(np.float32)
    store = vsk.VectorStore(dev, d, "cosine")
    store.add([vsk.VectorEntry(f"doc-{i}", x[i], {"lang": "en" if i % 3 else "de", "rank": i % 7}) for i in range(n)])
    q = rng.standard_normal((5, d)).astype(np.float32)
    res = store.batchSearch(q, 8)
    rd, ri = cpu_oracle.flat_search(oracle.COSINE, q, x, 8)
    for a in range(5):
        assert [r.id for r in res[a]] == [f"doc-{i}" for i in ri[a]]
        assert np.allclose([r.distance for r in res[a]], rd[a], rtol=1e-4, atol=1e-6)
    de = vsk.MetadataFilter("lang", vsk.FilterOperation.equals, "de")
    one = store.search(q[0], 8, filter=de)
    ok = np.arange(0, n, 3)
    rd, ri = cpu_oracle.flat_search(oracle.COSINE, q[:1], x[ok], 8)
    assert [r.id for r in one] == [f"doc-{ok[i]}" for i in ri[0]]
    assert all(r.metadata["lang"] == "de" for r in one)
    # rows added after a filtered search are found, filtered or not
    store.add([vsk.VectorEntry("late", q[0], {"lang": "de", "rank": 0})])
    assert store.search(q[0], 1, filter=de)[0].id == "late" and store.search(q[0], 1)[0].id == "late"
    store.close()
