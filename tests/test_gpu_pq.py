"""GPU parity of product quantisation (train, encode, decode, distance tables, asymmetric-distance scan) against
the CPU oracle and the golden outputs of the reference's shaders.  Codes, tables and distances are bit-exact."""
import os

import numpy as np
import pytest

from oracle import image_ref as ir

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "metal_shader_vectors.npz"))


@pytest.fixture(scope="module")
def vsk():
    import vectorstorekit_b200 as v
    return v


@pytest.fixture(scope="module")
def dev(vsk):
    return vsk.CUDAAcceleratorStrategy(0).initialize()


def _pq(vsk, dev, dim, m, bits, cb):
    pq = vsk.ProductQuantizer(dev, dim, segments=m, codeSize=bits)
    pq.set_codebooks(cb)
    return pq


def test_golden_reference_shader_codes(vsk, dev):
    pq = _pq(vsk, dev, 24, 4, 8, GOLD["pq_cb"])
    codes = pq.encodeBatch(GOLD["pq_x"])
    assert np.array_equal(codes, GOLD["pq_codes"])
    assert np.array_equal(pq.decodeBatch(codes), GOLD["pq_back"])


# segment lengths with a register path (1, 2, 4, 8, 16, 32) and without (3, 12, 96); 16 and 256 codewords
@pytest.mark.parametrize("shape", [(3000, 8, 8, 8), (3000, 16, 8, 4), (2500, 32, 8, 8), (2000, 64, 8, 8), (1500, 128, 8, 4),
                                   (1000, 128, 4, 8), (2000, 24, 8, 8), (1500, 96, 8, 4), (700, 768, 8, 8), (3000, 8, 2, 8),
                                   (900, 768, 96, 8)])
def test_encode_tables_decode_bit_exact(vsk, dev, cpu_oracle, shape):
    n, d, m, bits = shape
    rng = np.random.default_rng(n + d + m)
    x = rng.standard_normal((n, d)).astype(np.float32)
    cb = rng.standard_normal((m, 1 << bits, d // m)).astype(np.float32)
    cb[:, 5] = cb[:, 2]                                       # exact ties
    x[:10] = np.concatenate([cb[s, 5] for s in range(m)])     # rows on the duplicated codeword
    q = rng.standard_normal((9, d)).astype(np.float32)
    pq = _pq(vsk, dev, d, m, bits, cb)
    codes = pq.encodeBatch(x)
    assert np.array_equal(codes, cpu_oracle.pq_encode(x, cb))
    assert np.all(codes[:10] == 2)
    import torch
    codes_dev = pq.encodeBatch(torch.as_tensor(x, device="cuda"))
    assert np.array_equal(codes_dev.cpu().numpy(), codes)
    assert np.array_equal(pq.precomputeDistanceTables(q), cpu_oracle.pq_tables(q, cb))
    assert np.array_equal(pq.decodeBatch(codes), cpu_oracle.pq_decode(codes, cb))


@pytest.mark.parametrize("shape", [(20_000, 64, 8, 8, 300, 10), (50_000, 128, 16, 8, 200, 100), (5000, 32, 4, 4, 50, 7),
                                   (30_000, 768, 96, 8, 40, 10), (12_345, 48, 48, 8, 33, 50), (300, 16, 2, 8, 5, 300),
                                   (40_000, 96, 32, 8, 1, 10), (8000, 64, 8, 8, 17, 1)])
def test_adc_search_bit_exact(vsk, dev, cpu_oracle, shape):
    n, d, m, bits, nq, k = shape
    rng = np.random.default_rng(n + m)
    ks = 1 << bits
    centres = rng.standard_normal((64, d)).astype(np.float32)
    x = (centres[rng.integers(0, 64, n)] + 0.3 * rng.standard_normal((n, d))).astype(np.float32)
    q = (centres[rng.integers(0, 64, nq)] + 0.3 * rng.standard_normal((nq, d))).astype(np.float32)
    cb = np.stack([x[rng.choice(n, ks, replace=False)][:, s * (d // m):(s + 1) * (d // m)] for s in range(m)])
    pq = _pq(vsk, dev, d, m, bits, cb)
    codes = pq.encodeBatch(x)
    ix = pq.index()
    ix.add(codes[: n // 2])
    ix.add(codes[n // 2:])                                    # incremental add
    assert ix.count == n
    dist, ids = ix.batchSearch(q, k)
    rd, ri = cpu_oracle.pq_search(q, codes, cb, k)
    assert np.array_equal(ids, ri)
    assert np.array_equal(dist, rd)


def test_adc_heavy_ties_and_device_pointers(vsk, dev, cpu_oracle):
    """Quantised distances tie in bulk.  16 distinct code rows among 60 000: thousands of rows tie at every
    distance, and the result must list the tied rows in row order."""
    import torch
    rng = np.random.default_rng(3)
    n, d, m = 60_000, 8, 2
    cb = rng.standard_normal((m, 16, d // m)).astype(np.float32)
    codes = rng.integers(0, 4, (n, m)).astype(np.uint8)
    q = rng.standard_normal((20, d)).astype(np.float32)
    pq = _pq(vsk, dev, d, m, 4, cb)
    ix = pq.index()
    ix.add(torch.as_tensor(codes, device="cuda"))
    dist, ids = ix.batchSearch(torch.as_tensor(q, device="cuda"), 100)
    rd, ri = cpu_oracle.pq_search(q, codes, cb, 100)
    assert np.array_equal(ids.cpu().numpy(), ri) and np.array_equal(dist.cpu().numpy(), rd)


def test_adc_late_block_of_identical_best_rows(vsk, dev, cpu_oracle):
    """The nearest code row appears only in the second half of the database, 30 000 times in a row: a chunk
    appends more keys than a candidate list holds, the overflow is detected and the queries are re-run with
    smaller chunks (fallback_queries), and the answer is still the first 100 of those rows."""
    rng = np.random.default_rng(33)
    n, d, m = 60_000, 8, 2
    cb = rng.standard_normal((m, 16, d // m)).astype(np.float32)
    star = np.array([7, 11], np.uint8)
    codes = rng.integers(0, 6, (n, m)).astype(np.uint8)           # codes 0..5: never the star row
    codes[n // 2:] = star
    target = np.concatenate([cb[0, 7], cb[1, 11]])
    q = (target + 0.01 * rng.standard_normal((12, d))).astype(np.float32)
    pq = _pq(vsk, dev, d, m, 4, cb)
    ix = pq.index()
    ix.add(codes)
    before = dev.stats()["fallback_queries"]
    dist, ids = ix.batchSearch(q, 100)
    rd, ri = cpu_oracle.pq_search(q, codes, cb, 100)
    assert np.array_equal(ids, ri) and np.array_equal(dist, rd)
    assert np.array_equal(ids[0], np.arange(n // 2, n // 2 + 100))
    assert dev.stats()["fallback_queries"] > before


def test_train_against_oracle(vsk, dev, cpu_oracle):
    rng = np.random.default_rng(4)
    n, d, m, bits = 6000, 32, 4, 4
    centres = rng.standard_normal((40, d)).astype(np.float32)
    x = (centres[rng.integers(0, 40, n)] + 0.2 * rng.standard_normal((n, d))).astype(np.float32)
    pq = vsk.ProductQuantizer(dev, d, segments=m, codeSize=bits, trainingIterations=6)
    cb = pq.train(x)                                          # default start: segments of the first 16 rows
    init = np.stack([x[:16, s * 8:(s + 1) * 8] for s in range(m)])
    ref = cpu_oracle.pq_train(x, init, 6)
    assert np.max(np.abs(cb - ref)) < 1e-3
    agree = np.mean(pq.encodeBatch(x) == cpu_oracle.pq_encode(x, ref))
    assert agree > 0.999, agree
    # quantisation error shrinks with training
    err0 = np.mean(np.sum((cpu_oracle.pq_decode(cpu_oracle.pq_encode(x, init), init) - x) ** 2, 1))
    err1 = np.mean(np.sum((pq.decodeBatch(pq.encodeBatch(x)) - x) ** 2, 1))
    assert err1 < 0.8 * err0
    import torch
    cb_dev = vsk.ProductQuantizer(dev, d, segments=m, codeSize=bits, trainingIterations=6).train(
        torch.as_tensor(x, device="cuda"), init)
    assert np.array_equal(cb_dev.cpu().numpy(), cb)


def test_errors(vsk, dev):
    with pytest.raises(vsk.InvalidInput):
        vsk.ProductQuantizer(dev, 30, segments=8)             # invalidSegmentation
    with pytest.raises(vsk.InvalidInput):
        vsk.ProductQuantizer(dev, 32, segments=8, codeSize=3)  # invalidCodeSize
    with pytest.raises(vsk.UnsupportedOperation):
        vsk.ProductQuantizer(dev, 32, segments=8, codeSize=12)
    pq = vsk.ProductQuantizer(dev, 32, segments=8, codeSize=8)
    with pytest.raises(vsk.NotTrained):
        pq.encodeBatch(np.zeros((4, 32), np.float32))
    with pytest.raises(vsk.InsufficientTrainingData):
        pq.train(np.zeros((100, 32), np.float32))             # needs 256 * 8 rows
    with pytest.raises(vsk.DimensionMismatch):
        pq.train(np.zeros((5000, 31), np.float32))
    small = _pq(vsk, dev, 8, 2, 4, np.zeros((2, 16, 4), np.float32))
    ix = small.index()
    with pytest.raises(vsk.InvalidInput, match="outside the codebook"):
        ix.add(np.full((10, 2), 16, np.uint8))
    assert ix.count == 0
    ix.add(np.zeros((10, 2), np.uint8))
    with pytest.raises(vsk.InvalidInput):
        small.decodeBatch(np.full((3, 2), 99, np.uint8))
    import ctypes as C
    q = np.zeros((1, 8), np.float32)
    qm = np.ones(1, np.uint64)
    od, oi = np.empty((1, 1), np.float32), np.empty((1, 1), np.int64)
    st = dev._lib.vsk_search(ix._h, q.ctypes.data, 1, 1, qm.ctypes.data, od.ctypes.data, oi.ctypes.data)
    assert st == vsk.UnsupportedOperation.status
    with pytest.raises(vsk.InvalidBufferSize):                # 300 tables of 256 floats exceed shared memory
        vsk.PQIndex(dev, 600, 300, 256, np.zeros((300, 256, 2), np.float32))


def test_pq_index_image(vsk, dev, cpu_oracle, tmp_path):
    rng = np.random.default_rng(5)
    n, d, m = 4001, 40, 5
    x = rng.standard_normal((n, d)).astype(np.float32)
    cb = rng.standard_normal((m, 256, d // m)).astype(np.float32)
    pq = _pq(vsk, dev, d, m, 8, cb)
    codes = pq.encodeBatch(x)
    ix = pq.index()
    ix.add(codes)
    img = ix.export()
    meta, sections = ir.parse_image(img)
    assert meta["kind"] == "pq" and meta["pq_segments"] == m and meta["pq_codebook_size"] == 256
    assert sections["pq_codebooks"] == cb.tobytes() and sections["pq_codes"] == codes.tobytes()
    for s in meta["sections"]:
        assert int(s["checksum"], 16) == ir.checksum(sections[s["name"]])
    back = vsk.import_index(dev, img)
    assert isinstance(back, vsk.PQIndex) and back.count == n and back.segments == m
    q = rng.standard_normal((12, d)).astype(np.float32)
    d0, i0 = ix.batchSearch(q, 10)
    d1, i1 = back.batchSearch(q, 10)
    assert np.array_equal(i0, i1) and np.array_equal(d0, d1)
    # a code outside a 16-word codebook is refused on load as it is on add
    bad = ir.build_image("pq", "euclidean", 8, 3, [("pq_codebooks", np.zeros((2, 16, 4), np.float32).tobytes()),
                                                    ("pq_codes", np.array([[0, 1], [2, 16], [3, 4]], np.uint8).tobytes())],
                         pq_segments=2, pq_codebook_size=16)
    with pytest.raises(vsk.InvalidInput, match="outside the codebook"):
        vsk.import_index(dev, bad)
    good = ir.build_image("pq", "euclidean", 8, 3, [("pq_codebooks", np.zeros((2, 16, 4), np.float32).tobytes()),
                                                     ("pq_codes", np.array([[0, 1], [2, 15], [3, 4]], np.uint8).tobytes())],
                          pq_segments=2, pq_codebook_size=16)
    assert vsk.import_index(dev, good).count == 3
