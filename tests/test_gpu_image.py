"""Index images on the GPU: what the library writes equals the arrays that went in (bit for bit), its device
checksums equal the CPU restatement, and an index rebuilt from an image answers searches identically.  Damaged
images are refused."""
import os
import time

import numpy as np
import pytest

from oracle import image_ref as ir

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def vsk():
    import vectorstorekit_b200 as v
    return v


@pytest.fixture(scope="module")
def dev(vsk):
    return vsk.CUDAAcceleratorStrategy(0).initialize()


def _check_sections(img, meta_expect, arrays):
    meta, sections = ir.parse_image(img)
    for k, v in meta_expect.items():
        assert meta[k] == v, (k, meta[k], v)
    assert [s["name"] for s in meta["sections"]] == list(arrays)
    for s in meta["sections"]:
        want = arrays[s["name"]].tobytes()
        assert sections[s["name"]] == want, s["name"]
        assert int(s["checksum"], 16) == ir.checksum(want), s["name"]     # the GPU's sum == the CPU restatement
    return meta


@pytest.mark.parametrize("metric", ["cosine", "euclidean", "manhattan"])
def test_flat_export_import(vsk, dev, metric):
    rng = np.random.default_rng(5)
    n, d = 3001, 67                       # odd sizes: sections end off the 64-byte grid
    x = rng.standard_normal((n, d)).astype(np.float32)
    masks = rng.integers(1, 2 ** 63, n, dtype=np.uint64)
    q = rng.standard_normal((37, d)).astype(np.float32)
    qm = (np.uint64(1) << rng.integers(0, 63, 37).astype(np.uint64))
    ix = vsk.FlatIndex(dev, d, metric)
    ix.add(x, masks=masks)
    ix.set_id_base(1000)
    img = ix.export()
    _check_sections(img, {"kind": "flat_f32", "metric": metric, "dimensions": d, "count": n, "id_base": 1000,
                          "has_masks": True}, {"rows": x, "masks": masks})
    back = vsk.import_index(dev, img)
    assert isinstance(back, vsk.FlatIndex) and back.count == n and back.info()["has_masks"]
    for fm in (None, qm):
        d0, i0 = ix.batchSearch(q, 10, filter_masks=fm)
        d1, i1 = back.batchSearch(q, 10, filter_masks=fm)
        assert np.array_equal(i0, i1) and np.array_equal(d0, d1)
    # an image of the rebuilt index is the same bytes
    assert back.export() == img
    # rows can still be added to a loaded index
    back.add(x[:5], masks=masks[:5])
    assert back.count == n + 5


def test_flat_without_masks_file_round_trip(vsk, dev, tmp_path):
    rng = np.random.default_rng(6)
    x = rng.standard_normal((20_000, 128)).astype(np.float32)
    q = rng.standard_normal((300, 128)).astype(np.float32)
    ix = vsk.FlatIndex(dev, 128, "euclidean")
    ix.add(x)
    path = str(tmp_path / "flat.vstr")
    ix.save(path)
    img = open(path, "rb").read()
    _check_sections(img, {"kind": "flat_f32", "has_masks": False, "count": 20_000}, {"rows": x})
    back = vsk.load_index(dev, path)
    d0, i0 = ix.batchSearch(q, 10)
    d1, i1 = back.batchSearch(q, 10)
    assert np.array_equal(i0, i1) and np.array_equal(d0, d1)


def test_ivf_save_load(vsk, dev, tmp_path):
    rng = np.random.default_rng(7)
    n, d, nlist = 30_000, 48, 64
    centres = rng.standard_normal((nlist, d)).astype(np.float32)
    x = (centres[rng.integers(0, nlist, n)] + 0.2 * rng.standard_normal((n, d))).astype(np.float32)
    q = (centres[rng.integers(0, nlist, 200)] + 0.2 * rng.standard_normal((200, d))).astype(np.float32)
    ivf = vsk.IVFIndex(dev, d, numberOfCentroids=nlist, numberOfProbes=8, maxIterations=5, tolerance=-1.0)
    ivf.train(x)
    ivf.insert(x)
    path = str(tmp_path / "ivf.vstr")
    ivf.save(path)
    meta, sections = ir.parse_image(open(path, "rb").read())
    assert meta["kind"] == "ivf" and meta["nlist"] == nlist and meta["count"] == n
    asg = ivf.assignments()
    assert sections["assignments"] == asg.tobytes()
    off = np.frombuffer(sections["list_offsets"], np.int64)
    assert off[0] == 0 and off[-1] == n and np.array_equal(np.diff(off), np.bincount(asg, minlength=nlist))
    order = np.frombuffer(sections["list_rows"], np.int32)
    assert np.array_equal(order, np.argsort(asg, kind="stable"))          # lists keep insertion order
    assert sections["rows"] == x[order].tobytes()                          # rows are stored list by list
    assert sections["centroids"] == np.asarray(ivf.centroids, np.float32).tobytes()
    for s in meta["sections"]:
        assert int(s["checksum"], 16) == ir.checksum(sections[s["name"]])
    back = vsk.load_index(dev, path)
    assert isinstance(back, vsk.IVFIndex) and back.trained and back.numberOfCentroids == nlist
    assert np.array_equal(back.centroids, np.asarray(ivf.centroids, np.float32))
    assert np.array_equal(back.assignments(), asg)
    back.numberOfProbes = 8
    for strategy in (vsk.SearchStrategy.adaptive, vsk.SearchStrategy.exact):
        d0, i0 = ivf.batchSearch(q, 10, strategy)
        d1, i1 = back.batchSearch(q, 10, strategy)
        assert np.array_equal(i0, i1) and np.array_equal(d0, d1)


@pytest.mark.parametrize("metric", ["dotProduct", "euclidean"])
def test_sq8_export_import(vsk, dev, metric):
    rng = np.random.default_rng(8)
    n, d = 5003, 96
    x = rng.standard_normal((n, d)).astype(np.float32)
    q = rng.standard_normal((64, d)).astype(np.float32)
    sq = vsk.ScalarQuantizer(dev, per_dim=True)
    sq.train(x)
    codes = sq.quantizeBatch(x)
    ix = vsk.QuantizedFlatIndex(dev, d, metric, sq.scale, sq.offset)
    ix.add(codes)
    img = ix.export()
    _check_sections(img, {"kind": "flat_i8", "metric": metric, "count": n},
                    {"sq_scale": np.asarray(sq.scale, np.float32), "sq_offset": np.asarray(sq.offset, np.float32),
                     "codes": np.asarray(codes, np.int8)})
    back = vsk.import_index(dev, img)
    assert isinstance(back, vsk.QuantizedFlatIndex)
    d0, i0 = ix.batchSearch(q, 10)
    d1, i1 = back.batchSearch(q, 10)
    assert np.array_equal(i0, i1) and np.array_equal(d0, d1)


def test_accepts_an_image_built_on_the_cpu(vsk, dev):
    """The format is what the CPU restatement says it is: an image assembled by it loads and searches."""
    rng = np.random.default_rng(9)
    x = rng.standard_normal((500, 16)).astype(np.float32)
    img = ir.build_image("flat_f32", "dotProduct", 16, 500, [("rows", x.tobytes())])
    ix = vsk.import_index(dev, img)
    q = rng.standard_normal((4, 16)).astype(np.float32)
    d1, i1 = ix.batchSearch(q, 3)
    ref = -(q @ x.T)
    assert np.array_equal(i1, np.argsort(ref, axis=1, kind="stable")[:, :3])


def test_damaged_images_are_refused(vsk, dev, tmp_path):
    rng = np.random.default_rng(10)
    x = rng.standard_normal((1000, 32)).astype(np.float32)
    ix = vsk.FlatIndex(dev, 32, "cosine")
    ix.add(x)
    img = bytearray(ix.export())
    meta, _ = ir.parse_image(bytes(img))
    data0 = 16 + int.from_bytes(img[8:16], "little")
    flipped = bytearray(img)
    flipped[data0 + 12345] ^= 0x10                               # one bit inside the rows
    with pytest.raises(vsk.ImportFailed, match="corrupt"):
        vsk.import_index(dev, bytes(flipped))
    with pytest.raises(vsk.ImportFailed):
        vsk.import_index(dev, bytes(img[: len(img) // 2]))       # truncated
    with pytest.raises(vsk.ImportFailed, match="magic"):
        vsk.import_index(dev, b"VSTX" + bytes(img[4:]))
    with pytest.raises(vsk.ImportFailed, match="version"):
        vsk.import_index(dev, bytes(img[:4]) + bytes([2, 0, 0, 0]) + bytes(img[8:]))
    with pytest.raises(vsk.ImportFailed):
        vsk.import_index(dev, bytes(img[:16]) + b"{" * (data0 - 16) + bytes(img[data0:]))   # metadata is not JSON
    wrong = ir.build_image("flat_f32", "cosine", 32, 999, [("rows", x.tobytes())])         # count disagrees with bytes
    with pytest.raises(vsk.ImportFailed, match="size"):
        vsk.import_index(dev, wrong)
    bad_lists = ir.build_image("ivf", "euclidean", 2, 4, [
        ("centroids", np.zeros((2, 2), np.float32).tobytes()), ("list_offsets", np.array([0, 5, 4], np.int64).tobytes()),
        ("list_rows", np.arange(4, dtype=np.int32).tobytes()), ("assignments", np.zeros(4, np.int32).tobytes()),
        ("rows", np.zeros((4, 2), np.float32).tobytes())], nlist=2)
    with pytest.raises(vsk.ImportFailed, match="partition"):
        vsk.import_index(dev, bad_lists)
    with pytest.raises(vsk.ImportFailed):
        vsk.load_index(dev, str(tmp_path / "missing.vstr"))
    with pytest.raises(vsk.ExportFailed):
        ix.save(str(tmp_path / "no_such_dir" / "x.vstr"))
    with pytest.raises(vsk.ExportFailed):
        ix.export(format="json")
    # the context is still usable afterwards
    assert vsk.import_index(dev, bytes(img)).count == 1000


def test_export_needs_room_and_rows(vsk, dev):
    import ctypes as C
    ix = vsk.FlatIndex(dev, 8, "euclidean")
    with pytest.raises(vsk.EmptyInput):
        ix.export()
    ix.add(np.ones((10, 8), np.float32))
    size = C.c_int64()
    dev.check(dev._lib.vsk_index_image_size(ix._h, C.byref(size)))
    assert size.value == len(ix.export())
    small = np.empty(size.value - 1, np.uint8)
    written = C.c_int64()
    st = dev._lib.vsk_index_export(ix._h, small.ctypes.data, small.size, C.byref(written))
    assert st == vsk.ExportFailed.status


def test_image_throughput(vsk, dev, tmp_path):
    """768 MB of rows through save and load; prints the rates (the file lands in the page cache)."""
    import torch
    x = torch.randn((250_000, 768), device="cuda")
    ix = vsk.FlatIndex(dev, 768, "cosine")
    ix.add(x)
    path = str(tmp_path / "big.vstr")
    t0 = time.perf_counter(); ix.save(path); t1 = time.perf_counter()
    back = vsk.load_index(dev, path); t2 = time.perf_counter()
    gb = os.path.getsize(path) / 1e9
    print(f"\nindex image {gb:.2f} GB: save {gb / (t1 - t0):.2f} GB/s, load {gb / (t2 - t1):.2f} GB/s")
    q = torch.randn((64, 768), device="cuda")
    d0, i0 = ix.batchSearch(q, 10)
    d1, i1 = back.batchSearch(q, 10)
    assert torch.equal(i0, i1) and torch.equal(d0, d1)
