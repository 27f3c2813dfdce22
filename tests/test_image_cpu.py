"""Index-image format on the CPU: the two restatements of the section checksum agree with each other and with
hand-computed words, and the envelope follows the reference's "VSTR" layout (API/VectorStore.swift:707-727)."""
import json

import numpy as np
import pytest

from oracle import image_ref as ir


def test_checksum_known_words():
    # one zero word: mix(0 + 1 * GOLDEN)
    assert ir.checksum_scalar(b"\0" * 8) == ir._mix_int(ir.GOLDEN)
    # a short tail is padded with zero bytes to one word
    assert ir.checksum_scalar(b"\x01") == ir._mix_int((1 + ir.GOLDEN) & ir.MASK)
    assert ir.checksum_scalar(b"") == 0
    # position matters: swapping two different words changes the sum
    a, b = (1).to_bytes(8, "little"), (2).to_bytes(8, "little")
    assert ir.checksum_scalar(a + b) != ir.checksum_scalar(b + a)


@pytest.mark.parametrize("n", [0, 1, 7, 8, 9, 63, 64, 65, 1000, 4099])
def test_checksum_vectorised_equals_scalar(n):
    rng = np.random.default_rng(n)
    data = rng.integers(0, 256, n, dtype=np.uint8).tobytes()
    assert ir.checksum(data) == ir.checksum_scalar(data)


def test_envelope_round_trip():
    rows = np.arange(15, dtype=np.float32).tobytes()           # 60 bytes: padded to 64
    masks = np.arange(5, dtype=np.uint64).tobytes()
    img = ir.build_image("flat_f32", "cosine", 3, 5, [("rows", rows), ("masks", masks)], has_masks=True)
    assert img[:4] == b"VSTR" and img[4:8] == bytes([1, 0, 0, 0])
    mlen = int.from_bytes(img[8:16], "little")
    assert (16 + mlen) % 64 == 0
    meta = json.loads(img[16:16 + mlen])
    assert meta["kind"] == "flat_f32" and meta["count"] == 5 and meta["has_masks"] is True
    meta2, sections = ir.parse_image(img)
    assert meta2 == meta and sections["rows"] == rows and sections["masks"] == masks
    assert len(img) == 16 + mlen + 64 + 64
    with pytest.raises(ValueError):
        ir.parse_image(img[:-1])
    with pytest.raises(ValueError):
        ir.parse_image(b"VSTX" + img[4:])
