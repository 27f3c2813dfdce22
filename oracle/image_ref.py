"""TEST INFRASTRUCTURE — CPU restatement of the index-image format (numpy), used only by tests to check what
the library writes and to build images it must accept or reject.  Nothing in the product imports this file.

Parity unpinned: the reference has no such image.  Its envelope is followed — "VSTR", version bytes 1,0,0,0,
u64 metadata length, JSON metadata, index data (API/VectorStore.swift:707-727) — but its IVF export keeps only the
centroids (Indexes/IVFIndex.swift:297-326, 612-616), so there are no reference bytes to compare the data
sections with.  What is checked instead: the library's bytes against the arrays that went in, its device
checksums against the two independent restatements below, and search results before and after a round trip.
"""
import json

import numpy as np

GOLDEN = 0x9E3779B97F4A7C15
MASK = (1 << 64) - 1
ALIGN = 64


def _mix_int(z: int) -> int:
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & MASK
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & MASK
    z ^= z >> 31
    return z


def checksum_scalar(data: bytes) -> int:
    """Word-by-word definition with Python integers (small inputs only)."""
    total = 0
    nwords = (len(data) + 7) // 8
    padded = data + b"\0" * (nwords * 8 - len(data))
    for i in range(nwords):
        w = int.from_bytes(padded[8 * i: 8 * i + 8], "little")
        total = (total + _mix_int((w + (i + 1) * GOLDEN) & MASK)) & MASK
    return total


def checksum(data) -> int:
    """Same sum, vectorised: sum over little-endian 64-bit words w_i (last one zero padded) of
    splitmix64_finalise(w_i + (i + 1) * GOLDEN), modulo 2^64."""
    b = np.frombuffer(bytes(data) if not isinstance(data, np.ndarray) else data.tobytes(), np.uint8)
    nwords = (b.size + 7) // 8
    if nwords == 0:
        return 0
    pad = np.zeros(nwords * 8, np.uint8)
    pad[: b.size] = b
    w = pad.view("<u8").astype(np.uint64)
    with np.errstate(over="ignore"):
        z = w + (np.arange(1, nwords + 1, dtype=np.uint64) * np.uint64(GOLDEN))
        z ^= z >> np.uint64(30)
        z *= np.uint64(0xBF58476D1CE4E5B9)
        z ^= z >> np.uint64(27)
        z *= np.uint64(0x94D049BB133111EB)
        z ^= z >> np.uint64(31)
        return int(z.sum(dtype=np.uint64))


def _padded(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


def parse_image(data: bytes):
    """-> (metadata dict, {section name: bytes}).  Raises ValueError on a malformed envelope."""
    if len(data) < 16 or data[:4] != b"VSTR":
        raise ValueError("magic")
    if data[4:8] != bytes([1, 0, 0, 0]):
        raise ValueError("version")
    mlen = int.from_bytes(data[8:16], "little")
    meta = json.loads(data[16: 16 + mlen].decode("ascii"))
    pos = 16 + mlen
    if pos % ALIGN:
        raise ValueError("data does not start on a 64-byte boundary")
    sections = {}
    for s in meta["sections"]:
        n = int(s["bytes"])
        if pos + n > len(data):
            raise ValueError("truncated section " + s["name"])
        sections[s["name"]] = data[pos: pos + n]
        if any(data[pos + n: pos + _padded(n)]):
            raise ValueError("non-zero padding")
        pos += _padded(n)
    if pos != len(data):
        raise ValueError("trailing bytes")
    return meta, sections


def build_image(kind: str, metric: str, dim: int, count: int, sections, id_base=0, has_masks=False, nlist=0,
                pq_segments=0, pq_codebook_size=0) -> bytes:
    """An image as the library writes it, from (name, bytes) pairs."""
    meta = {"format": "vsk-b200-index-image", "format_version": 1, "kind": kind, "metric": metric, "dimensions": dim,
            "count": count, "id_base": id_base, "has_masks": has_masks, "nlist": nlist,
            "pq_segments": pq_segments, "pq_codebook_size": pq_codebook_size,
            "sections": [{"name": n, "bytes": len(b), "checksum": "%016x" % checksum(b)} for n, b in sections]}
    text = json.dumps(meta, separators=(",", ":"))
    while (16 + len(text)) % ALIGN:
        text += " "
    out = bytearray(b"VSTR" + bytes([1, 0, 0, 0]) + len(text).to_bytes(8, "little") + text.encode("ascii"))
    for _, b in sections:
        out += b + b"\0" * (_padded(len(b)) - len(b))
    return bytes(out)
