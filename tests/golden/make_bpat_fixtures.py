"""Writes the small `.bpat` fixtures under tests/golden/ with an independent Python encoder
(struct + zlib.crc32) following the layouts documented in the reference
(crates/fused_gpu/src/io/headers.rs:16-117), and, when the reference tree is present, a summary of
its own example checkpoint data/v2f32_readme.bpat (shapes, size, SHA-256, first values); FERROGRAD_REFERENCE names
the reference tree.

    [FERROGRAD_REFERENCE=<reference tree>] python tests/golden/make_bpat_fixtures.py
"""
import hashlib
import json
import os
import struct
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def tensors():
    r = np.random.Generator(np.random.Philox(77))
    return [r.standard_normal((3, 5)).astype(np.float32), np.arange(7, dtype=np.float32) * 0.5,
            r.standard_normal((2, 3, 4)).astype(np.float32)]


def bf16_bits(a):
    """float32 -> bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype("<u2")


def storage(fmt, t):
    """The bytes of one tensor's data in the file's storage type."""
    if fmt in ("v0", "v1"):
        return t.astype("<f8").tobytes()
    if fmt == "v2f16":
        return t.astype("<f2").tobytes()
    if fmt == "v2bf16":
        return bf16_bits(t).tobytes()
    return t.astype("<f4").tobytes()


def encode(fmt, ts):
    magic = {"v0": b"bpat", "v1": b"BPATv1\0\0", "v1m": b"BPATv1m\0", "v2": b"BPAT\0f32", "v2f16": b"BPAT\0f16",
             "v2bf16": b"BPATbf16"}[fmt]
    wide = fmt in ("v0", "v1")
    crc = fmt in ("v1", "v1m")
    out = bytearray(magic + bytes([len(ts)]))
    for t in ts:
        body = struct.pack("<Q" if wide else "<I", t.ndim)
        body += b"".join(struct.pack("<Q" if wide else "<I", d) for d in t.shape)
        body += storage(fmt, t)
        out += body
        if crc:
            out += struct.pack("<I", zlib.crc32(body) & 0xFFFFFFFF)
    if crc:
        out += struct.pack("<I", zlib.crc32(bytes(out)) & 0xFFFFFFFF)
    return bytes(out)


def main():
    ts = tensors()
    for fmt in ("v0", "v1", "v1m", "v2", "v2f16", "v2bf16"):
        with open(os.path.join(HERE, f"fixture_{fmt}.bpat"), "wb") as f:
            f.write(encode(fmt, ts))
    ref = os.path.join(os.environ.get("FERROGRAD_REFERENCE", ""), "data", "v2f32_readme.bpat")
    if os.environ.get("FERROGRAD_REFERENCE") and os.path.exists(ref):
        d = open(ref, "rb").read()
        off, shapes, heads = 9, [], []
        for _ in range(d[8]):
            nd = struct.unpack_from("<I", d, off)[0]
            off += 4
            shape = struct.unpack_from(f"<{nd}I", d, off)
            off += 4 * nd
            n = int(np.prod(shape))
            heads.append([float(v) for v in np.frombuffer(d, "<f4", 4, off)])
            shapes.append(list(shape))
            off += 4 * n
        json.dump({"file": "data/v2f32_readme.bpat", "bytes": len(d), "sha256": hashlib.sha256(d).hexdigest(),
                   "magic": d[:8].decode("latin1"), "shapes": shapes, "first_values": heads},
                  open(os.path.join(HERE, "bpat_reference_readme_summary.json"), "w"), indent=1)


if __name__ == "__main__":
    main()
