"""BIDMat's .smat / .fmat binary files (src/main/scala/BIDMat/HMat.scala:1232-1264,
1444-1479, 337-365, 876-890): byte layout pinned by a hand-built file, round
trips plain, gzip- and lz4-compressed (lz4-java's block stream, HMat.scala:90-107),
the public known answers of the codec's pieces, error cases."""
import struct

import numpy as np
import pytest

from util import random_csc


def test_smat_byte_layout_matches_the_reference_format(tmp_path):
    from bidmat_b200 import smatio
    # 3 x 2 matrix, column 0 = {(0, 1.5), (2, -2.0)}, column 1 = {(1, 4.0)}
    raw = struct.pack("<4i", 231, 3, 2, 3) + struct.pack("<3i", 0, 2, 3) + struct.pack("<3i", 0, 2, 1) + \
        struct.pack("<3f", 1.5, -2.0, 4.0)
    f = tmp_path / "tiny.smat"
    f.write_bytes(raw)
    m = smatio.loadSMat(str(f))
    assert (m.nrows, m.ncols, m.nnz) == (3, 2, 3)
    assert m.jc.tolist() == [0, 2, 3] and m.ir.tolist() == [0, 2, 1] and m.data.tolist() == [1.5, -2.0, 4.0]
    g = tmp_path / "copy.smat"
    smatio.saveSMat(str(g), m)
    assert g.read_bytes() == raw


@pytest.mark.parametrize("suffix", [".smat", ".smat.gz", ".smat.lz4"])
def test_smat_round_trip(tmp_path, suffix):
    from bidmat_b200 import smatio
    from bidmat_b200.mat import SMat
    rng = np.random.default_rng(4)
    jc, ir, data = random_csc(200, 150, 0.05, rng, empty_cols=(0, 149))
    m = SMat(200, 150, jc, ir, data).check()
    f = str(tmp_path / ("m" + suffix))
    smatio.saveSMat(f, m)
    r = smatio.loadSMat(f).check()
    assert (r.nrows, r.ncols) == (200, 150)
    assert np.array_equal(r.jc, jc) and np.array_equal(r.ir, ir) and np.array_equal(r.data, data)


def test_fmat_round_trip_and_layout(tmp_path):
    from bidmat_b200 import smatio
    a = np.arange(12, dtype=np.float32).reshape(4, 3)       # 3 x 4 column-major
    f = str(tmp_path / "a.fmat.gz")
    smatio.saveFMat(f, a)
    assert np.array_equal(smatio.loadFMat(f), a)
    p = tmp_path / "a.fmat"
    smatio.saveFMat(str(p), a)
    raw = p.read_bytes()
    assert struct.unpack("<4i", raw[:16]) == (130, 3, 4, 0)
    assert struct.unpack("<3f", raw[16:28]) == (0.0, 1.0, 2.0)   # first column


def test_bad_files_are_refused(tmp_path):
    from bidmat_b200 import smatio
    f = tmp_path / "bad.smat"
    f.write_bytes(struct.pack("<4i", 130, 3, 2, 3))
    with pytest.raises(RuntimeError, match="expected type field 231"):
        smatio.loadSMat(str(f))
    f.write_bytes(struct.pack("<4i", 231, 3, 2, 3) + struct.pack("<3i", 0, 2, 3))
    with pytest.raises(RuntimeError, match="truncated"):
        smatio.loadSMat(str(f))
    g = tmp_path / "frame.smat.lz4"
    g.write_bytes(struct.pack("<I", 0x184D2204) + b"\x00" * 32)      # the lz4 tool's frame format is another format
    with pytest.raises(RuntimeError, match="bad magic"):
        smatio.loadSMat(str(g))


def test_xxh32_known_answers():
    """Public test vectors of the 32-bit xxHash."""
    from bidmat_b200.lz4block import xxh32
    assert xxh32(b"", 0) == 0x02CC5D05
    assert xxh32(b"a", 0) == 0x550D7456
    assert xxh32(b"abc", 0) == 0x32D153FF
    assert xxh32(b"Nobody inspects the spammish repetition", 0) == 0xE2293B2F


def test_lz4_blocks_built_by_hand_from_the_format_description():
    from bidmat_b200.lz4block import decompress_block
    # 4 literals, a match of 8 at offset 4 (overlapping: the pattern repeats), 5 closing literals
    blk = bytes([0x44]) + b"abcd" + bytes([4, 0]) + bytes([0x50]) + b"xyzxy"
    assert decompress_block(blk, 17) == b"abcdabcdabcdxyzxy"
    # literal length 20 = 15 + 5 in an extension byte, no match
    lit = bytes(range(65, 85))
    assert decompress_block(bytes([0xF0, 5]) + lit, 20) == lit
    # match length 4 + 15 + 255 + 3 = 277 of a single byte (offset 1), then 5 literals
    blk = bytes([0x1F]) + b"z" + bytes([1, 0, 255, 3]) + bytes([0x50]) + b"12345"
    assert decompress_block(blk, 1 + 277 + 5) == b"z" * 278 + b"12345"
    with pytest.raises(ValueError, match="offset"):
        decompress_block(bytes([0x10]) + b"a" + bytes([9, 0]) + bytes([0x00]), 5)
    with pytest.raises(ValueError, match="header says"):
        decompress_block(bytes([0x10]) + b"a", 2)


def test_lz4_block_stream_layout_round_trip_and_corruption(tmp_path):
    import io
    from bidmat_b200 import lz4block as z
    rng = np.random.default_rng(9)
    data = rng.integers(0, 300, 100000, dtype=np.int32).tobytes() + bytes(rng.integers(0, 256, 5000, dtype=np.uint8))
    f = tmp_path / "s.lz4"
    w = z.LZ4BlockWriter(open(f, "wb"))
    w.write(data[:70001])
    w.write(data[70001:])
    w.close()
    raw = f.read_bytes()
    magic, token, clen, olen, check = struct.unpack_from("<8sBiii", raw, 0)
    assert magic == b"LZ4Block" and token == (0x20 | 6) and olen == 65536 and 0 < clen < olen   # 64 KB blocks: level 6
    assert check == z.xxh32(data[:65536], 0x9747B28C) & 0x0FFFFFFF
    assert raw[-21:] == b"LZ4Block" + bytes([0x10 | 6]) + bytes(12)                            # the end block
    assert z.LZ4BlockReader(open(f, "rb")).read() == data
    r = z.LZ4BlockReader(open(f, "rb"))
    assert r.read(10) + r.read(100000) + r.read() == data                                      # reads across blocks
    # incompressible bytes are stored raw
    noise = bytes(rng.integers(0, 256, 3000, dtype=np.uint8))
    bio = io.BytesIO()
    bio.close = lambda: None
    w = z.LZ4BlockWriter(bio, block_size=1 << 12)
    w.write(noise)
    w.close()
    assert bio.getvalue()[8] == (0x10 | 2) and z.LZ4BlockReader(io.BytesIO(bio.getvalue())).read() == noise
    # a flipped payload byte is caught by the checksum (or by the block decoder)
    bad = bytearray(raw)
    bad[21 + clen // 2] ^= 0x40
    with pytest.raises((RuntimeError, ValueError)):
        z.LZ4BlockReader(io.BytesIO(bytes(bad))).read()
