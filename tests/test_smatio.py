"""BIDMat's .smat / .fmat binary files (src/main/scala/BIDMat/HMat.scala:1232-1264,
1444-1479, 337-365, 876-890): byte layout pinned by a hand-built file, round
trips plain and gzip-compressed, error cases."""
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


@pytest.mark.parametrize("suffix", [".smat", ".smat.gz"])
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
    with pytest.raises(RuntimeError, match="lz4"):
        smatio.loadSMat(str(tmp_path / "x.smat.lz4"))
