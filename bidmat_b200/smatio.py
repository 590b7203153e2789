"""BIDMat's binary matrix files for the operands of the sparse-dense path, so
that matrices written by BIDMat can be fed to this library and results read
back by BIDMat.

  .smat  int32 {231, nrows, ncols, nnz}, jc[ncols+1], ir[nnz], data[nnz] fp32
         (type 331 = "no rows": ir is absent); indices are 0-based on disk
         whatever BIDMat's in-memory index base is
         (src/main/scala/BIDMat/HMat.scala:1232-1264 load, 1444-1479 save)
  .fmat  int32 {130, nrows, ncols, 0}, then nrows*ncols fp32 column-major
         (HMat.scala:337-365 load, 876-890 save)

Little-endian (HMat.scala:34).  A name ending in .gz is gzip-compressed
(HMat.scala:86-95); a name ending in .lz4 is an lz4-java block stream
(HMat.scala:90-91, 101-107), read and written by the codec in lz4block.py.
"""
import gzip

import numpy as np

from .mat import SMat

_LE_I32 = np.dtype("<i4")
_LE_F32 = np.dtype("<f4")


def _open(fname, mode):
    if fname.endswith(".lz4"):
        from .lz4block import LZ4BlockReader, LZ4BlockWriter
        return LZ4BlockReader(open(fname, "rb")) if "r" in mode else LZ4BlockWriter(open(fname, "wb"))
    return gzip.open(fname, mode) if fname.endswith(".gz") else open(fname, mode)


def _read(f, dtype, count, what):
    raw = f.read(count * dtype.itemsize)
    if len(raw) != count * dtype.itemsize:
        raise RuntimeError("truncated file while reading %s" % what)
    return np.frombuffer(raw, dtype=dtype, count=count)


def loadSMat(fname):
    """HMat.loadSMat: returns an SMat (0-based)."""
    with _open(fname, "rb") as f:
        ftype = int(_read(f, _LE_I32, 1, "type")[0])
        if ftype not in (231, 331):
            raise RuntimeError("loadSMat expected type field 231 or 331 but was %d" % ftype)
        nrows, ncols, nnz = (int(x) for x in _read(f, _LE_I32, 3, "header"))
        jc = _read(f, _LE_I32, ncols + 1, "jc").astype(np.int32)
        if ftype == 231:
            ir = _read(f, _LE_I32, nnz, "ir").astype(np.int32)
        else:
            raise RuntimeError("loadSMat: 'no rows' sparse files (type 331) carry no row indices and cannot be "
                               "used as an operand of the sparse-dense products")
        data = _read(f, _LE_F32, nnz, "data").astype(np.float32)
    if int(jc[ncols]) != nnz:
        raise RuntimeError("loadSMat: jc(ncols) = %d but the header says nnz = %d" % (int(jc[ncols]), nnz))
    return SMat(nrows, ncols, jc, ir, data)


def saveSMat(fname, m):
    """HMat.saveSMat."""
    with _open(fname, "wb") as f:
        f.write(np.asarray([231, m.nrows, m.ncols, m.nnz], dtype=_LE_I32).tobytes())
        for arr, dt in ((m.jc, _LE_I32), (m.ir[:m.nnz], _LE_I32), (m.data[:m.nnz], _LE_F32)):
            f.write(np.ascontiguousarray(arr, dtype=dt).tobytes())


def loadFMat(fname):
    """HMat.loadFMat for 2-D matrices: returns a (ncols, nrows) float32 array,
    i.e. the column-major nrows x ncols matrix in the layout GMat.from_numpy takes."""
    with _open(fname, "rb") as f:
        ftype = int(_read(f, _LE_I32, 1, "type")[0])
        if ftype != 130:
            raise RuntimeError("loadFMat expected type field 130 but was %d" % ftype)
        nrows, ncols, _ = (int(x) for x in _read(f, _LE_I32, 3, "header"))
        data = _read(f, _LE_F32, nrows * ncols, "data").astype(np.float32)
    return data.reshape(ncols, nrows)


def saveFMat(fname, a):
    """HMat.saveFMat; `a` is (ncols, nrows) = column-major nrows x ncols."""
    a = np.ascontiguousarray(a, dtype=_LE_F32)
    ncols, nrows = a.shape
    with _open(fname, "wb") as f:
        f.write(np.asarray([130, nrows, ncols, 0], dtype=_LE_I32).tobytes())
        f.write(a.tobytes())
