"""Host-side mirror of BIDMat's operator interface for the sparse-dense path.

BIDMat's host code is Scala and no JVM exists where this library is built, so
the interface the Scala classes offer for this path is mirrored here with the
same names, argument meaning and error behaviour, on top of the C ABI in
include/bidmat_b200.h.  PyTorch only supplies device memory and streams.

  SMat    CPU CSC sparse matrix      src/main/scala/BIDMat/SMat.scala, SparseMat.scala
  GMat    dense fp32 device matrix   src/main/scala/BIDMat/GMat.scala
  GSMat   sparse device matrix       src/main/scala/BIDMat/GSMat.scala
  DDS     sampled dense-dense prod.  src/main/scala/BIDMat/MatFunctions.scala:1620-1674

Indices are 0-based everywhere (BIDMat's CPU SMat is 1-based internally and is
shifted on upload, GSMat.scala:626-628; the device layout is 0-based).
"""
import numpy as np
import torch

from . import _lib

_L = _lib.lib


class Mat:
    """The few globals of BIDMat's `object Mat` that this path reads or writes
    (src/main/scala/BIDMat/Mat.scala:670-724)."""
    nflops = 0          # Mat.nflops: 2*k*nnz per product (GMat.scala:1057,1092; GSMat.scala:665)
    debugStructure = False  # validate GSMat structure on the device before each native call


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _check(err, what):
    if err != 0:
        raise RuntimeError("%s %s" % (what, _lib.error_string(err)))


def _stream(device):
    """The stream the mirror's native calls run on: torch's current stream of the
    operand's device, the one the tensors handed in were produced on.  BIDMat's
    launchers use the per-thread default stream and synchronise it
    (jni/include/MatKernel.hpp:15, jni/src/Arith.cu:57); here the stream-ordered entry
    points run on torch's stream, which is then synchronised, so a call is complete on
    return as in BIDMat and is ordered after whatever prepared its operands, also
    inside `with torch.cuda.stream(s)`."""
    return torch.cuda.current_stream(device)


def _settle(device):
    """Before a native call that runs on the per-thread default stream (the synchronous
    entry points without a stream argument): wait for torch's current stream, on which the
    operands were prepared, so the two streams cannot race."""
    torch.cuda.current_stream(device).synchronize()


def _finish(err, what, st):
    _check(err, what)
    st.synchronize()


class SMat:
    """CPU sparse matrix in CSC form: jc (ncols+1), ir (nnz), data (nnz)."""

    def __init__(self, nrows, ncols, jc, ir, data):
        self.nrows = int(nrows)
        self.ncols = int(ncols)
        self.jc = np.ascontiguousarray(jc, dtype=np.int32)
        self.ir = np.ascontiguousarray(ir, dtype=np.int32)
        self.data = np.ascontiguousarray(data, dtype=np.float32)
        if len(self.jc) != self.ncols + 1:
            raise RuntimeError("jc should have ncols+1 entries")

    @property
    def nnz(self):
        return int(self.jc[self.ncols])

    def check(self):
        """SparseMat.check (SparseMat.scala:710-740), 0-based."""
        jc, ir = self.jc, self.ir
        if jc[0] != 0:
            raise RuntimeError("jc(0) should be 0")
        if np.any(np.diff(jc) < 0):
            raise RuntimeError("jc(i) out of order")
        if jc[self.ncols] != len(ir):
            raise RuntimeError("jc(ncols) should be %d" % len(ir))
        if len(ir):
            if ir.min() < 0:
                raise RuntimeError("ir too small")
            if ir.max() >= self.nrows:
                raise RuntimeError("ir out of range")
            ic = np.repeat(np.arange(self.ncols), np.diff(jc))
            if np.any((np.diff(ir) <= 0) & (np.diff(ic) == 0)):
                raise RuntimeError("ir(j) out of order")
        return self

    def full(self):
        """Dense copy as a column-major (ncols, nrows) numpy array."""
        out = np.zeros((self.ncols, self.nrows), dtype=np.float32)
        ic = np.repeat(np.arange(self.ncols), np.diff(self.jc))
        np.add.at(out, (ic, self.ir), self.data)
        return out

    @staticmethod
    def from_scipy(S):
        S = S.tocsc()
        S.sort_indices()
        return SMat(S.shape[0], S.shape[1], S.indptr, S.indices, S.data)


class TransposedPlan:
    """Handle of a prepared transposed product (bidmat_b200_dsmultT_plan_create): the
    row-sorted structure of one GSMat for dense operands of `k` rows.  BIDMat keeps
    derived structure on the matrix object in the same way (pic, GSMat.scala:620-647)."""

    OVERWRITE = 1
    _INFO = ("nnz", "ncols", "m", "k", "elem_bytes", "blocks", "chunks", "split_runs", "slots", "cleared_rows",
             "touched_rows", "bytes", "row_runs")

    def __init__(self, k, S=None, elem_bytes=4, stream=None, m=None, ncols=None, pir=None, pic=None):
        """From a GSMat `S`, or from raw device tensors pir / pic of an m x ncols structure."""
        import ctypes
        if S is not None:
            m, ncols, pir, pic = S.nrows, S.ncols, S.pir, S.pic
        self.handle = ctypes.c_void_p(0)
        self.k, self.ncols, self.nnz, self.m = int(k), int(ncols), int(pir.numel()), int(m)
        self.device = pir.device
        with torch.cuda.device(self.device):
            st = (stream or torch.cuda.current_stream()).cuda_stream
            err = _L.bidmat_b200_dsmultT_plan_create(self.k, self.ncols, self.nnz, self.m, _ptr(pir), _ptr(pic),
                                                     elem_bytes, st, ctypes.byref(self.handle))
        _check(err, "CUMAT.dsmultT plan:")

    def info(self):
        import ctypes
        out = (ctypes.c_longlong * len(self._INFO))()
        _check(_L.bidmat_b200_plan_info(self.handle, out, len(self._INFO)), "plan_info")
        return dict(zip(self._INFO, [int(v) for v in out]))

    def touched_rows(self):
        """Bitmap (int32 words, bit r%32 of word r//32) of the rows of S that hold a nonzero."""
        out = torch.empty((self.m + 31) // 32, dtype=torch.int32, device=self.device)
        with torch.cuda.device(self.device):
            _check(_L.bidmat_b200_plan_touched_rows(self.handle, out.data_ptr(),
                                                    torch.cuda.current_stream().cuda_stream), "plan_touched_rows")
        return out

    def verify(self, S):
        """True when S still has the structure the plan was made from (exact check)."""
        with torch.cuda.device(self.device):
            err = _L.bidmat_b200_plan_verify(self.handle, S.ncols, S.nnz, _ptr(S.pir), _ptr(S.pic),
                                             torch.cuda.current_stream().cuda_stream)
        if err == 1:
            return False
        _check(err, "plan_verify")
        return True

    def run(self, B, S, out, flags=0, stream=None):
        """out (k x m) += B (k x ncols) * S^T with S's current values (stream-ordered)."""
        with torch.cuda.device(self.device):
            st = (stream or torch.cuda.current_stream()).cuda_stream
            err = _L.bidmat_b200_dsmultT_planned(self.handle, B.nrows, S.ncols, S.nnz, B.pdata, _ptr(S.pdata),
                                                 out.pdata, flags, st)
        _check(err, "GMult: CUDA kernel error in CUMAT.dsmultT (planned)")
        return out

    def close(self):
        if self.handle:
            _L.bidmat_b200_plan_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GMat:
    """Dense fp32 matrix on the device, column-major nrows x ncols
    (GMat.scala:20).  Backed by a contiguous torch tensor of shape
    (ncols, nrows), so row i of the tensor is column i of the matrix."""

    def __init__(self, tensor):
        if tensor.dtype != torch.float32 or tensor.dim() != 2 or not tensor.is_contiguous():
            raise RuntimeError("GMat needs a contiguous 2-D float32 tensor (ncols, nrows)")
        if not tensor.is_cuda:
            raise RuntimeError("GMat data must live on a CUDA device (no CPU fallback)")
        self.t = tensor

    @property
    def nrows(self):
        return int(self.t.shape[1])

    @property
    def ncols(self):
        return int(self.t.shape[0])

    @property
    def pdata(self):
        return self.t.data_ptr()

    @staticmethod
    def zeros(nrows, ncols, device=None):
        return GMat(torch.zeros((ncols, nrows), dtype=torch.float32, device=device or "cuda"))

    @staticmethod
    def from_numpy(a, device=None):
        """`a` is (ncols, nrows) C-contiguous = column-major nrows x ncols."""
        return GMat(torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device or "cuda"))

    def to_numpy(self):
        return self.t.cpu().numpy()

    def clear(self):
        self.t.zero_()
        return self

    # ---- A * S ----------------------------------------------------------
    def GSMult(self, a, oldmat=None):
        """GMat.GSMult (GMat.scala:1041-1049): new or recycled zeroed output, then madd."""
        a = GSMat.of(a, self.t.device)
        if self.ncols != a.nrows:
            raise RuntimeError("GSMult dimensions mismatch (%d %d) (%d %d)"
                               % (self.nrows, self.ncols, a.nrows, a.ncols))
        out = _new_or_check(self.nrows, a.ncols, oldmat, self.t.device)
        out.clear()
        return self.madd(a, out)

    def madd(self, a, out):
        """GMat.madd(SMat, FMat) (GMat.scala:1051-1074): out += this * a."""
        a = GSMat.of(a, self.t.device)
        if self.ncols != a.nrows or self.nrows != out.nrows or a.ncols != out.ncols:
            raise RuntimeError("GSMadd dimensions mismatch (%d %d) (%d %d) (%d %d)"
                               % (self.nrows, self.ncols, a.nrows, a.ncols, out.nrows, out.ncols))
        Mat.nflops += 2 * self.nrows * a.nnz
        a._debug_check()
        with torch.cuda.device(self.t.device):
            st = _stream(self.t.device)
            err = _L.bidmat_b200_dsmult_async(self.nrows, a.ncols, a.nnz, self.pdata, _ptr(a.pdata),
                                              _ptr(a.pir), _ptr(a.pic), out.pdata, st.cuda_stream)
            _finish(err, "GMult: CUDA kernel error in CUMAT.dsmult", st)
        return out

    def GSMultDDS(self, b, s, omatC=None, omatP=None):
        """(this * s, DDS(this, b, s)) in one pass over s.  BIDMat computes the two with two
        native calls on the same operands (GMat.GSMult, GMat.scala:1041-1049, and GSMat.DDS,
        GSMat.scala:649-667); both gather the same columns of `this`, so the library offers them
        together.  Same checks, outputs and flop count as the two calls."""
        s = GSMat.of(s, self.t.device)
        if self.ncols != s.nrows:
            raise RuntimeError("GSMult dimensions mismatch (%d %d) (%d %d)" % (self.nrows, self.ncols, s.nrows, s.ncols))
        if self.nrows != b.nrows or s.ncols != b.ncols:
            raise RuntimeError("dimensions mismatch %d,%d  %d,%d  %d,%d"
                               % (self.nrows, self.ncols, b.nrows, b.ncols, s.nrows, s.ncols))
        C = _new_or_check(self.nrows, s.ncols, omatC, self.t.device)
        C.clear()
        P = s._like(omatP)
        P.pir.copy_(s.pir)
        P.pic.copy_(s.pic)
        P._plans = s._plans
        P.pdata.zero_()
        s._debug_check()
        Mat.nflops += 4 * self.nrows * s.nnz
        with torch.cuda.device(self.t.device):
            st = _stream(self.t.device)
            err = _L.bidmat_b200_dsmult_dds_async(self.nrows, s.ncols, s.nnz, self.pdata, b.pdata, _ptr(s.pdata),
                                                  _ptr(s.pir), _ptr(s.pic), C.pdata, _ptr(P.pdata), st.cuda_stream)
            _finish(err, "GMult: CUDA kernel error in CUMAT.dsmult / CUMAT.dds (one pass)", st)
        return C, P

    # ---- B *^ S ---------------------------------------------------------
    def GSMultT(self, a, oldmat=None):
        """GMat.GSMultT (GMat.scala:1076-1084)."""
        a = GSMat.of(a, self.t.device)
        if self.ncols != a.ncols:
            raise RuntimeError("GSMult dimensions mismatch (%d %d) (%d %d)"
                               % (self.nrows, self.ncols, a.ncols, a.nrows))
        out = _new_or_check(self.nrows, a.nrows, oldmat, self.t.device)
        out.clear()
        return self.maddT(a, out)

    def maddT(self, a, out):
        """GMat.maddT (GMat.scala:1086-1096): out += this * a^T."""
        a = GSMat.of(a, self.t.device)
        if self.ncols != a.ncols or self.nrows != out.nrows or a.nrows != out.ncols:
            raise RuntimeError("GSMadd dimensions mismatch (%d %d) (%d %d) (%d %d)"
                               % (self.nrows, self.ncols, a.ncols, a.nrows, out.nrows, out.ncols))
        Mat.nflops += 2 * self.nrows * a.nnz
        a._debug_check()
        with torch.cuda.device(self.t.device):
            st = _stream(self.t.device)
            plan = a.transposed_plan(self.nrows, create=False)
            if plan is not None:
                # prepared structure: no sort, no host round trip (the values may be new)
                err = _L.bidmat_b200_dsmultT_planned(plan.handle, self.nrows, a.ncols, a.nnz, self.pdata,
                                                     _ptr(a.pdata), out.pdata, 0, st.cuda_stream)
            else:
                err = _L.bidmat_b200_dsmultT_async(self.nrows, a.ncols, a.nnz, self.pdata, _ptr(a.pdata),
                                                   _ptr(a.pir), _ptr(a.pic), out.pdata, a.nrows, st.cuda_stream)
            _finish(err, "GMult: CUDA kernel error in CUMAT.dsmultT", st)
        return out

    # ---- tiles (GMat.scala:961-997) --------------------------------------
    def _tile(self, nr, nc, kk, aroff, acoff, b, broff, bcoff, c, croff, ccoff, transpose, name):
        b = GSMat.of(b, self.t.device)
        if min(aroff, acoff, broff, bcoff, croff, ccoff, nr, nc, kk) < 0:
            raise RuntimeError("%s: cant have negative offsets or dimensions" % name)
        brows, bcols = (nc, kk) if transpose else (kk, nc)
        if (aroff + nr > self.nrows or acoff + kk > self.ncols or broff + brows > b.nrows or bcoff + bcols > b.ncols
                or croff + nr > c.nrows or ccoff + nc > c.ncols):
            raise RuntimeError("%s: tile strays outside matrix dimensions" % name)
        Mat.nflops += 2 * nr * b.nnz
        _settle(self.t.device)
        err = _L.bidmat_b200_dsmultTile(nr, nc, kk, b.nnz, self.pdata + 4 * (aroff + acoff * self.nrows), self.nrows,
                                        _ptr(b.pdata), _ptr(b.pir), _ptr(b.pic), broff, bcoff,
                                        c.pdata + 4 * (croff + ccoff * c.nrows), c.nrows, 1 if transpose else 0)
        _check(err, "CUMAT.%s error" % name)
        return c

    def tileMult(self, nr, nc, kk, aroff, acoff, b, broff, bcoff, c, croff, ccoff):
        """c[croff:+nr, ccoff:+nc] += this[aroff:+nr, acoff:+kk] * b[broff:+kk, bcoff:+nc]
        (GMat.tileMult with a GSMat operand, GMat.scala:961-979)."""
        return self._tile(nr, nc, kk, aroff, acoff, b, broff, bcoff, c, croff, ccoff, False, "tileMult")

    def tileMultNT(self, nr, nc, kk, aroff, acoff, b, broff, bcoff, c, croff, ccoff):
        """c[croff:+nr, ccoff:+nc] += this[aroff:+nr, acoff:+kk] * b[broff:+nc, bcoff:+kk]^T
        (GMat.tileMultNT, GMat.scala:981-997)."""
        return self._tile(nr, nc, kk, aroff, acoff, b, broff, bcoff, c, croff, ccoff, True, "tileMultNT")

    # ---- operators (GMat.scala:1684-1686, 1746-1748, 1972-1976) ----------
    def __mul__(self, a):
        """`A * S`."""
        if isinstance(a, (GSMat, SMat)):
            return self.GSMult(a, None)
        return NotImplemented

    def xT(self, a):
        """`B *^ S` (also spelled xT in BIDMat)."""
        return self.GSMultT(a, None)

    def __matmul__(self, s):
        """`B @@ S`: pairs a dense matrix with a sparsity pattern (GMat.scala:1972)."""
        return GDSPair(self, s)

    def Tx(self, pair):
        """`A ^* (B @@ S)` = DDS(A, B, S) (GMat.scala:1973-1976)."""
        if not isinstance(pair, GDSPair):
            raise RuntimeError("^* on a GMat needs a (B @@ S) pair")
        return DDS(self, pair.left, pair.right, None)


class GDSPair:
    """GDSPair (GMat.scala:1978-1990)."""

    def __init__(self, left, right):
        self.left = left
        self.right = right


def _new_or_check(nrows, ncols, oldmat, device):
    """GMat.newOrCheckGMat without the GUID cache: reuse `oldmat` when it has the
    right shape, else allocate."""
    if oldmat is None:
        return GMat(torch.empty((ncols, nrows), dtype=torch.float32, device=device))
    if oldmat.nrows != nrows or oldmat.ncols != ncols:
        raise RuntimeError("dimensions mismatch in output (%d %d) (%d %d)"
                           % (oldmat.nrows, oldmat.ncols, nrows, ncols))
    return oldmat


class GSMat:
    """Sparse matrix on the device in BIDMat's layout (GSMat.scala:14-15):
    pir  int32 row per nonzero, pic int32 column per nonzero (non-decreasing),
    pjc  int32 column pointers (ncols+1), pdata fp32 values."""

    def __init__(self, nrows, ncols, nnz, pir, pic, pjc, pdata):
        self.nrows = int(nrows)
        self.ncols = int(ncols)
        self.nnz = int(nnz)
        self.pir, self.pic, self.pjc, self.pdata = pir, pic, pjc, pdata
        self._plans = {}     # dense height k -> TransposedPlan; shared with matrices that copy this pattern

    @property
    def device(self):
        return self.pjc.device

    def transposed_plan(self, k, create=True):
        """The prepared structure for `B *^ this` with dense operands of k rows.  Created on
        request (prepareT) and kept on the matrix, like the per-nonzero columns BIDMat derives
        once in fromSMat (GSMat.scala:620-647); DDS results share it because they copy this
        matrix's pattern (GSMat.scala:656-661).  Changing pir/pic afterwards makes it stale:
        call dropPlans().  With Mat.debugStructure every use is verified exactly."""
        plan = self._plans.get(int(k))
        if plan is None and create and self.nnz > 0:
            plan = TransposedPlan(k, self)
            self._plans[int(k)] = plan
        if plan is not None and Mat.debugStructure and not plan.verify(self):
            raise RuntimeError("GSMat: the prepared transposed structure does not match pir/pic")
        return plan

    def prepareT(self, k):
        self.transposed_plan(k, create=True)
        return self

    def dropPlans(self):
        for plan in self._plans.values():
            plan.close()
        self._plans = {}

    @staticmethod
    def of(a, device=None):
        if isinstance(a, GSMat):
            return a
        if isinstance(a, SMat):
            return GSMat.fromSMat(a, device)
        raise RuntimeError("expected a GSMat or SMat")

    @staticmethod
    def fromSMat(a, device=None):
        """GSMat.fromSMat (GSMat.scala:620-647): three uploads, then the column
        pointers are expanded into per-nonzero columns on the device (the
        reference calls cuSPARSE csr2coo for that step)."""
        device = device or "cuda"
        jc = torch.from_numpy(a.jc).to(device)
        ir = torch.from_numpy(a.ir).to(device)
        data = torch.from_numpy(a.data).to(device)
        return GSMat.from_csc(a.nrows, a.ncols, jc, ir, data)

    @staticmethod
    def from_csc(nrows, ncols, jc, ir, data):
        """Build from device tensors jc/ir/data, deriving pic on the device."""
        nnz = int(ir.numel())
        ic = torch.empty(nnz, dtype=torch.int32, device=ir.device)
        if nnz:
            with torch.cuda.device(ir.device):
                err = _L.bidmat_b200_expand_jc(ncols, nnz, jc.data_ptr(), ic.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream)
                _check(err, "Cuda error in GSMAT.fromSMat")
        return GSMat(nrows, ncols, nnz, ir, ic, jc, data)

    def toSMat(self):
        """GSMat.toSMat (GSMat.scala:108-127): jc is rebuilt from pic."""
        ic = self.pic.cpu().numpy()
        jc = np.zeros(self.ncols + 1, dtype=np.int32)
        np.cumsum(np.bincount(ic, minlength=self.ncols), out=jc[1:])
        return SMat(self.nrows, self.ncols, jc, self.pir.cpu().numpy(), self.pdata.cpu().numpy())

    @property
    def t(self):
        """GSMat.t (GSMat.scala:218-223), done on the device instead of through a
        CPU SMat: stable sort of the nonzeros by row."""
        out = GSMat(self.ncols, self.nrows, self.nnz, torch.empty_like(self.pir), torch.empty_like(self.pic),
                    torch.empty(self.nrows + 1, dtype=torch.int32, device=self.device), torch.empty_like(self.pdata))
        with torch.cuda.device(self.device):
            err = _L.bidmat_b200_transpose_csc(self.nrows, self.ncols, self.nnz, _ptr(self.pir), _ptr(self.pic),
                                               _ptr(self.pdata), _ptr(out.pir), _ptr(out.pic), _ptr(out.pjc),
                                               _ptr(out.pdata), torch.cuda.current_stream().cuda_stream)
        _check(err, "Cuda error in GSMat.t")
        return out

    def copy(self):
        return GSMat(self.nrows, self.ncols, self.nnz, self.pir.clone(), self.pic.clone(), self.pjc.clone(),
                     self.pdata.clone())

    def sum(self, n=0):
        """GSMat.sum (GSMat.scala:250-261): n == 1 column sums (1 x ncols), n == 2
        row sums (nrows x 1); n == 0 picks 2 for a single-row matrix, else 1."""
        nn = n if n > 0 else (2 if self.nrows == 1 else 1)
        out = GMat.zeros(1 if nn == 1 else self.nrows, self.ncols if nn == 1 else 1, self.device)
        Mat.nflops += self.nnz
        _settle(self.device)
        err = _L.bidmat_b200_spsum(self.nrows, self.ncols, self.nnz, _ptr(self.pir), _ptr(self.pic), _ptr(self.pdata),
                                   out.pdata, nn)
        _check(err, "Cuda error in GSMAT.sum")
        return out

    def GSDop(self, b, op):
        """GSMat.GSDop (GSMat.scala:315-330): combine every stored value with the
        entry of a row vector (1 x ncols), a column vector (nrows x 1) or a scalar."""
        if b.nrows > 1 and b.ncols > 1:
            raise RuntimeError("Sorry only edge operators supported for GSMat op GMat")
        length = b.nrows * b.ncols
        if b.nrows != self.nrows and b.ncols != self.ncols and length > 1:
            raise RuntimeError("GSMat op GMat: dimensions mismatch")
        Mat.nflops += self.nnz
        out = self.copy()
        _settle(self.device)
        if b.ncols > 1:
            err = _L.bidmat_b200_sdoprow(self.nrows, self.ncols, self.nnz, _ptr(out.pdata), _ptr(out.pic), b.pdata,
                                         length, op)
        else:
            err = _L.bidmat_b200_sdopcol(self.nrows, self.ncols, self.nnz, _ptr(out.pdata), _ptr(out.pir), b.pdata,
                                         length, op)
        _check(err, "Cuda error in GSMat op GMat")
        return out

    def __add__(self, b):
        return self.GSDop(b, 0)

    def __sub__(self, b):
        return self.GSDop(b, 1)

    def mul_at(self, b):
        """`S *@ v` (element-wise product with an edge vector)."""
        return self.GSDop(b, 2)

    def __truediv__(self, b):
        return self.GSDop(b, 3)

    def colslice(self, col1, col2):
        """GSMat.colslice (GSMat.scala:77-104): columns [col1, col2) with local,
        zero-based column indices and re-based column pointers."""
        j0 = int(self.pjc[col1])
        j1 = int(self.pjc[col2])
        return GSMat(self.nrows, col2 - col1, j1 - j0, self.pir[j0:j1].clone(),
                     (self.pic[j0:j1] - col1).to(torch.int32), (self.pjc[col1:col2 + 1] - j0).to(torch.int32),
                     self.pdata[j0:j1].clone())

    def _debug_check(self):
        if Mat.debugStructure and self.nnz:
            _settle(self.device)
            err = _L.bidmat_b200_check_structure(self.nrows, self.ncols, self.nnz, _ptr(self.pir), _ptr(self.pic))
            _check(err, "GSMat structure check failed:")

    def _like(self, oldmat):
        if oldmat is not None:
            if oldmat.nrows != self.nrows or oldmat.ncols != self.ncols or oldmat.nnz != self.nnz:
                raise RuntimeError("dimensions mismatch in output GSMat")
            return oldmat
        return GSMat(self.nrows, self.ncols, self.nnz, torch.empty_like(self.pir), torch.empty_like(self.pic),
                     self.pjc.clone(), torch.empty_like(self.pdata))

    @staticmethod
    def DDS(A, B, C, oldmat=None):
        """GSMat.DDS (GSMat.scala:649-667): copy C's row and column indices into
        the output, clear its values, accumulate the sampled products."""
        if A.nrows != B.nrows or C.nrows != A.ncols or C.ncols != B.ncols:
            raise RuntimeError("dimensions mismatch %d,%d  %d,%d  %d,%d"
                               % (A.nrows, A.ncols, B.nrows, B.ncols, C.nrows, C.ncols))
        out = C._like(oldmat)
        out.pir.copy_(C.pir)
        out.pic.copy_(C.pic)
        out._plans = C._plans            # same pattern: the prepared structure carries over
        out.pdata.zero_()
        C._debug_check()
        with torch.cuda.device(C.device):
            st = _stream(C.device)
            err = _L.bidmat_b200_dds_async(A.nrows, C.nnz, A.pdata, B.pdata, _ptr(C.pir), _ptr(C.pic),
                                           _ptr(out.pdata), st.cuda_stream)
            _finish(err, "DDS kernel error", st)
        Mat.nflops += 2 * C.nnz * A.nrows
        return out

    @staticmethod
    def DDS0(A, B, C, oldmat=None):
        """GSMat.DDS0 (GSMat.scala:669-684): the column-pointer driven form."""
        if A.nrows != B.nrows or C.nrows != A.ncols or C.ncols != B.ncols:
            raise RuntimeError("dimensions mismatch")
        out = C._like(oldmat)
        out.pir.copy_(C.pir)
        out.pic.copy_(C.pic)
        out.pdata.zero_()
        with torch.cuda.device(C.device):
            st = _stream(C.device)
            err = _L.bidmat_b200_dds0_async(A.nrows, C.ncols, C.nnz, A.pdata, B.pdata, _ptr(C.pir), _ptr(C.pjc),
                                            _ptr(out.pdata), st.cuda_stream)
            _finish(err, "DDS kernel error", st)
        Mat.nflops += 2 * C.nnz * A.nrows
        return out


def DDS(A, B, C, omat=None):
    """MatFunctions.DDS (MatFunctions.scala:1620-1674) for (GMat, GMat, GSMat):
    P = C's pattern sampled from A^T * B."""
    if isinstance(A, GMat) and isinstance(B, GMat) and isinstance(C, (GSMat, SMat)):
        return GSMat.DDS(A, B, GSMat.of(C, A.t.device), omat)
    raise RuntimeError("DDS: unsupported operand types (device operands only; no CPU fallback)")
