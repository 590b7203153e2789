"""Device-side helpers shared by the GPU tests: raw C-ABI calls on torch
tensors (the tests go through the same boundary a BIDMat binding would)."""
import numpy as np
import torch

import oracle
from bidmat_b200 import _lib

L = _lib.lib


def dev(a, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


class DeviceCSC:
    def __init__(self, m, n, jc, ir, data, device):
        self.m, self.n = m, n
        self.jc_h, self.ir_h, self.data_h = (np.asarray(jc, np.int32), np.asarray(ir, np.int32),
                                             np.asarray(data, np.float32))
        self.ic_h = oracle.uncompress_inds(self.jc_h)
        self.nnz = len(self.ir_h)
        self.jc, self.ir, self.ic, self.data = (dev(self.jc_h, device), dev(self.ir_h, device),
                                                dev(self.ic_h, device), dev(self.data_h, device))


def abi_dsmult(A, S, C):
    err = L.bidmat_b200_dsmult(A.shape[1], S.n, S.nnz, A.data_ptr(), S.data.data_ptr(), S.ir.data_ptr(),
                               S.ic.data_ptr(), C.data_ptr())
    assert err == 0, _lib.error_string(err)
    return C


def abi_dsmultT(B, S, G):
    err = L.bidmat_b200_dsmultT(B.shape[1], S.n, S.nnz, B.data_ptr(), S.data.data_ptr(), S.ir.data_ptr(),
                                S.ic.data_ptr(), G.data_ptr())
    assert err == 0, _lib.error_string(err)
    return G


def abi_dds(A, B, S, P):
    err = L.bidmat_b200_dds(A.shape[1], S.nnz, A.data_ptr(), B.data_ptr(), S.ir.data_ptr(), S.ic.data_ptr(),
                            P.data_ptr())
    assert err == 0, _lib.error_string(err)
    return P


def abi_dds0(A, B, S, P):
    err = L.bidmat_b200_dds0(A.shape[1], S.n, A.data_ptr(), B.data_ptr(), S.ir.data_ptr(), S.jc.data_ptr(),
                             P.data_ptr())
    assert err == 0, _lib.error_string(err)
    return P
