"""Seeded synthetic configurations: same seed -> same matrices, structure obeys
BIDMat's CSC invariants (SparseMat.check, SparseMat.scala:710-740), shapes and
distributions follow the benchmark configurations at reduced size."""
import numpy as np
import torch

import oracle
from bidmat_b200 import gen


def _csc_ok(p):
    jc, ir = p.jc.numpy(), p.ir.numpy()
    assert oracle.check_csc(p.m, p.n, ir, jc) == 0
    assert p.data.dtype == torch.float32 and p.ir.dtype == torch.int32 and p.jc.dtype == torch.int32
    assert float(p.data.abs().min()) > 0.0          # no stored zeros
    return jc, ir


def test_config1_fixed_column_length_and_determinism():
    a = gen.config1(0.02, seed=0)
    b = gen.config1(0.02, seed=0)
    c = gen.config1(0.02, seed=1)
    jc, ir = _csc_ok(a)
    assert a.k == 128 and np.all(np.diff(jc) == 100)
    assert torch.equal(a.ir, b.ir) and torch.equal(a.data, b.data) and torch.equal(a.A, b.A)
    assert not torch.equal(a.ir, c.ir)
    assert a.A.shape == (a.m, 128) and a.B.shape == (a.n, 128)
    assert 0.0 < float(a.data.min()) and float(a.data.max()) < 1.0


def test_config2_is_lda_shaped():
    p = gen.config2(0.01, seed=0)
    jc, ir = _csc_ok(p)
    lens = np.diff(jc)
    assert p.k == 256 and lens.min() >= 1
    # Zipf rows: the most popular row is in most columns, the median row index is small
    assert (ir == 0).sum() > 0.5 * p.n
    assert np.median(ir) < 0.05 * p.m
    vals = p.data.numpy()
    assert np.all(vals == np.round(vals)) and vals.min() >= 1.0          # counts 1 + Poisson
    assert 0.0 <= float(p.A.min()) and float(p.A.max()) <= 1.0 / 256


def test_config3_and_config5_shapes():
    p3 = gen.config3(64, 0.01, seed=0)
    jc3, _ = _csc_ok(p3)
    assert p3.k == 64 and p3.m == p3.n and np.all(np.diff(jc3) == 64)
    p5 = gen.config5(0.002, seed=0)
    jc5, ir5 = _csc_ok(p5)
    lens = np.diff(jc5)
    assert p5.k == 128 and p5.n == 2 * p5.m
    assert lens.max() > 10 * np.median(lens)                               # Pareto tail of column lengths
    assert abs(float(p5.A.std()) - 0.1) < 0.01


def test_sprand_like_and_shard_bounds():
    jc, ir, data = gen.sprand_like(30, 20, 0.2, seed=3)
    assert oracle.check_csc(30, 20, ir.numpy(), jc.numpy()) == 0
    dens = len(ir) / 600.0
    assert 0.08 < dens < 0.35
    p = gen.config2(0.01, seed=0)
    for w in (2, 4, 8):
        b = gen.shard_columns(p.jc, w)
        nnz = [int(p.jc[b[i + 1]] - p.jc[b[i]]) for i in range(w)]
        assert sum(nnz) == p.nnz and max(nnz) < 1.1 * p.nnz / w + 25000
