"""Shared helpers of the test-suite: small structured inputs and the tolerance
rule.  The rule: |result - oracle| <= rtol * sum|terms| per element, with
rtol = 1e-5 for A*S and DDS and 1e-4 for B*^S (the sum of absolute terms comes
from the fp64 companion of the oracle), plus BIDMat's own absolute 1e-4 check
at the reference's test shapes (src/test/scala/BIDMat/BIDMatSpec.scala:13-16)."""
import numpy as np

RTOL_DSMULT = 1e-5
RTOL_DDS = 1e-5
RTOL_DSMULTT = 1e-4


def random_csc(m, n, density, rng, empty_cols=(), sorted_rows=True, dup_rows=False):
    """Random CSC pattern; returns (jc, ir, data) as numpy arrays."""
    jc = [0]
    ir = []
    for c in range(n):
        if c in empty_cols:
            jc.append(len(ir))
            continue
        cnt = rng.binomial(m, density)
        rows = rng.choice(m, size=cnt, replace=dup_rows)
        rows = np.sort(rows) if sorted_rows else rows
        ir.extend(rows.tolist())
        jc.append(len(ir))
    ir = np.asarray(ir, dtype=np.int32)
    data = rng.uniform(0.05, 1.0, size=len(ir)).astype(np.float32)
    return np.asarray(jc, dtype=np.int32), ir, data


def assert_close_scaled(got, want, scale, rtol, what=""):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    err = np.abs(got - want)
    bound = rtol * np.asarray(scale, dtype=np.float64) + 1e-30
    bad = err > bound
    if np.any(bad):
        i = np.argmax(err / bound)
        raise AssertionError("%s: %d of %d elements outside rtol=%g of sum|terms|; worst ratio %.3g "
                             "(got %r want %r scale %r)" % (what, int(bad.sum()), bad.size, rtol,
                                                            float((err / bound).flat[i]), got.flat[i],
                                                            want.flat[i], np.asarray(scale).flat[i]))


def error_summary(got, want32, want64, scale):
    """The figures reported beside the acceptance rule: the worst error of the result against
    the fp32 CPU loops and against the fp64 oracle, both in units of sum|terms|, the same for the
    CPU loops against fp64, and the largest relative error over the elements that are not
    cancellation leftovers (|cpu| > 1e-3 * sum|terms|)."""
    got = np.asarray(got, dtype=np.float64).ravel()
    want32 = np.asarray(want32, dtype=np.float64).ravel()
    want64 = np.asarray(want64, dtype=np.float64).ravel()
    scale = np.asarray(scale, dtype=np.float64).ravel() + 1e-300
    big = np.abs(want32) > 1e-3 * scale
    return {
        "gpu_vs_cpu32_over_sumabs": float(np.max(np.abs(got - want32) / scale)),
        "gpu_vs_fp64_over_sumabs": float(np.max(np.abs(got - want64) / scale)),
        "cpu32_vs_fp64_over_sumabs": float(np.max(np.abs(want32 - want64) / scale)),
        "max_rel_err_significant": float(np.max(np.abs(got - want32)[big] / np.abs(want32)[big])) if big.any() else 0.0,
        "significant_fraction": float(big.mean()),
    }
