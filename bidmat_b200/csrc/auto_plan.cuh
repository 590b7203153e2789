// Entry of the kept-plan path of the reference-signature B*^S calls (auto_plan.cu).
#pragma once

namespace bidmat {

// Tries to run C += A * B^T (B = CSC arrays Bdata/Bir/Bic of `elem`-byte values) through a plan
// the library keeps for this structure.  *handled = 1: done, the return value is the call's
// status and the per-thread stream is synchronised.  *handled = 0: the caller takes the
// ordinary path; *m_seen is then the number of rows the index array names, or 0 if unknown.
int auto_plan_dsmultT(int elem, int k, int ncols, int nnz, const void *A, const void *Bdata, const int *Bir,
                      const int *Bic, void *C, int *handled, int *m_seen);

}  // namespace bidmat
