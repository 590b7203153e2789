"""CPU checker for the sparse-dense path.  TEST INFRASTRUCTURE ONLY: imported by
tests/, by the smoke check and by the benchmark's CPU-baseline leg, never by
the product package."""
from .cpu_oracle import (  # noqa: F401
    dsmult, dsmultT, dds, dsmult_f64, dsmultT_f64, dds_f64,
    uncompress_inds, compress_inds, check_csc,
    ref_available, ref_smcscm, ref_smcsrm,
    dsmult_d, dsmultT_d, dds_d, ref_dmcscm, ref_dmcsrm,
    use_native, ref_gpu_available, ref_gpu_dsmult, ref_gpu_dsmultT, ref_gpu_dds, ref_gpu_dds0, ref_gpu_spsum,
)
