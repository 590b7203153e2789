/* TEST INFRASTRUCTURE.  Empty stand-in: BIDMat_SPBLAS.c includes <cblas.h>
 * when not built with the Intel compiler but calls nothing from it. */
