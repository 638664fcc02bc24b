// The GEMV family with per-group zero points (an extension: the reference's operator has the implicit zero
// point 2^(b-1) and no zero-point argument, csrc/matgptq_gemm.cu:552,631).  Same source, second object.
#define MG_GEMV_ZP 1
#include "gemv.cu"
