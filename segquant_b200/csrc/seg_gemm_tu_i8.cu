// Kernel translation unit: SQ_GEMM_W8A8_I8.  All code is in seg_gemm_kernels.cuh.
#define SQ_TU_KIND SQ_GEMM_W8A8_I8
#define SQ_TU_DUAL false
#include "seg_gemm_kernels.cuh"
