// Kernel translation unit: SQ_GEMM_W8A8_F8, DualScale.  All code is in seg_gemm_kernels.cuh.
#define SQ_TU_KIND SQ_GEMM_W8A8_F8
#define SQ_TU_DUAL true
#include "seg_gemm_kernels.cuh"
