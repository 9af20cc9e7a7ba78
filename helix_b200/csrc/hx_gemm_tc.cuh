// hx_gemm_tc.cuh -- interface of the tcgen05 block-scaled NVFP4 GEMM (hx_gemm_tc.cu).
#pragma once
#include "hx_common.cuh"

#define HX_T128_CELL 4608          // one (128-row tile, 64-column step) cell of A: 4096 B codes + 512 B scales
#define HX_TC_STAGES 4
#define HX_TC_MAX_SK 8             // 64-column steps per ring stage (upper bound)

struct HxGemmTC {
    const uint8_t* a;              // T128 cells, [tile][kstep]
    const uint8_t* b;              // B cells, [kstep]: 2 x ncols x 16 B codes + 512 B scale chunk
    float* y;                      // [rows][ncols]
    int rows, ntiles, ksteps, ncols, stage_ksteps;
    int* err;                      // set when a bounded wait ran out
};

int hx_gemm_tc_launch(const HxGemmTC& g, cudaStream_t st);
size_t hx_gemm_tc_smem(int ncols, int stage_ksteps);
