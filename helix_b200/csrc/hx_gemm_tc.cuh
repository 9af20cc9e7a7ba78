// hx_gemm_tc.cuh -- interface of the tcgen05 block-scaled NVFP4 GEMM (hx_gemm_tc.cu).
#pragma once
#include "hx_common.cuh"

#define HX_T128_CELL 18432         // one (128-row tile, 256-column group) cell of A: 16384 B codes + 4 x 512 B scales
#define HX_TC_STAGES 4
#define HX_TC_MAX_SK 8             // 64-column steps per ring stage (4 or 8)

struct HxGemmTC {
    const uint8_t* a;              // T128 cells, [tile][kstep]
    const uint8_t* b;              // B cells, [256-column group]: ncols x 128 B swizzled codes + 4 x 512 B scale chunks
    float* y;                      // [rows][ncols]
    int rows, ntiles, ksteps, ncols, stage_ksteps;
    int* err;                      // set when a bounded wait ran out
    int dbg;                       // timing probes (bit 0: copy scale factors once, bit 1: fixed scale columns)
};

int hx_gemm_tc_launch(const HxGemmTC& g, cudaStream_t st);
size_t hx_gemm_tc_smem(int ncols, int stage_ksteps);
