// hx_gemm_tc.cuh -- interface of the tcgen05 block-scaled NVFP4 GEMM (hx_gemm_tc.cu).
#pragma once
#include "hx_common.cuh"

#define HX_T128_CELL 18432         // one (128-row tile, 256-column group) cell of A: 16384 B codes + 4 x 512 B scales
#ifndef HX_TC_STAGES
#define HX_TC_STAGES 4
#endif
#ifndef HX_TC_MAX_SK
#define HX_TC_MAX_SK 8             // 64-column steps per ring stage (4 or 8)
#endif
#define HX_TC_RES_CELLS 4          // digit cells of a (K piece, token group) that fit beside the ring of A cells
#define HX_TC_DIGITS 10            // balanced base-9 digits (-4 .. 4, all E2M1 values) of a 30-bit magnitude per activation
#define HX_TC_MAX_TOK 24           // tokens per work unit in digit mode: digit d of token t is column 24 d + t, 240 columns per MMA
#define HX_TC_GROUP_COLS (HX_TC_DIGITS * HX_TC_MAX_TOK)
#define HX_TC_MAX_GROUPS 3         // groups of HX_TC_MAX_TOK tokens per launch
#define HX_TC_NTOK 64              // tokens per launch at most (the token slots of `partial`)
#define HX_TC_DIGIT_UNIT 536870912.0f      // 2^29: the integer a digit vector spells is |x| / scale * 2^29 < 2^30 < (9^10 - 1) / 2

struct HxGemmTC {
    const uint8_t* a;              // T128 cells, [tile][kstep]
    const uint8_t* b;              // B cells, [256-column group of K]: ncols x 128 B swizzled codes + 4 x 512 B scale chunks
    float* y;                      // [rows][ncols]
    int rows, ntiles, ksteps, ncols, stage_ksteps;
    int* err;                      // set when a bounded wait ran out
    // ---- digit mode (the chunk paths): B holds HX_TC_DIGITS balanced base-9 digit columns per token with unit scales, in
    // groups of HX_TC_MAX_TOK tokens (a cell of B = groups x HX_TC_GROUP_COLS rows of 128 bytes, no scale chunks; `ncols`
    // is not used); the epilogue recombines them per token:
    //   out[t * ld_out + row] (+)= col_scale[t] * ts(row) * sum_d 9^(9-d) D[row][group of t][24 d + t % 24]
    int digit_mode;                // 0: raw accumulators to y
    int ntok;                      // digit mode: tokens of the launch (<= HX_TC_NTOK)
    const float* col_scale;        // [ntok] scale of each token's digit integer (a power of two)
    float* out; int ld_out;        // token-major output
    int resid;                     // 1: add to out instead of storing
    float ts[3]; int bound0, bound1;   // per-row tensor scale: rows < bound0 ts[0], < bound1 ts[1], else ts[2]
    int pair64;                    // 1: ts[0] for rows with (row % 128) < 64, ts[1] for the others (gate/up tiles)
    int swiglu;                    // 1: tiles hold 64 gate + 64 up rows; out[t][tile * 64 + r] = silu(gate_r) * up_r, rows = hidden size
    int ksplit;                    // > 1: K pieces per tile (digit mode), merged in K order by the last piece to finish
    float* partial;                // [ntiles][ksplit][HX_TC_NTOK][128] partial sums of the pieces
    unsigned* tickets;             // [ntiles][groups of the launch], zero between launches
    int b_resident;                // digit mode: keep the B cells of a CTA's K piece in shared memory (grid is a multiple of ksplit;
                                   // a piece of at most HX_TC_RES_CELLS cells at 256 columns)
};

int hx_gemm_tc_launch(const HxGemmTC& g, cudaStream_t st);
int hx_gemm_tc_prepare();      // sets the kernel's shared-memory attribute; call once outside stream capture
size_t hx_gemm_tc_smem(int ncols, int stage_ksteps);
