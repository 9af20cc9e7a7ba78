// hx_kernels.cuh -- launch interfaces of the decode-path kernels (hx_decode.cu), shared with the
// model sequencer (hx_model.cu).
#pragma once
#include "hx_common.cuh"

// ---- fused dequant linear over the dense decode layout -----------------------------------------
enum { HX_NORM_NONE = 0, HX_NORM_RMS = 1, HX_NORM_LAYER = 2,
       HX_NORM_ATTN = 3 };   // persistent tensor-core kernel: x is the merge of the attention splits' partial outputs
enum {
    HX_EPI_STORE = 0,     // y[n] = acc (+ bias)
    HX_EPI_RESID = 1,     // y[n] = resid[n] + acc (+ bias)      (y may alias resid)
    HX_EPI_SWIGLU = 2,    // rows are (gate_i, up_i) pairs: y[i] = silu(gate_i) * up_i
    HX_EPI_GELU = 3,      // y[n] = gelu_new(acc + bias)
    HX_EPI_ARGMAX = 4,    // y[n] = acc; the last CTA to finish writes the arg-max row to *next_tok
    HX_EPI_QKV = 5        // fused q|k|v rows: per-head RMSNorm + RoPE on q and k; q -> y, k and v -> the cache row of the position
};

struct HxLinear {
    const uint4* codes;        // [N][Kd/32] pieces of 32 codes (16 B)
    const uint8_t* scales;     // [N][Kd/16] E4M3 bytes
    float ts[3];               // per-tensor scales of up to three row ranges
    int bound0, bound1;        // row < bound0 -> ts[0]; row < bound1 -> ts[1]; else ts[2]
                               // (HX_EPI_SWIGLU: even rows ts[0], odd rows ts[1])
    int N, K, Kd;
    const float* x;            // [K] input
    int norm; const float* norm_g; const float* norm_b; float eps;
    const float* bias;         // [N] or null
    const float* resid;        // HX_EPI_RESID
    float* y;
    int epi;
    // HX_EPI_ARGMAX
    float* part_val; int* part_idx; unsigned* counter; int* next_tok; int* pos_inc; int* hist;
};

int hx_launch_linear(const HxLinear& a, cudaStream_t st, bool pdl);
size_t hx_linear_smem_bytes(int Kd);

// ---- attention -----------------------------------------------------------------------------------
struct HxAttn {
    const float* qkv;          // [QD + 2*KVD] raw projections of the current token
    float* q_rot;              // [QD] normalised + rotated queries
    const float* qn_g; const float* kn_g;    // per-head RMSNorm gains [DH] (null: no QK-norm)
    const float* q_bias;       // unused for the Llama family
    const float* cosT; const float* sinT;    // [cap][DH/2] (null: no RoPE)
    float* kc; float* vc;      // this layer's cache base: [NKV][cap][DH]
    const int* pos;            // device scalar: position of the current token
    int NH, NKV, DH, cap;
    float eps, scale;
    int nsplit;
    float* part_m; float* part_l; float* part_acc;   // split partials: [NH][nsplit], [NH][nsplit][DH]
    unsigned* counters;        // [NKV], zero between launches
    float* ctx;                // [QD] output
};
int hx_launch_qk_prep(const HxAttn& a, cudaStream_t st, bool pdl);
int hx_launch_attn(const HxAttn& a, cudaStream_t st, bool pdl);

// ---- small ops -----------------------------------------------------------------------------------
// x[0..DM) = emb[t] (+ wpe[*pos]) with t = tok[*pos] when index_by_pos, else tok[0]; emb f32 [NV][DM]
int hx_launch_embed(const float* emb, const float* wpe, const int* tok, const int* pos, int index_by_pos, float* x,
                    int DM, cudaStream_t st, bool pdl);
// synthetic N(0, sigma) fill, counter-based
int hx_launch_fill_normal(float* p, size_t n, float sigma, uint64_t seed, cudaStream_t st);
int hx_launch_fill_const(float* p, size_t n, float v, cudaStream_t st);
