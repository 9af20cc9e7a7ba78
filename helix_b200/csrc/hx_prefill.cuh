// hx_prefill.cuh -- kernels of the batched prefill (hx_prefill.cu): a chunk of up to 16 prompt tokens goes through
// every linear as ONE tcgen05 block-scaled GEMM (hx_gemm_tc.cu, digit mode).
#pragma once
#include "hx_common.cuh"

#define HX_PF_TB 16                // tokens per chunk: 16 digit columns each = the 256 columns of one MMA

// Positions are read from device memory (*posp = position of the chunk's first token) so that the launches of a
// chunk can be replayed as one CUDA graph.
// X[t][:] = emb[ids[*posp + t]][:]
void hx_pf_embed(const int* ids, const int* posp, const float* emb, float* X, int n_tok, int DM, cudaStream_t st);

// Digit columns of a chunk of activation vectors, in the B-cell layout of the digit-mode GEMM.
//   src [n_tok][ld] f32; swiglu != 0: the vector is silu(gate)*up read from gate/up tiles of 128 rows
//   (64 gate rows then the 64 matching up rows), K = hidden size;
//   g != null: RMSNorm with gain g and eps first;
//   cells: K rounded up to 256 columns, per 256-column cell ncols x 128 bytes, row 16*t + j = digit j of token t;
//   scale[t] = power of two with x_n = scale * sum_j (digit_j / 2) 4^-j.
void hx_pf_digits(const float* src, int ld, int n_tok, int K, int swiglu, const float* g, float eps,
                  uint8_t* cells, int ncols, float* scale, cudaStream_t st);

// Per token and head of a chunk: RMSNorm (gains qn_g / kn_g, may be null) + rotate_half RoPE at position *posp + t on
// q (in place) and k; k and v are written to the cache rows of their positions.
void hx_pf_qkpost(float* qkv, int ld, int n_tok, const int* posp, int NH, int NKV, int DH, const float* qn_g, const float* kn_g,
                  float eps, const float* cosT, const float* sinT, float* kc, float* vc, int cap, cudaStream_t st);

// Causal attention of a chunk over the cache: query t (position *posp + t) attends to positions 0 .. *posp + t.
// One CTA per (kv head, token); the query heads of a kv head share its K and V rows.
int hx_pf_attn(const float* qkv, int ld, int n_tok, const int* posp, int NH, int NKV, int DH, const float* kc, const float* vc,
               int cap, float scale, float* ctx, int ld_ctx, cudaStream_t st);

// *posp += n
void hx_pf_advance(int* posp, int n, cudaStream_t st);

// First maximum of logits[0..n): index to *tok and hist[pos + 1]; *pos_out = pos + 1.
void hx_pf_argmax(const float* logits, int n, int* tok, int* hist, int* pos_out, int pos, cudaStream_t st);
