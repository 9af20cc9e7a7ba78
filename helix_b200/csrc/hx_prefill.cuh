// hx_prefill.cuh -- kernels of the batched prefill (hx_prefill.cu): a chunk of up to 16 prompt tokens goes through
// every linear as ONE tcgen05 block-scaled GEMM (hx_gemm_tc.cu, digit mode).
#pragma once
#include "hx_common.cuh"

#define HX_PF_TB 64                // tokens per chunk: three groups of up to 24 tokens x 10 digit columns = the 240 columns of one MMA

// Where the tokens of a chunk sit.  Prefill: consecutive positions of one sequence starting at *posp (device memory, so
// that the launches of a chunk can be replayed as one CUDA graph).  Batched decode: token t is at position pos_arr[t] of
// sequence seq_arr[t], whose KV cache starts seq_stride floats after the previous sequence's.
// With pos_arr == null and seqp != null the whole chunk belongs to sequence *seqp (prefill into one KV slot of a batch).
struct HxPfWhere { const int* posp; const int* pos_arr; const int* seq_arr; size_t seq_stride; const int* seqp; };

// Positions are read from device memory (*posp = position of the chunk's first token) so that the launches of a
// chunk can be replayed as one CUDA graph.
// X[t][:] = emb[ids[*posp + t]][:]
void hx_pf_embed(const int* ids, HxPfWhere wh, const float* emb, float* X, int n_tok, int DM, cudaStream_t st);

// Digit columns of a chunk of activation vectors, in the B-cell layout of the digit-mode GEMM.
//   src [n_tok][ld] f32; swiglu != 0: the vector is silu(gate)*up read from gate/up tiles of 128 rows
//   (64 gate rows then the 64 matching up rows), K = hidden size;
//   g != null: RMSNorm with gain g and eps first;
//   cells: K rounded up to 256 columns; per 256-column cell and group of 24 tokens 240 rows of 128 bytes, row 24 d + t % 24 =
//   digit d of token t (ten balanced base-9 digits, most significant first, as E2M1 codes);
//   scale[t]: x_n = scale[t] * sum_d digit_d 9^(9-d)  (a power of two).
void hx_pf_digits(const float* src, int ld, int n_tok, int K, int swiglu, const float* g, float eps,
                  uint8_t* cells, float* scale, cudaStream_t st);

// Per token and head of a chunk: RMSNorm (gains qn_g / kn_g, may be null) + rotate_half RoPE at position *posp + t on
// q (in place) and k; k and v are written to the cache rows of their positions.
void hx_pf_qkpost(float* qkv, int ld, int n_tok, HxPfWhere wh, int NH, int NKV, int DH, const float* qn_g, const float* kn_g,
                  float eps, const float* cosT, const float* sinT, float* kc, float* vc, int cap, cudaStream_t st);

// Causal attention of a chunk over the cache: query t (position *posp + t) attends to positions 0 .. *posp + t.
// CTAs per (kv head, group of tokens, run of key tiles); the query heads of a kv head share its K and V rows, and so do
// the tokens of a group in a prefill chunk.  `part` (hx_pf_attn_scratch floats) and `tickets` (n_tok * NKV words, zero
// between launches) carry the runs' partial results; *err is raised when a bounded wait ran out.
size_t hx_pf_attn_scratch(int n_tok, int NH, int NKV, int DH);
int hx_pf_attn(const float* qkv, int ld, int n_tok, HxPfWhere wh, int NH, int NKV, int DH, const float* kc, const float* vc,
               int cap, float scale, float* ctx, int ld_ctx, float* part, unsigned* tickets, int* err, cudaStream_t st);

// *posp += n
void hx_pf_advance(int* posp, int n, cudaStream_t st);

// First maximum of logits[0..n): index to *tok and hist[pos + 1]; *pos_out = pos + 1.
void hx_pf_argmax(const float* logits, int n, int* tok, int* hist, int* pos_out, int pos, cudaStream_t st);
// per-row arg-max of logits [rows][ld] (n valid columns) -> next[row]; pos_arr[row] += 1 when given
// Tensor parallel: x[i] += sum over the ranks of part[i] (i < count), the ranks' values exchanged as (value, epoch)
// pairs through peer_areas[w] (rank r writes slot r of every peer; slots are area_pairs pairs apart).
void hx_pf_tp_reduce(const float* part, float* x, unsigned long long* const* peer_areas, int rank, int world, int count, size_t area_pairs,
                     unsigned ep, unsigned wait_limit, int* err, cudaStream_t st);
// Tensor parallel: per row the first maximum over the ranks' vocabulary slices (this rank's slice starts at vocab_off).
void hx_pf_tp_argmax_rows(const float* logits, int n, int ld, int rows, int vocab_off, unsigned long long* const* peer_areas, int rank, int world,
                          size_t area_pairs, unsigned ep, unsigned wait_limit, int* err, int* next, int* pos_arr, cudaStream_t st);
void hx_pf_top2_rows(const float* logits, int n, int ld, int rows, int* next, float* margin, cudaStream_t st);
void hx_pf_argmax_rows(const float* logits, int n, int ld, int rows, int* next, int* pos_arr, cudaStream_t st);
