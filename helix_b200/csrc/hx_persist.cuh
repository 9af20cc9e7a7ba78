// hx_persist.cuh -- interface of the persistent decode-step kernel (hx_persist.cu).
#pragma once
#include "hx_common.cuh"

// ---- "T16" tile layout of a linear weight ----------------------------------------------------------
// Rows are grouped in m-tiles of 16, columns in k-groups of 128 elements (8 scale blocks).  One
// (m-tile, k-group) cell is 1152 bytes: 16 rows x 64 code bytes, then 16 rows x 8 E4M3 scale bytes.
// Cells of one m-tile are contiguous in k, so any run of k-groups of a tile is one bulk copy.
// Inside a row's 64 code bytes the 16-byte quarter t (0..3) holds, for mma step m (0..7), two bytes:
//   byte0 = codes of (block 2p, element t+8h) | (block 2p+1, element t+8h) << 4
//   byte1 = codes of (block 2p, element t+4+8h) | (block 2p+1, element t+4+8h) << 4      p = m/2, h = m%2
// which is exactly what lane (row, t) of an m16n8k16 A fragment consumes, with the two halves of every
// f16x2 register coming from two neighbouring scale blocks (so one cvt.e4m3x2 scales both).
#define HX_T16_ROWS 16
#define HX_T16_KG 128
#define HX_T16_CELL 1152
#define HX_SLOT_CELLS 16           // k-groups per ring slot = consumer warps
#define HX_RING_SLOT (HX_SLOT_CELLS * HX_T16_CELL)    // 18432 B; also 36 cache rows of 128 floats
#define HX_RING_SLOTS 7

static inline int hx_t16_kgroups(int K) { return (K + HX_T16_KG - 1) / HX_T16_KG; }
static inline int hx_t16_tiles(int N) { return (N + HX_T16_ROWS - 1) / HX_T16_ROWS; }
static inline size_t hx_t16_bytes(int N, int K) { return (size_t)hx_t16_tiles(N) * hx_t16_kgroups(K) * HX_T16_CELL; }

// committed layout -> T16.  Source row r goes to destination row (r / grp) * grp * row_mul + row_off * grp + r % grp
// (grp = 16, row_mul = 2 interleaves gate and up tile by tile; grp = 1 is a plain offset).
void hx_repack_t16(const int32_t* words, const uint8_t* micro, int rows, int K, int Kpad, uint8_t* dst,
                   int dstKG, int grp, int row_mul, int row_off, cudaStream_t st);

enum { HX_PH_LINEAR = 0, HX_PH_ATTN = 1, HX_PH_LINEAR_TC = 2 };

// What one CTA does in a tensor-core linear phase of the dataflow engine, worked out on the host (the kernel carries no
// divisions for it): its run of cells [b0, b1) in storage order (tile-major, K-minor), the K cell of the first one, the
// number of distinct K cells, the tiles the run touches, and its part in the split-K merge.  The CTA that holds the
// first cell of a tile merges it: the first tile of a run is either merged here (first_merger) or handed to its merger
// as piece first_piece; every later tile of the run starts here and is merged here; only the last tile can have pieces
// in the CTAs that follow (last_others of them).
struct alignas(16) HxCtaPlan { int b0, b1, k0, run, t_first, t_last, first_merger, first_piece, last_others, C, pad0, pad1; };
void hx_df_plan(int ntiles, int kcells, int grid, HxCtaPlan* out /* [grid] */, int* max_pieces, int* max_run);

struct alignas(16) HxPhase {
    int type;
    // ---- linear ----
    const uint8_t* w;         // T16 base
    int ntiles;               // m-tiles
    int KG;                   // k-groups per row
    int unit;                 // m-tiles per assignment unit (2 for gate/up pairs)
    int N;                    // valid output rows (SwiGLU: hidden size = rows / 2)
    const float* x;           // input vector, K floats (or the embedding table when tok != null)
    const int* tok;           // when set: input = x + (*tok) * K, and it is copied to x_out
    float* x_out;
    int K;
    int norm;                 // HX_NORM_NONE / HX_NORM_RMS
    const float* g; float eps;
    int epi;                  // HX_EPI_STORE / RESID / SWIGLU / ARGMAX
    float* y;
    float ts[3]; int bound0, bound1;
    // ---- linear on the tensor cores (HX_PH_LINEAR_TC): w = T128 cells, ntiles = 128-row tiles ----
    int ksteps;               // 64-column steps per row (a multiple of 4: whole 256-column cells)
    int pieces;               // most pieces a tile is cut into = stride of its partial sums in tc_partial
    // ---- attention ----
    const float* qkv; const float* qn_g; const float* kn_g; const float* cosT; const float* sinT;
    float* kc; float* vc; float* ctx;
    // ---- tensor parallel (persistent tensor-core kernel) ----
    int tp_partial;           // s + 1: the epilogue writes this rank's partial sums of all rows to slot s of every rank's exchange buffer
    int tp_sum;               // s + 1: the input vector is x + the partial sums of all ranks in slot s; the sum is written to x_out
    int tp_barrier;           // a cross-GPU barrier follows the grid barrier of this phase; tp_epoch counts them within a launch
    int tp_epoch;
    int NH, NKV, DH, cap, nsplit; float scale;   // attention also uses eps (per-head RMSNorm)
    // ---- dataflow engine (hx_decode_df.cu): vectors travel between CTAs as (value, epoch) pairs of 8 bytes; the epoch
    // of the data a phase writes is ep_base + its index + 1, `*_dep` names the phase whose epoch tags an input ----
    const unsigned long long* in_ll;       // input vector (linear: x; attention: q); null: x / tok or the attention partials
    const unsigned long long* in_stat;     // per-tile sums of squares of the input (RMS norm), n_in_stat of them
    int in_dep, n_in_stat;
    unsigned long long* out_ll;            // output vector (residual stream, SwiGLU hidden, q)
    unsigned long long* out_stat;          // per-tile sum of squares of the output (residual epilogue)
    const unsigned long long* res_ll;      // residual rows added by the residual epilogue (null: row *tok of the table x)
    int res_dep, res_ld;                   // res_ld: row length of the table x when tok is set
    unsigned long long* part_ll;           // split-K partial sums of pieces 1.. of every tile: [tile][piece - 1][128]
    const HxCtaPlan* plan;                 // [grid] work split of this phase
    unsigned long long* kv_ll;             // this position's k and v rows [2 * NKV * DH] (qkv epilogue -> attention)
    unsigned long long* pacc_ll;           // attention partial outputs [head][split][DH]
    unsigned long long* pml_ll;            // attention partial (max, sum) lines [head][split][2]
};

struct HxPersist {
    const HxPhase* phases; int nphases;
    const int* pos;                       // device scalar, position of the token being decoded
    unsigned long long* bar;              // grid barrier counter (monotonic over launches)
    unsigned long long bar_base;          // value of the counter when this launch starts
    int* err;                             // set non-zero when a bounded wait ran out
    // attention scratch
    float* part_m; float* part_l; float* part_acc; unsigned* attn_cnt;
    float* part_amax;                     // per (head, split): largest |partial output| / l, bounds the merged output
    // arg-max
    float* am_val; int* am_idx; unsigned* am_cnt; int* next_tok; int* pos_inc; int* hist; float* logits;
    int dig_bytes;                        // shared-memory bytes reserved for the f16 split of x
    int tok_by_pos;                       // the input token is tok[pos] (prompt) instead of tok[0]
    int advance_pos;                      // no head in this launch: CTA 0 advances *pos_inc at the end
    unsigned long long* dbg;              // optional: CTA dbg_cta writes globaltimer stamps per phase
    int dbg_cta;
    unsigned long long* dbg_all;          // optional: every CTA writes the time it finished the work of each phase
    float* tc_partial; unsigned* tc_cnt;  // split-K scratch of the tensor-core linear phases
    int bdig_bytes;                       // shared-memory bytes for the digit columns of x (tensor-core path)
    int tc_ring;                          // ring depth of the tensor-core kernel (3..10 slots)
    // tensor parallel: exchange buffers of all ranks (own entry = local), mapped through CUDA IPC.  Layout in floats:
    // [2 slots][world][tp_dm] partial sums | [world][2] arg-max pairs | [world] barrier flags | [world] arg-max flags | go
    float* tp_peer[8]; int tp_rank, tp_world, tp_dm; unsigned tp_epoch_base; int tp_vocab_off;
    // dataflow engine
    unsigned ep_base;                     // epochs of this launch are ep_base + 1 .. ep_base + nphases + 1
    unsigned wait_limit;                  // polls before a bounded wait gives up
    int inject_stall;                     // test hook: thread 0 of every CTA first waits on a word that nothing sets
    unsigned long long* tp_x[8];          // tensor parallel: exchange buffers of all ranks as (value, epoch) pairs:
                                          // [2 slots][world][tp_dm] partial rows | [world][2] arg-max pairs
    unsigned* done_cnt;                   // ticket of the launches without an lm_head
    int att_nkv, att_nsplit, att_dh;      // attention geometry (the same in every layer): kv heads, most splits, head size
};

int hx_persist_launch(const HxPersist& p, int grid, cudaStream_t st);
int hx_persist_tc_launch(const HxPersist& p, int grid, cudaStream_t st);
int hx_decode_df_launch(const HxPersist& p, int grid, cudaStream_t st);     // dataflow engine (hx_decode_df.cu)
int hx_decode_df_prepare();
int hx_decode_df_ring(int bdig_bytes);
int hx_decode_df_att_bytes(int grp);                                                 // per-device function attributes
size_t hx_persist_tc_smem(int bdig_bytes);            // shared memory besides the ring
int hx_persist_tc_ring(int bdig_bytes);               // ring depth that fits (0: the digit columns do not fit)
// how the tensor-core kernel cuts ntiles x kcells cells over `grid` CTAs: most pieces of one tile, most K cells of one CTA
void hx_tc_split(int ntiles, int kcells, int grid, int* max_pieces, int* max_run);
// committed layout -> T128 cells (hx_persist_tc.cu); destination row = (r/grp)*grp*row_mul + row_off*grp + r%grp
void hx_repack_t128(const int32_t* words, const uint8_t* micro, int rows, int K, int Kpad, uint8_t* dst,
                    int kcells, int grp, int row_mul, int row_off, cudaStream_t st, int k0 = 0);
size_t hx_persist_smem(int dig_bytes);
