/* helix_b200.h -- C ABI of libhelix_b200.so: the NVFP4 quantizer and the transformer
 * decode/prefill loop of Helix's quantized-inference path, implemented for NVIDIA B200 (sm_100a).
 *
 * Conventions (they mirror the reference's C host programs): every function returns an int status,
 * 0 = success, non-zero = one of the HX_ERR_* codes; hx_last_error() gives the message of the last
 * failure on the calling thread.  The library never exits or aborts the process, never falls back
 * to a CPU path, and fails with HX_ERR_CUDA when no usable GPU is present.  Buffers are owned by
 * the caller unless a function says otherwise.  An hx_model may be driven by one thread at a time.
 *
 * "Reference" citations are paths inside the Helix source tree.
 */
#ifndef HELIX_B200_H
#define HELIX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HX_OK            0
#define HX_ERR_ARG       1   /* bad argument (null pointer, size out of range, misaligned) */
#define HX_ERR_CUDA      2   /* a CUDA call failed; hx_last_error() has the CUDA error string */
#define HX_ERR_IO        3   /* file could not be opened / read / written */
#define HX_ERR_FORMAT    4   /* not an HXGW v3 file, or its descriptors do not tile the file */
#define HX_ERR_STATE     5   /* call out of order (e.g. decode past the KV capacity) */
#define HX_ERR_NOMEM     6   /* host or device allocation failed */
#define HX_ERR_COMM      7   /* collective library missing or failed */
#define HX_ERR_TIMEOUT   8   /* a bounded device-side wait ran out */

const char* hx_last_error(void);
const char* hx_version(void);

/* ---------------------------------------------------------------- device memory helpers ------ */
/* Thin wrappers so that callers without a CUDA binding (ctypes, cgo) can own device buffers. */
int hx_device_count(int* n);
int hx_set_device(int dev);
int hx_malloc(void** dptr, size_t bytes);
int hx_free(void* dptr);
int hx_memcpy_h2d(void* dst, const void* src, size_t bytes);
int hx_memcpy_d2h(void* dst, const void* src, size_t bytes);
int hx_memset(void* dptr, int value, size_t bytes);
int hx_sync(void);
/* Pinned host memory for the end-to-end paths. */
int hx_host_alloc(void** hptr, size_t bytes);
int hx_host_free(void* hptr);

/* ---------------------------------------------------------------- codecs ---------------------- */
/* Scalar codecs, host side.  Reference: e2m1_decode / e2m1_encode / e4m3_decode / e4m3_encode,
 * helixc/runtime/gpt2_pack.c:291-343.  The encoders reproduce the reference's tie-breaking
 * (nearest value, the lower code on a tie), which is not IEEE round-to-nearest-even. */
float hx_e2m1_decode(int code);
int   hx_e2m1_encode(float v);
float hx_e4m3_decode(int code);
int   hx_e4m3_encode(float v);

/* ---------------------------------------------------------------- quantizer ------------------- */
/* Kpad = K rounded up to a multiple of 112 (gpt2_pack.c:351). */
int hx_kpad(int K);

/* NVFP4 forward quantizer on the GPU, all pointers are DEVICE pointers.
 * Replaces nvfp4_quantize_tensor, helixc/runtime/gpt2_pack.c:350-373, bit for bit:
 *   w      [rows*K] f32 row-major
 *   words  [rows*(Kpad/7)] int32, seven E2M1 codes per word, low nibble first
 *   micro  [rows*(Kpad/16)] uint8, E4M3 scale code per 16 elements along K     (may be NULL)
 *   sc     [rows*(Kpad/16)] f32, e4m3_decode(micro)*ts                          (may be NULL)
 *   ts     [1] f32 per-tensor scale amax/(6*448), 1.0 for an all-zero tensor    (may be NULL)
 * stream is a cudaStream_t (NULL = default stream); the call is asynchronous.  The first call on a device
 * allocates 256 bytes for the tensor maxima (64 words handed out in turn): calls on different streams may
 * overlap as long as no more than 64 are in flight on one device. */
int hx_quantize_nvfp4(const float* w, int rows, int K, int32_t* words, uint8_t* micro, float* sc,
                      float* ts, void* stream);

/* hx_quantize_nvfp4 for callers that must not allocate device memory (a host that owns all of it in an
 * arena of its own, a service that cannot take the device-wide stall of an allocation).  Same arguments,
 * same bytes out.  No counterpart in the reference: its quantizer runs on the CPU.
 * The per-row maxima live in an array inside the library (1 MiB, found with cudaGetSymbolAddress):
 *   - rows <= hx_noalloc_max_rows() (262144), else HX_ERR_ARG;
 *   - the first call on a device looks the array up (and loads the device code if nothing has yet): make
 *     it during start-up, ahead of any stream capture;
 *   - the array is shared by all callers and keeps the last call's contents; nothing needs clearing, a
 *     call only reads what it wrote;
 *   - calls that overlap in time on one device race on it: keep them on one stream or serialise them. */
int hx_quantize_nvfp4_noalloc(const float* w, int rows, int K, int32_t* words, uint8_t* micro, float* sc,
                              float* ts, void* stream);
int hx_noalloc_max_rows(void);

/* Same contract with HOST buffers: copies w to the device, quantizes, copies the results back and
 * synchronises.  This is the call that stands where the importer calls nvfp4_quantize_tensor
 * (gpt2_pack.c:676). */
int hx_quantize_nvfp4_host(const float* w, int rows, int K, int32_t* words, uint8_t* micro, float* sc,
                           float* ts);

/* Dequantize the packed layout to f32 [rows*Kpad] on the GPU (device pointers).
 * Replaces v3_dequant_packed, helixc/runtime/gpt2_infer.c:109-122 (micro bytes + ts), and
 * nvfp4_host_dequant, gpt2_pack.c:375-387 (pre-collapsed f32 scales; pass micro=NULL, sc!=NULL). */
int hx_dequant_nvfp4(const int32_t* words, const uint8_t* micro, const float* ts, const float* sc,
                     float* out, int rows, int Kpad, void* stream);

/* Micro bytes -> four-per-int32 words with row stride ceil(kblk/4), device pointers.
 * Replaces v3_pack_micro, gpt2_infer.c:2151-2161. */
int hx_pack_micro(const uint8_t* micro, int rows, int kblk, int32_t* dst, void* stream);

/* ---------------------------------------------------------------- fused dequant GEMV ---------- */
/* y[n] = sum_{col<Kpad} x[col] * dequant(W[n,col]) over the committed (7-per-word) layout.
 * Device pointers; x is Kpad long with a zero tail; micro4 is the four-per-word micro layout;
 * ts is a 1-element device array.  Replaces fused_gemv, gpt2_infer.c:2281-2297. */
int hx_gemv_nvfp4(const float* x, const int32_t* words, const int32_t* micro4, const float* ts,
                  float* y, int N, int Kpad, void* stream);

/* Single-matrix round trip (12288 x 4096 in the benchmark) with HOST buffers: quantize W [rows*K], then y = dequant(W) x.
 * x has K elements.  Returns Kpad through kpad_out when non-NULL. */
int hx_roundtrip_host(const float* w, int rows, int K, const float* x, float* y, int* kpad_out);

/* Dense decode layout ("D16"): per row, Kd/2 bytes of codes (two per byte, low nibble first, Kd = K
 * rounded up to 64) followed in a second array by Kd/16 scale bytes.  It carries exactly the
 * information of the committed layout; the commitment hash is always taken over the file bytes. */
int hx_kd(int K);
int hx_repack_d16(const int32_t* words, const uint8_t* micro, int rows, int K, int Kpad,
                  uint8_t* codes, uint8_t* scales, void* stream);
/* y[n] = ts * sum_k x[k] * mag(code[n,k]) * e4m3(scale[n,k/16]); x is Kd long, zero tail. */
int hx_gemv_d16(const float* x, const uint8_t* codes, const uint8_t* scales, const float* ts,
                float* y, int N, int Kd, void* stream);

/* Block-scaled NVFP4 GEMM on the tensor cores (tcgen05.mma kind::mxf4nvf4, TMEM accumulators), device
 * pointers: y[rows][ncols] = sum_k A[row,k]*SFA[row,k/16] * B[n,k]*SFB[n,k/16], f32 accumulation.
 *   a_t128  weights as 18432-byte cells [tile of 128 rows][group of 256 columns]: 128 rows x 128 bytes of codes
 *           (two per byte, low nibble first) in the K-major 128-byte-swizzle operand layout (the 16-byte chunk j
 *           of row r sits at position j ^ (r & 7)), then four 512-byte chunks of E4M3 scales, one per 64 columns
 *           (byte (row%32)*16 + (row/32)*4 + block)
 *   b_cells activations, per group of 256 columns: ncols rows x 128 swizzled bytes, then four scale chunks
 *           indexed by n the same way
 *   stage_ksteps  64-column steps per pipeline stage (4, 8, ... ; 0 = 4)
 * K % 256 == 0, ncols % 8 == 0, 8 <= ncols <= 256.  Replaces the f32 tiled_matmul_abt projections of
 * forward_layer_llama (gpt2_infer.c:1231-1287) for batched prefill.  Synchronous. */
int hx_gemm_nvfp4_tc(const uint8_t* a_t128, int rows, int K, const uint8_t* b_cells, int ncols, float* y,
                     int stage_ksteps, void* stream);
/* Same GEMM launched `reps` times between two CUDA events; *ms_per_launch receives the device time. */
int hx_gemm_nvfp4_tc_bench(const uint8_t* a_t128, int rows, int K, const uint8_t* b_cells, int ncols, float* y,
                           int stage_ksteps, int reps, float* ms_per_launch);

/* ---------------------------------------------------------------- measurement ----------------- */
/* Issue rate of the MMA this library uses (tcgen05.mma kind::mxf4nvf4 block16, M = 128, K = 64, N = ncols, a multiple
 * of 16 up to 256), operands resident in shared memory, one issuing thread per SM; with_scale_copies adds the four
 * scale-factor copies of a weight cell.  clk_per_mma in SM cycles, tflops for all SMs at the current clock.  No
 * counterpart in the reference; it is the tensor-side denominator of the batched GEMM's roofline. */
int hx_probe_mxf4_rate(int ncols, int with_scale_copies, double* clk_per_mma, double* tflops);

/* ---------------------------------------------------------------- importer -------------------- */
/* Safetensors checkpoint directory (config.json + model.safetensors, or model.safetensors.index.json and its
 * shards; F32 or BF16 tensors) -> HXGW v3 NVFP4 file, quantized on the GPU.  Replaces pack_qwen3,
 * helixc/runtime/gpt2_pack.c:587-733: same tensor order, header, descriptors and bytes.  With verify != 0 the
 * written file is read back like the reference does (:692-732): every packed tensor dequantized from the file
 * must stay within 0.15 relative RMS error of its source and every dense tensor must be bit-exact, else
 * HX_ERR_FORMAT.  Uses the current device; synchronous. */
typedef struct {
    int tensors, packed;       /* tensors written, of them NVFP4-packed */
    uint64_t bytes;            /* size of the file */
    double worst_rms;          /* worst rmse / rms_w over the packed tensors (0 without verify) */
    char worst_name[128];
    int f32_exact, verified;
    float ms_pack, ms_verify;
} hx_pack_report;
int hx_pack_qwen3(const char* model_dir, const char* out_path, int verify, hx_pack_report* report);

/* ---------------------------------------------------------------- SHA-256 / receipt ----------- */
/* FIPS 180-4.  Replaces sha256 / sha256_hex / sha256_file, gpt2_infer.c:137-213. */
int hx_sha256(const void* data, size_t n, uint8_t out[32]);
int hx_sha256_hex(const void* data, size_t n, char hex[65]);
int hx_sha256_file(const char* path, char hex[65]);

/* Write a HELIX_V16_RECEIPT and its "<out_path>.logits" side file.  Same fields and formats as
 * run_v3_receipt_from_logits, gpt2_infer.c:2827-2871.  oracle_logits may be NULL (max_abs = -1,
 * argmax_match = -1); tau <= 0 writes the measured max_abs as tier3_tau (calib_tau, :2765-2769). */
int hx_receipt_emit(const char* out_path, const char* weights_path, const int* ids, int n_ids,
                    const float* logits, int n_logits, const float* oracle_logits, double tau,
                    const char* tau_prov);
/* The independent verifier: 0 = RECEIPT_CHECK_PASS, otherwise HX_ERR_FORMAT with the reference's
 * REJECT=<reason> token in hx_last_error().  Replaces run_v3_receipt_check, :2876-2912. */
int hx_receipt_check(const char* receipt, const char* weights_path, const char* logits_path,
                     const char* oracle_path);

/* ---------------------------------------------------------------- model ----------------------- */
typedef struct hx_model hx_model;

typedef struct {
    int32_t arch;        /* 1 = Llama/Qwen3 family (RMSNorm, RoPE, GQA, SwiGLU); 0 = GPT-2 */
    int32_t n_layers, d_model, n_heads, n_kv_heads, head_dim, d_ff, vocab, max_ctx;
    float   rope_theta;
    float   norm_eps;    /* eps the kernels use; the reference computes with 1e-5 whatever the file says */
    int32_t qk_norm;     /* 1 = per-head RMSNorm on q and k before RoPE (Qwen3) */
} hx_config;

#define HX_LOAD_KEEP_COMMITTED  1   /* keep the 7-per-word layout resident beside the decode layout */
#define HX_LOAD_VERIFY_SHA      2   /* hash the file while loading (hx_model_sha256) */
#define HX_LOAD_FILE_EPS        4   /* use the header's rms_norm_eps instead of the reference's 1e-5 */

/* Load an HXGW v3 file (helixc/runtime/gpt2_pack.c:578-733 writes it) into HBM.  Validation follows
 * load_gpt2_weights / peek_weights_header, gpt2_infer.c:581-603, 648-667.  Replaces the per-layer
 * streaming loader (upload_layer_ll, v3_upload_gpu, v3_resident_ptrs, :2163-2276, 2407-2450) with
 * one-time residency.  kv_cap = positions of KV cache to allocate; batch = independent sequences.
 * tp_rank / tp_size select this process's tensor-parallel shard (1-GPU: 0 / 1). */
int hx_model_load(hx_model** out, const char* path, int kv_cap, int batch, int flags,
                  int tp_rank, int tp_size);

/* Build a model of the given shape with seeded synthetic weights generated and quantized on the
 * GPU (linear weights and embedding N(0, 0.02), norm gains 1).  Stands in for checkpoints. */
int hx_model_synth(hx_model** out, const hx_config* cfg, uint64_t seed, int kv_cap, int batch,
                   int flags, int tp_rank, int tp_size);

/* GPT-2 (the GPT-2-124M configuration): LayerNorm, learned positions, fused qkv with biases, gelu_new MLP, tied lm_head.
 * Host f32 tensors, every linear as [out][in] (transpose of the Conv1D storage); the library quantizes all linears
 * and the lm_head copy of wte to NVFP4 with the bit-exact quantizer.  cfg: arch 0, n_kv_heads = n_heads,
 * head_dim = d_model / n_heads, max_ctx = rows of wpe, norm_eps 1e-5.  Decodes with a KV cache through
 * hx_prefill / hx_decode_step / hx_generate_greedy (the reference re-forwards the whole context every token,
 * forward_layer_gpt2, gpt2_infer.c:1131-1193; it has no NVFP4 GPT-2 path). */
typedef struct {
    const float *ln1_g, *ln1_b, *w_qkv /*[3*DM][DM]*/, *b_qkv, *w_proj /*[DM][DM]*/, *b_proj,
                *ln2_g, *ln2_b, *w_fc /*[DFF][DM]*/, *b_fc, *w_proj2 /*[DM][DFF]*/, *b_proj2;
} hx_gpt2_layer;
typedef struct { const float *wte /*[NV][DM]*/, *wpe /*[max_ctx][DM]*/, *lnf_g, *lnf_b; const hx_gpt2_layer* layers; } hx_gpt2_weights;
int hx_model_gpt2(hx_model** out, const hx_config* cfg, const hx_gpt2_weights* w, int kv_cap);

int hx_model_free(hx_model* m);
int hx_model_config(const hx_model* m, hx_config* cfg);
/* Bytes of weights read per decoded token in the decode layout (this rank's shard). */
int hx_model_weight_bytes(const hx_model* m, uint64_t* decode_layout, uint64_t* committed_layout);

/* Size of / copy of the HXGW v3 image of the model (needs HX_LOAD_KEEP_COMMITTED, tp_size 1). */
int hx_model_v3_size(const hx_model* m, uint64_t* bytes);
int hx_model_v3_export(const hx_model* m, void* host_buf, uint64_t bytes);
int hx_model_v3_save(const hx_model* m, const char* path);
/* SHA-256 of the HXGW v3 image (the reference's model_sha256 commitment, gpt2_infer.c:2791). */
int hx_model_sha256(const hx_model* m, char hex[65]);

/* Forget the KV cache (gpt2_infer.c:3354 resets kv_len per request). */
int hx_model_reset(hx_model* m);

/* One decode step of sequence 0 (KV slot 0; the other slots of a model created with batch > 1 are driven by
 * hx_prefill_seq / hx_decode_batch): ids[0] is the token at position `pos` (HOST pointer); on return next_ids[0]
 * (HOST, may be NULL) holds the arg-max token and, when logits != NULL, logits[vocab] (HOST) the f32 logits.
 * Replaces decode_step_llama + the host argmax, gpt2_infer.c:1341-1613, 1735-1739. */
int hx_decode_step(hx_model* m, const int32_t* ids, int pos, int32_t* next_ids, float* logits);

/* Prefill ids[T] (HOST) into KV slot 0 and return the arg-max of the last position in next_ids[0] (and its
 * logits[vocab] when logits != NULL).  Replaces forward_full, :1297-1333. */
int hx_prefill(hx_model* m, const int32_t* ids, int T, int32_t* next_ids, float* logits);

/* hx_prefill for sequence `seq` of a model created with batch > 1: the prompt goes into that sequence's KV slot
 * (chunks through the tcgen05 GEMM), next_id / logits as hx_prefill.  hx_decode_batch(_loop) then advances all slots
 * together.  The reference runs one sequence at a time (run_generate, gpt2_infer.c:3123-3195). */
int hx_prefill_seq(hx_model* m, int seq, const int32_t* ids, int T, int32_t* next_id, float* logits);

/* Greedy generation, tokens never leave the GPU between steps: prefill the prompt, then n_new
 * steps feeding each arg-max back, on sequence 0.  out_ids[n_new] HOST.  Replaces run_generate, :3123-3195.
 * ms_decode (may be NULL) receives the device time of the decode steps alone. */
int hx_generate_greedy(hx_model* m, const int32_t* prompt, int T, int n_new, int32_t* out_ids,
                       float* ms_prefill, float* ms_decode);

/* Prompt-lookup speculative greedy decode (the reference's HX_SPEC path: pld_draft, forward_verify, spec_step,
 * helixc/runtime/gpt2_infer.c:2972-3118, driven from run_generate :3150-3161).  The tokens written to out_ids are
 * the plain greedy sequence of hx_generate_greedy; a step that finds the last k_max..k_min tokens earlier in the
 * sequence verifies the (at most m, at most 15) tokens that followed them in one batched forward and keeps the
 * leading ones the model agrees with, plus the model's own next token.
 * Differences from the reference: no EOS stop (n_new tokens are always produced, as in hx_generate_greedy); a
 * verify row is used only if its best logit leads the runner-up by more than min_margin, because the batched rows
 * and the single-token kernel add their products in different orders -- a closer call is left to the plain step.
 * cfg NULL = {3, 1, 6, 1e-3f}.  Counters steps..forwards are the reference's [specprof] counters. */
#define HX_SPEC_DRAFT_MAX 16
typedef struct { int k_max, k_min, m; float min_margin; } hx_spec_config;
typedef struct {
    long steps;        /* drafter calls */
    long hits;         /* of them, with a draft */
    long drafted;      /* draft tokens proposed */
    long accepted;     /* draft tokens kept */
    long emitted;      /* tokens produced by verify forwards */
    long forwards;     /* verify forwards */
    long single_steps; /* plain decode steps (no draft, or a near tie on the first verify row) */
    long near_ties;    /* verify rows not trusted */
} hx_spec_stats;
int hx_pld_draft(const int32_t* ids, int T, int k_min, int k_max, int m, int32_t* draft);   /* host only; returns the draft length */
int hx_generate_spec(hx_model* m, const int32_t* prompt, int T, int n_new, const hx_spec_config* cfg,
                     int32_t* out_ids, hx_spec_stats* stats, float* ms_prefill, float* ms_decode);

/* Device time accounting of the last hx_generate_greedy / hx_decode_loop call. */
typedef struct {
    float    ms_total;          /* CUDA-event time of the timed region */
    uint32_t kernel_launches;   /* kernels of this library launched inside it */
    float    ms_gemv;           /* when per-kernel profiling is on (hx_model_set_profile) */
    float    ms_attn;
    float    ms_other;
} hx_step_stats;
int hx_model_last_stats(const hx_model* m, hx_step_stats* st);
/* Name of the decode engine in use: "persistent-tcgen05-dataflow" (the default: one cooperative launch per token,
 * linear phases on tcgen05.mma, CTAs hand results to one another as (value, epoch) pairs without grid barriers),
 * "persistent-tcgen05" (the same with grid barriers, HX_SYNC=barrier), "persistent-mma" (mma.sync linears,
 * HX_LINEAR=mma) or "graph" (one CUDA graph of per-op kernels, HX_DECODE=graph and GPT-2; the only engine for which
 * hx_model_set_profile yields per-category times). */
const char* hx_model_engine(const hx_model* m);
/* Test hook of the bounded device-side waits.  Every wait of the decode kernels polls at most wait_limit times
 * (0 restores the default, about ten seconds) and then makes the call return HX_ERR_TIMEOUT with the model still
 * usable.  inject_stall != 0 makes every launch begin with a wait on a word that nothing writes, so that the
 * time-out path can be exercised without faulting or hanging the GPU.  No reference counterpart. */
int hx_model_debug_waits(hx_model* m, unsigned wait_limit, int inject_stall);
int hx_model_set_profile(hx_model* m, int on);

/* Run n_steps decode steps starting at position pos0 with the KV cache as it stands, feeding back
 * the arg-max (first token ids[0], HOST), on sequence 0.  Used by the benchmark: inputs resident, one timed
 * region.  out_ids[n_steps] may be NULL. */
int hx_decode_loop(hx_model* m, const int32_t* ids, int pos0, int n_steps, int32_t* out_ids, float* ms);

/* Batched decode (independent sequences sharing one weight copy, 64 per GPU in the benchmark).  The model is created with
 * batch = number of sequences; sequence i owns KV slot i.  One call decodes one token of each of n_seq sequences:
 * ids[i] at position pos[i] (HOST arrays), arg-max to next_ids[i].  Internally chunks of 64 sequences go through every
 * linear as one tcgen05 GEMM (the weights are streamed once per 64 tokens instead of once per token), attention and
 * the KV append run per sequence.  The reference has no batch dimension (one sequence at a time). */
int hx_decode_batch(hx_model* m, const int32_t* ids, const int32_t* pos, int n_seq, int32_t* next_ids);
/* n_steps such steps from position pos0 for every sequence, feeding back the arg-max on the device; the step is
 * captured once and replayed.  out_ids [n_steps][n_seq] may be NULL; *ms = device time of the loop. */
int hx_decode_batch_loop(hx_model* m, const int32_t* ids, int pos0, int n_seq, int n_steps, int32_t* out_ids, float* ms);

/* Fill the KV cache for positions [0, T) with seeded synthetic values (benchmark set-up for a long
 * context without running a long prefill). */
int hx_model_fill_kv(hx_model* m, int T, uint64_t seed);

/* Read / write n cached positions [pos0, pos0 + n) of one (sequence, layer, kv head): k and v are HOST arrays of
 * n * head_dim floats, K as cached (after QK-norm and RoPE).  The cache layout is the reference's
 * [layer][kv head][position][head_dim], gpt2_infer.c:709-721; the reference keeps it device-private, these two calls
 * exist so that a host can checkpoint / restore a sequence and so that tests can mirror a synthetic cache. */
int hx_model_kv_read(hx_model* m, int seq, int layer, int kv_head, int pos0, int n, float* k, float* v);
int hx_model_kv_write(hx_model* m, int seq, int layer, int kv_head, int pos0, int n, const float* k, const float* v);

/* ---------------------------------------------------------------- tokenizer ------------------- */
/* GPT-2 byte-level BPE from a vocab.json and a merges.txt (helixc/runtime/gpt2_tok.c: load_vocab :251-297,
 * load_merges :355-386, encode_bytes :532-640, encode_bytes_special :500-530, decode_range :660-671).  Host code.
 * with_specials != 0 splits vocabulary entries of the form <...> off the text first (tok_enable_specials, :485-499).
 * encode: *n_ids is the token count of the text; HX_ERR_ARG when it exceeds max_ids.  decode: the bytes the ids stand
 * for, no terminator; *len is their number; HX_ERR_ARG when it exceeds cap; unknown ids contribute nothing. */
typedef struct hx_tokenizer hx_tokenizer;
int hx_tokenizer_load(hx_tokenizer** t, const char* vocab_json, const char* merges_txt);
int hx_tokenizer_free(hx_tokenizer* t);
int hx_tokenizer_vocab_size(const hx_tokenizer* t);
int hx_tokenizer_encode(const hx_tokenizer* t, const char* text, size_t n, int with_specials, int32_t* ids, int max_ids, int* n_ids);
int hx_tokenizer_decode(const hx_tokenizer* t, const int32_t* ids, int n, char* out, size_t cap, size_t* len);

/* ---------------------------------------------------------------- serve worker ---------------- */
/* The reference's seeded sampler (sample_next, helixc/runtime/gpt2_infer.c:1660-1711; PCG32 :1632-1644), host code
 * on host logits, double precision, the reference's order of operations: repetition penalty, frequency / presence
 * penalties, temperature, top-k, soft-max, sort by (-p, id), top-p, min-p, renormalise, one draw.  temperature <= 0
 * is the arg-max (first maximum).  hx_sampler_reset = sample_reset (:1651-1657) with the limits of
 * sample_cfg_from_json (:1729-1732); call hx_sampler_count for every token generated while sampling, as the serve
 * loop does (:3374). */
typedef struct hx_sampler hx_sampler;
typedef struct {
    double temperature, top_p, min_p, rep_penalty, freq_penalty, pres_penalty;   /* neutral: 0, 1, 0, 1, 0, 0 */
    int top_k;                                                                    /* 0 = all */
    uint64_t seed;
} hx_sample_config;
int hx_sampler_create(hx_sampler** s, int vocab);          /* generator unseeded, no counts: the reference's state at start-up */
int hx_sampler_configure(hx_sampler* s, const hx_sample_config* cfg);   /* parameters only: counts and generator untouched */
int hx_sampler_reset(hx_sampler* s, const hx_sample_config* cfg, const int32_t* prompt, int n_prompt);
int hx_sampler_next(hx_sampler* s, const float* logits, int32_t* id);
int hx_sampler_count(hx_sampler* s, int32_t id);
int hx_sampler_free(hx_sampler* s);

/* The request loop of the reference's --serve mode (run_serve, gpt2_infer.c:3284-3400) on model m: one JSON frame
 * per line from in_fd ({"ids":[..],"n_gen":N, sampling fields} or {"cmd":"quit"}), newline-delimited JSON events to
 * out_fd: hello, tokenize, forward_begin + token per generated token, done; error events for a bad frame, a context
 * beyond max_ctx, or a "prompt" frame (this entry has no tokenizer; see hx_serve_text).  The event fields are the reference's (:845-1121);
 * its per-op telemetry and logit lens describe its own launch sequence and are not emitted.  As in the reference, the sampler state is reset at the start of a
 * request only if the previous frame sampled, and with that frame's seed (run_serve resets before it parses the
 * frame's own sampling fields).  Returns when the stream ends or a quit frame arrives.  m must have a
 * KV capacity of at least max_ctx rounded up to 64.  helix_b200/hx_worker wraps this call in a process. */
int hx_serve(hx_model* m, int in_fd, int out_fd, int max_ctx);
/* The same loop with a tokenizer (the reference's --vocab / --merges): "prompt" frames are tokenized (with the control
 * tokens split off when with_specials != 0, the reference's HX_SPECIALS), tokenize.strings, token.string and
 * done.text carry the decoded pieces, "stop":[..] sequences (up to four of up to 31 bytes, matched on the decoded
 * tail, :1043-1094) and eos_id >= 0 (the reference's HX_EOS) end a request early. */
int hx_serve_text(hx_model* m, const hx_tokenizer* tok, int with_specials, int eos_id, int in_fd, int out_fd, int max_ctx);

/* ---------------------------------------------------------------- kernel-entry image ---------- */
/* helix_b200_kernels.fatbin exports, for sm_100a, the entry names and parameter lists of the kernels
 * the reference's worker loads from its emitted PTX (dequant_gemv_warp, dequant_gemv_blockred,
 * nvfp4_dequant_tiled, fused_decode_attn, gpu_rmsnorm_fwd_eps, ... 21 entries), so the file can be
 * given to the reference's launchers in place of that PTX.  These three calls are the launcher
 * side: they do what cuda_launch.c:1058-1088 and gpt2_infer.c:373-375 do (cuModuleLoadData,
 * cuModuleGetFunction, cuLaunchKernel with the caller's grid and block, no dynamic shared memory,
 * the NULL stream, then a synchronize).  args is the usual array of pointers to the arguments. */
int hx_image_open(void** module, const char* path);
int hx_image_launch(void* module, const char* entry, unsigned gx, unsigned gy, unsigned gz,
                    unsigned bx, unsigned by, unsigned bz, void** args);
int hx_image_close(void* module);

/* Kernels launched by this library since it was loaded (all streams). */
unsigned long long hx_launch_count(void);

/* ---------------------------------------------------------------- tensor parallel ------------- */
/* One process per GPU; rank r of a group of tp_size builds its shard with hx_model_load / hx_model_synth
 * (tp_rank, tp_size): q/k/v, gate/up and lm_head rows and o_proj/down_proj columns of its heads, hidden slice and
 * vocabulary slice (column-split qkv/gate/up, row-split o/down as in the reference plan for the 32B shape).
 * The all-reduce after o_proj and down_proj happens INSIDE the persistent decode kernel over NVLink peer memory:
 * every rank stores its partial sums into all ranks' exchange buffers, a flag handshake orders them, and the next
 * linear's prologue adds them in rank order (bit-identical residual stream on every rank).  The arg-max over the
 * vocabulary slices is exchanged the same way.  hx_model_config reports the shard's dimensions; logits returned by
 * hx_decode_step / hx_prefill are the shard's vocabulary slice [vocab / tp_size], token ids are global.
 * Set-up: each rank calls hx_model_tp_handle, the caller gathers the 64-byte handles of all ranks (any channel),
 * each rank calls hx_model_tp_connect with the table [tp_size][64].  All ranks must then issue the same sequence
 * of prefill / decode calls.  Replaces the NCCL all-reduce of the reference plan (no reference code exists). */
int hx_model_tp_handle(hx_model* m, uint8_t handle[64]);
int hx_model_tp_connect(hx_model* m, const uint8_t* handles, int tp_size);

#ifdef __cplusplus
}
#endif
#endif /* HELIX_B200_H */
