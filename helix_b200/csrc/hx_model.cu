// hx_model.cu -- weight residency and the decode / prefill sequencer.
//
// Reference: load_gpt2_weights (v3 branch) and peek_weights_header, helixc/runtime/gpt2_infer.c:581-603,
// 648-667 (container validation); v3_upload_gpu / v3_resident_ptrs / upload_layer_ll(_fused),
// :2163-2276, 2407-2450 (the streaming loader this file replaces with one-time HBM residency);
// decode_step_llama :1341-1613, forward_full :1297-1333, run_generate :3123-3195 (sequencing);
// RoPE tables :2040-2057; KV layout :709-721.
//
// Layout in HBM.  Every linear weight lives in the dense decode layout (hx_repack_d16): per row
// Kd/2 code bytes and Kd/16 scale bytes.  Tensors that are consumed together are stored together:
// q|k|v rows back to back, gate and up rows interleaved (row 2i = gate_i, row 2i+1 = up_i).  With
// HX_LOAD_KEEP_COMMITTED the committed 7-per-word layout (words, micro bytes, ts) stays resident as
// well, so that the HXGW v3 image and its SHA-256 can be reproduced from the GPU.
#include "hx_kernels.cuh"
#include "hx_persist.cuh"
#include "hx_gemm_tc.cuh"
#include "hx_prefill.cuh"
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <stdlib.h>
#include <string>
#include <vector>

namespace {

#pragma pack(push, 1)
struct V3Desc { uint32_t packed, rows, K, Kpad; uint64_t data_off, scale_off; };
#pragma pack(pop)
static_assert(sizeof(V3Desc) == 32, "descriptor is 32 bytes");

const uint32_t HXGW_MAGIC = 0x48584757u;
enum { T_INLN = 0, T_Q, T_QN, T_K, T_KN, T_V, T_O, T_POSTLN, T_GATE, T_UP, T_DOWN, T_PER_LAYER };

struct Committed {           // one packed tensor in the 7-per-word layout (device)
    int rows = 0, K = 0, Kpad = 0;
    int32_t* words = nullptr; uint8_t* micro = nullptr; float ts = 1.0f;
};
struct Fused {               // rows of one or more tensors in the dense decode layout (device)
    int N = 0, K = 0, Kd = 0;
    uint8_t* codes = nullptr; uint8_t* scales = nullptr;
    float ts[3] = {1.f, 1.f, 1.f}; int bound0 = 0, bound1 = 0;
    uint8_t* t16 = nullptr; int KG = 0, ntiles = 0;      // tile layout for the persistent kernel (mma.sync path)
    uint8_t* t128 = nullptr; int ksteps = 0, tiles128 = 0;   // T128 cells for the tensor-core path
    size_t bytes() const { return (size_t)N * (Kd / 2 + Kd / 16); }
};
struct Layer {
    float *in_g = nullptr, *post_g = nullptr, *qn_g = nullptr, *kn_g = nullptr;
    // GPT-2 (arch 0): LayerNorm biases and linear biases; in_g / post_g are the LayerNorm gains, gu holds c_fc
    float *ln1_b = nullptr, *ln2_b = nullptr, *b_qkv = nullptr, *b_o = nullptr, *b_fc = nullptr, *b_down = nullptr;
    Fused qkv, o, gu, down;
    Committed c[T_PER_LAYER];      // only packed slots used; kept when HX_LOAD_KEEP_COMMITTED
};

}  // namespace

void hx_repack_rows(const int32_t* words, const uint8_t* micro, int rows, int K, int Kpad, uint8_t* codes,
                    uint8_t* scales, int row_mul, int row_off, cudaStream_t st);

struct hx_model {
    hx_config cfg{};
    int QD = 0, KVD = 0, kv_cap = 0, batch = 1, flags = 0;
    std::vector<Layer> layers;
    float* emb = nullptr;          // [NV][DM] f32
    float* final_g = nullptr;
    float *final_b = nullptr, *wpe = nullptr;      // GPT-2: ln_f bias, learned position embedding [max_ctx][DM]
    Fused head; Committed head_c;
    // decode state
    float *x = nullptr, *qkv = nullptr, *q_rot = nullptr, *ctx = nullptr, *h = nullptr, *logits = nullptr;
    float *kc = nullptr, *vc = nullptr, *cosT = nullptr, *sinT = nullptr;
    float *part_m = nullptr, *part_l = nullptr, *part_acc = nullptr, *part_amax = nullptr; unsigned* attn_cnt = nullptr;
    float* am_val = nullptr; int* am_idx = nullptr; unsigned* am_cnt = nullptr;
    int *d_tok = nullptr, *d_pos = nullptr, *d_hist = nullptr, *d_prompt = nullptr;
    int nsplit = 1;
    cudaStream_t st = nullptr;
    cudaGraphExec_t g_decode = nullptr, g_prefill = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    bool pdl = true;
    bool persist = true;                 // one cooperative kernel per token instead of the launch graph
    bool want_t128 = true, use_tc = true; // linear phases on the tensor cores (tcgen05) inside the persistent kernel
    float* tc_partial = nullptr; unsigned* tc_cnt = nullptr; int bdig_bytes = 0, tc_ring = 0; size_t tc_units_max = 0; int tc_tiles_max = 0;
    HxPhase *ph_decode = nullptr, *ph_prefill = nullptr; int nph_decode = 0, nph_prefill = 0;
    unsigned long long* d_bar = nullptr; unsigned long long bar_count = 0; int* d_err = nullptr;
    int* h_flags = nullptr;        // page-locked: [0] the chunk kernels' error word, [1] the decode kernel's, fetched with a step's results
    int grid_persist = 0, dig_bytes = 0, nsplit_persist = 1;
    unsigned long long* d_dbg = nullptr;
    bool profile = false;
    std::vector<cudaEvent_t> prof_ev; std::vector<int> prof_cat; size_t prof_n = 0;
    hx_step_stats stats{};
    std::vector<void*> allocs;
    uint64_t decode_bytes = 0, committed_bytes = 0;
    int kv_len = 0;
    // tensor parallel: cfg holds THIS RANK's shard dimensions (heads, kv heads, hidden, vocabulary slice); gcfg the model's
    hx_config gcfg{}; int tp_rank = 0, tp_world = 1;
    float* tp_buf = nullptr; size_t tp_buf_floats = 0; float* tp_peer[8] = {nullptr}; bool tp_connected = false; unsigned tp_launches = 0;
    float* x2 = nullptr; int tp_nbar = 0;
    // batched prefill (chunks of HX_PF_TB tokens through the tcgen05 GEMM); buffers are created on first use
    float *pf_x = nullptr, *pf_qkv = nullptr, *pf_ctx = nullptr, *pf_gu = nullptr, *pf_scale = nullptr; uint8_t* pf_cells = nullptr; int* pf_err = nullptr; float* pf_partial = nullptr; unsigned* pf_tickets = nullptr; float* pf_att_part = nullptr; unsigned* pf_att_tickets = nullptr;
    int pf_gu_ld = 0; bool pf_batched = true; size_t pf_partial_n = 0;
    float* pf_part = nullptr; size_t tp_pf_off = 0, tp_pf_area = 0; unsigned tp_pf_ep = 0;      // tensor-parallel chunk exchange
    int *d_bids = nullptr, *d_bpos = nullptr, *d_bseq = nullptr, *d_bnext = nullptr; float* pf_logits = nullptr; int b_cap = 0;   // batched decode
    int* sp_next = nullptr; float* sp_margin = nullptr;                                   // speculative decode: verify rows
    cudaGraphExec_t g_bstep = nullptr; int g_bstep_n = 0;
    int* d_pf_pos = nullptr; cudaGraphExec_t g_pf_chunk = nullptr; bool pf_graph_failed = false; int pf_chunk_launches = 0;
    // dataflow engine (hx_decode_df.cu): vectors that cross CTAs as (value, epoch) pairs
    bool use_df = false;
    unsigned long long *xll[2] = {nullptr, nullptr}, *statll[2] = {nullptr, nullptr}, *qll = nullptr, *kvll = nullptr, *hll = nullptr;
    unsigned long long *pacc_ll = nullptr, *pml_ll = nullptr, *ctxll = nullptr, *part_ll[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    unsigned ep_count = 0, wait_limit = 1u << 24; int inject_stall = 0; unsigned* done_cnt = nullptr;
    std::vector<long long> plan_keys; std::vector<HxCtaPlan*> plan_tabs;
};

namespace {

template <typename T>
int dalloc(hx_model* m, T** p, size_t n) {
    void* q = nullptr;
    cudaError_t e = cudaMalloc(&q, n * sizeof(T) ? n * sizeof(T) : 16);
    if (e != cudaSuccess) return hx_fail(HX_ERR_NOMEM, "cudaMalloc(%zu bytes): %s", n * sizeof(T), cudaGetErrorString(e));
    m->allocs.push_back(q);
    *p = (T*)q;
    return HX_OK;
}

int alloc_fused(hx_model* m, Fused& f, int N, int K) {
    f.N = N; f.K = K; f.Kd = hx_kd(K);
    int rc = HX_OK;
    m->decode_bytes += f.bytes();
    f.KG = hx_t16_kgroups(K); f.ntiles = hx_t16_tiles(N);
    // one resident layout: the one the selected engine reads (D16 for the per-op graph engine, T16 for the mma.sync
    // persistent engine, T128 for the tensor-core engines)
    if (!m->persist) {
        rc = dalloc(m, &f.codes, (size_t)N * (f.Kd / 2)); if (rc) return rc;
        rc = dalloc(m, &f.scales, (size_t)N * (f.Kd / 16)); if (rc) return rc;
    } else if (!m->use_tc) {
        rc = dalloc(m, &f.t16, hx_t16_bytes(N, K)); if (rc) return rc;
        HX_CUDA(cudaMemsetAsync(f.t16, 0, hx_t16_bytes(N, K), m->st));
    }
    f.ksteps = 4 * ((K + 255) / 256); f.tiles128 = (N + 127) / 128;     // whole 256-column cells, 128-row tiles
    if (m->want_t128) {
        const size_t tb = (size_t)f.tiles128 * (f.ksteps / 4) * HX_T128_CELL;
        rc = dalloc(m, &f.t128, tb); if (rc) return rc;
        HX_CUDA(cudaMemsetAsync(f.t128, 0, tb, m->st));
    }
    return HX_OK;
}

// Source of the model's tensors in build order: a mapped file or the synthetic generator.
struct Source {
    // file
    const uint8_t* map = nullptr; size_t maplen = 0; const V3Desc* desc = nullptr;
    // synth
    bool synth = false; uint64_t seed = 0;
    // staging (device)
    float* f32tmp = nullptr; size_t f32cap = 0;
    int32_t* wtmp = nullptr; uint8_t* mtmp = nullptr; float* tstmp = nullptr;
};

// Bring packed tensor `idx` (rows x K) to the device in the committed layout: into `keep` when the
// committed layout stays resident, else into the staging buffers.  Returns its buffers in `c`.
int fetch_packed(hx_model* m, Source& s, int idx, int rows, int K, Committed& c, bool keep) {
    const int Kpad = hx_kpad(K);
    const size_t nw = (size_t)rows * (Kpad / 7), nm = (size_t)rows * (Kpad / 16);
    c.rows = rows; c.K = K; c.Kpad = Kpad;
    if (keep) {
        int rc = dalloc(m, &c.words, nw); if (rc) return rc;
        rc = dalloc(m, &c.micro, nm); if (rc) return rc;
    } else { c.words = s.wtmp; c.micro = s.mtmp; }
    m->committed_bytes += nw * 4 + nm;
    if (s.synth) {
        int rc = hx_launch_fill_normal(s.f32tmp, (size_t)rows * K, 0.02f, s.seed + 0x1000 + (uint64_t)idx, m->st);
        if (rc) return rc;
        rc = hx_quantize_nvfp4(s.f32tmp, rows, K, c.words, c.micro, nullptr, s.tstmp, m->st); if (rc) return rc;
        HX_CUDA(cudaMemcpyAsync(&c.ts, s.tstmp, 4, cudaMemcpyDeviceToHost, m->st));
        HX_CUDA(cudaStreamSynchronize(m->st));
    } else {
        const V3Desc& d = s.desc[idx];
        if (!d.packed || (int)d.rows != rows || (int)d.K != K || (int)d.Kpad != Kpad)
            return hx_fail(HX_ERR_FORMAT, "tensor %d: descriptor (packed=%u rows=%u K=%u Kpad=%u) does not match the model shape (%d x %d)",
                           idx, d.packed, d.rows, d.K, d.Kpad, rows, K);
        HX_CUDA(cudaMemcpyAsync(c.words, s.map + d.data_off, nw * 4, cudaMemcpyHostToDevice, m->st));
        HX_CUDA(cudaMemcpyAsync(c.micro, s.map + d.scale_off, nm, cudaMemcpyHostToDevice, m->st));
        memcpy(&c.ts, s.map + d.scale_off + nm, 4);
        HX_CUDA(cudaStreamSynchronize(m->st));
    }
    return HX_OK;
}

int fetch_dense(hx_model* m, Source& s, int idx, size_t n, float** out, bool is_gain) {
    int rc = dalloc(m, out, n); if (rc) return rc;
    if (s.synth) {
        if (is_gain) return hx_launch_fill_const(*out, n, 1.0f, m->st);
        return hx_launch_fill_normal(*out, n, 0.02f, s.seed + 0x1000 + (uint64_t)idx, m->st);
    }
    const V3Desc& d = s.desc[idx];
    if (d.packed || (size_t)d.rows * d.K != n) return hx_fail(HX_ERR_FORMAT, "tensor %d: expected %zu dense f32", idx, n);
    HX_CUDA(cudaMemcpyAsync(*out, s.map + d.data_off, n * 4, cudaMemcpyHostToDevice, m->st));
    HX_CUDA(cudaStreamSynchronize(m->st));
    return HX_OK;
}

void put_rows(hx_model* m, const Committed& c, Fused& f, int row_mul, int row_off) {
    if (f.codes) hx_repack_rows(c.words, c.micro, c.rows, c.K, c.Kpad, f.codes, f.scales, row_mul, row_off, m->st);
    // tile layout: plain offset, or gate/up interleaved tile by tile (16 rows of gate, 16 rows of up)
    if (f.t16) {
        if (row_mul == 1) hx_repack_t16(c.words, c.micro, c.rows, c.K, c.Kpad, f.t16, f.KG, 1, 1, row_off, m->st);
        else hx_repack_t16(c.words, c.micro, c.rows, c.K, c.Kpad, f.t16, f.KG, 16, row_mul, row_off, m->st);
    }
    if (f.t128) {   // gate/up: 64 gate rows then the matching 64 up rows per 128-row tile
        if (row_mul == 1) hx_repack_t128(c.words, c.micro, c.rows, c.K, c.Kpad, f.t128, f.ksteps / 4, 1, 1, row_off, m->st);
        else hx_repack_t128(c.words, c.micro, c.rows, c.K, c.Kpad, f.t128, f.ksteps / 4, 64, row_mul, row_off, m->st);
    }
}

int build(hx_model* m, Source& s) {
    const hx_config& c = m->cfg;
    const int NL = c.n_layers, DM = c.d_model, DH = c.head_dim, DFF = c.d_ff, NV = c.vocab;     // this rank's shard
    const int QD = m->QD, KVD = m->KVD;
    // tensors are fetched whole (the per-tensor scale and the codes are those of the full tensor) and this rank's
    // rows or columns are laid out: q/k/v/gate/up/lm_head split by rows, o/down by columns
    const int W = m->tp_world, R = m->tp_rank;
    const int gQD = m->gcfg.n_heads * DH, gKVD = m->gcfg.n_kv_heads * DH, gDFF = m->gcfg.d_ff, gNV = m->gcfg.vocab;
    auto put = [&](const Committed& cm, Fused& f, int row_mul, int row_off, int rows_local, bool split_rows, int klen) {
        if (W == 1) { put_rows(m, cm, f, row_mul, row_off); return; }
        const int kwords = cm.Kpad / 7, kblk = cm.Kpad / 16;
        const int r0 = split_rows ? R * rows_local : 0, k0 = split_rows ? 0 : R * klen;
        const int grp = row_mul == 1 ? 1 : 64;
        hx_repack_t128(cm.words + (size_t)r0 * kwords, cm.micro + (size_t)r0 * kblk, rows_local, split_rows ? cm.K : klen, cm.Kpad,
                       f.t128, f.ksteps / 4, grp, row_mul, row_off, m->st, k0);
    };
    const bool keep = (m->flags & HX_LOAD_KEEP_COMMITTED) != 0;
    // staging sized for the largest tensor
    size_t maxel = (size_t)gNV * DM;
    const size_t cand[] = {(size_t)gQD * DM, (size_t)gDFF * DM, (size_t)DM * gDFF, (size_t)DM * gQD};
    for (size_t v : cand) if (v > maxel) maxel = v;
    int rc;
    std::vector<void*> staging;
    auto salloc = [&](void** p, size_t bytes) -> int {
        cudaError_t e = cudaMalloc(p, bytes);
        if (e != cudaSuccess) return hx_fail(HX_ERR_NOMEM, "staging cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
        staging.push_back(*p); return HX_OK;
    };
    auto sfree = [&]() { for (void* p : staging) cudaFree(p); staging.clear(); };
    if (s.synth) { rc = salloc((void**)&s.f32tmp, maxel * 4); if (rc) { sfree(); return rc; } }
    if (!keep) {
        const int shp[][2] = {{gQD, DM}, {gKVD, DM}, {DM, gQD}, {gDFF, DM}, {DM, gDFF}, {gNV, DM}};
        size_t wmax = 0, mmax = 0;
        for (auto& sh : shp) {
            const size_t kp = (size_t)hx_kpad(sh[1]);
            if ((size_t)sh[0] * (kp / 7) * 4 > wmax) wmax = (size_t)sh[0] * (kp / 7) * 4;
            if ((size_t)sh[0] * (kp / 16) > mmax) mmax = (size_t)sh[0] * (kp / 16);
        }
        rc = salloc((void**)&s.wtmp, wmax); if (rc) { sfree(); return rc; }
        rc = salloc((void**)&s.mtmp, mmax); if (rc) { sfree(); return rc; }
    }
    rc = salloc((void**)&s.tstmp, 256); if (rc) { sfree(); return rc; }

    m->layers.resize(NL);
    for (int L = 0; L < NL && !rc; L++) {
        Layer& ly = m->layers[L];
        const int b = L * T_PER_LAYER;
        do {
            if ((rc = fetch_dense(m, s, b + T_INLN, DM, &ly.in_g, true))) break;
            if ((rc = fetch_dense(m, s, b + T_POSTLN, DM, &ly.post_g, true))) break;
            if (c.qk_norm) {
                if ((rc = fetch_dense(m, s, b + T_QN, DH, &ly.qn_g, true))) break;
                if ((rc = fetch_dense(m, s, b + T_KN, DH, &ly.kn_g, true))) break;
            }
            if ((rc = alloc_fused(m, ly.qkv, QD + 2 * KVD, DM))) break;
            if ((rc = alloc_fused(m, ly.o, DM, QD))) break;
            if ((rc = alloc_fused(m, ly.gu, 2 * DFF, DM))) break;
            if (DFF % 16 && ly.gu.t16) {          // tile-interleaved pairs need whole tiles for gate and for up
                ly.gu.ntiles = 2 * hx_t16_tiles(DFF);
                if ((rc = dalloc(m, &ly.gu.t16, (size_t)ly.gu.ntiles * ly.gu.KG * HX_T16_CELL))) break;
                HX_CUDA(cudaMemsetAsync(ly.gu.t16, 0, (size_t)ly.gu.ntiles * ly.gu.KG * HX_T16_CELL, m->st));
            }
            if ((rc = alloc_fused(m, ly.down, DM, DFF))) break;
            if ((rc = fetch_packed(m, s, b + T_Q, gQD, DM, ly.c[T_Q], keep))) break;
            put(ly.c[T_Q], ly.qkv, 1, 0, QD, true, 0); ly.qkv.ts[0] = ly.c[T_Q].ts;
            if ((rc = fetch_packed(m, s, b + T_K, gKVD, DM, ly.c[T_K], keep))) break;
            put(ly.c[T_K], ly.qkv, 1, QD, KVD, true, 0); ly.qkv.ts[1] = ly.c[T_K].ts;
            if ((rc = fetch_packed(m, s, b + T_V, gKVD, DM, ly.c[T_V], keep))) break;
            put(ly.c[T_V], ly.qkv, 1, QD + KVD, KVD, true, 0); ly.qkv.ts[2] = ly.c[T_V].ts;
            ly.qkv.bound0 = QD; ly.qkv.bound1 = QD + KVD;
            if ((rc = fetch_packed(m, s, b + T_O, DM, gQD, ly.c[T_O], keep))) break;
            put(ly.c[T_O], ly.o, 1, 0, DM, false, QD); ly.o.ts[0] = ly.o.ts[1] = ly.o.ts[2] = ly.c[T_O].ts; ly.o.bound0 = ly.o.bound1 = DM;
            if ((rc = fetch_packed(m, s, b + T_GATE, gDFF, DM, ly.c[T_GATE], keep))) break;
            put(ly.c[T_GATE], ly.gu, 2, 0, DFF, true, 0); ly.gu.ts[0] = ly.c[T_GATE].ts;
            if ((rc = fetch_packed(m, s, b + T_UP, gDFF, DM, ly.c[T_UP], keep))) break;
            put(ly.c[T_UP], ly.gu, 2, 1, DFF, true, 0); ly.gu.ts[1] = ly.c[T_UP].ts; ly.gu.bound0 = ly.gu.bound1 = 2 * DFF;
            if ((rc = fetch_packed(m, s, b + T_DOWN, DM, gDFF, ly.c[T_DOWN], keep))) break;
            put(ly.c[T_DOWN], ly.down, 1, 0, DM, false, DFF); ly.down.ts[0] = ly.down.ts[1] = ly.down.ts[2] = ly.c[T_DOWN].ts; ly.down.bound0 = ly.down.bound1 = DM;
            cudaError_t e = cudaStreamSynchronize(m->st);
            if (e != cudaSuccess) { rc = hx_fail(HX_ERR_CUDA, "layer %d ingest: %s", L, cudaGetErrorString(e)); break; }
        } while (0);
    }
    if (!rc) do {
        const int b = NL * T_PER_LAYER;
        if ((rc = fetch_dense(m, s, b + 0, (size_t)gNV * DM, &m->emb, false))) break;
        if ((rc = fetch_dense(m, s, b + 1, DM, &m->final_g, true))) break;
        if ((rc = alloc_fused(m, m->head, NV, DM))) break;
        if ((rc = fetch_packed(m, s, b + 2, gNV, DM, m->head_c, keep))) break;
        put(m->head_c, m->head, 1, 0, NV, true, 0);
        m->head.ts[0] = m->head.ts[1] = m->head.ts[2] = m->head_c.ts; m->head.bound0 = m->head.bound1 = NV;
        cudaError_t e = cudaStreamSynchronize(m->st);
        if (e != cudaSuccess) rc = hx_fail(HX_ERR_CUDA, "head ingest: %s", cudaGetErrorString(e));
    } while (0);
    sfree();
    return rc;
}

int alloc_state(hx_model* m) {
    const hx_config& c = m->cfg;
    const int DM = c.d_model, DH = c.head_dim, NH = c.n_heads, NKV = c.n_kv_heads, cap = m->kv_cap;
    int rc;
    const int QDd = hx_kd(m->QD), DFFd = hx_kd(c.d_ff);
    if ((rc = dalloc(m, &m->x, (size_t)DM))) return rc;
    if ((rc = dalloc(m, &m->qkv, (size_t)m->QD + 2 * m->KVD))) return rc;
    if ((rc = dalloc(m, &m->q_rot, (size_t)m->QD))) return rc;
    if ((rc = dalloc(m, &m->ctx, (size_t)QDd))) return rc;
    if ((rc = dalloc(m, &m->h, (size_t)DFFd))) return rc;
    if ((rc = dalloc(m, &m->logits, (size_t)c.vocab))) return rc;
    HX_CUDA(cudaMemset(m->ctx, 0, (size_t)QDd * 4));
    HX_CUDA(cudaMemset(m->h, 0, (size_t)DFFd * 4));
    const size_t kvn = (size_t)c.n_layers * NKV * cap * DH * (size_t)m->batch;      // [sequence][layer][kv head][position][dim]
    if ((rc = dalloc(m, &m->kc, kvn))) return rc;
    if ((rc = dalloc(m, &m->vc, kvn))) return rc;
    HX_CUDA(cudaMemset(m->kc, 0, kvn * 4));
    HX_CUDA(cudaMemset(m->vc, 0, kvn * 4));
    // RoPE tables, double precision on the host, cast to f32 (gpt2_infer.c:2040-2051)
    const int half = DH / 2;
    std::vector<float> hc((size_t)cap * half), hs((size_t)cap * half);
    for (int s = 0; s < cap; s++)
        for (int j = 0; j < half; j++) {
            const double inv = pow((double)c.rope_theta, -2.0 * (double)j / (double)DH);
            const double ang = (double)s * inv;
            hc[(size_t)s * half + j] = (float)cos(ang);
            hs[(size_t)s * half + j] = (float)sin(ang);
        }
    if ((rc = dalloc(m, &m->cosT, hc.size()))) return rc;
    if ((rc = dalloc(m, &m->sinT, hs.size()))) return rc;
    HX_CUDA(cudaMemcpy(m->cosT, hc.data(), hc.size() * 4, cudaMemcpyHostToDevice));
    HX_CUDA(cudaMemcpy(m->sinT, hs.data(), hs.size() * 4, cudaMemcpyHostToDevice));
    int sms = 148; { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
    m->nsplit = sms / NKV; if (m->nsplit < 1) m->nsplit = 1; if (m->nsplit > 64) m->nsplit = 64;
    if ((rc = dalloc(m, &m->part_m, (size_t)NH * m->nsplit))) return rc;
    if ((rc = dalloc(m, &m->part_l, (size_t)NH * m->nsplit))) return rc;
    if ((rc = dalloc(m, &m->part_acc, (size_t)NH * m->nsplit * DH))) return rc;
    if ((rc = dalloc(m, &m->part_amax, (size_t)NH * m->nsplit))) return rc;
    if ((rc = dalloc(m, &m->attn_cnt, (size_t)NKV))) return rc;
    HX_CUDA(cudaMemset(m->attn_cnt, 0, (size_t)NKV * 4));
    if ((rc = dalloc(m, &m->am_val, (size_t)4096))) return rc;
    if ((rc = dalloc(m, &m->am_idx, (size_t)4096))) return rc;
    if ((rc = dalloc(m, &m->am_cnt, (size_t)4))) return rc;
    HX_CUDA(cudaMemset(m->am_cnt, 0, 16));
    if ((rc = dalloc(m, &m->d_tok, (size_t)4))) return rc;
    if ((rc = dalloc(m, &m->d_pos, (size_t)4))) return rc;
    if ((rc = dalloc(m, &m->d_hist, (size_t)cap + 8))) return rc;
    if ((rc = dalloc(m, &m->d_prompt, (size_t)cap + 8))) return rc;
    HX_CUDA(cudaMemset(m->d_hist, 0, ((size_t)cap + 8) * 4));
    HX_CUDA(cudaEventCreate(&m->ev0));
    HX_CUDA(cudaEventCreate(&m->ev1));
    return HX_OK;
}

__global__ void k_advance(int* pos) { hx_grid_dep_launch(); hx_grid_dep_wait(); if (threadIdx.x == 0) *pos = *pos + 1; }

HxLinear lin(const Fused& f, const float* x, float* y, int epi) {
    HxLinear a = {};
    a.codes = reinterpret_cast<const uint4*>(f.codes); a.scales = f.scales;
    a.ts[0] = f.ts[0]; a.ts[1] = f.ts[1]; a.ts[2] = f.ts[2]; a.bound0 = f.bound0; a.bound1 = f.bound1;
    a.N = f.N; a.K = f.K; a.Kd = f.Kd; a.x = x; a.y = y; a.epi = epi; a.norm = HX_NORM_NONE;
    return a;
}

// Per-kernel timing (hx_model_set_profile): an event before and after every launch, eager stream order.
enum { CAT_GEMV = 0, CAT_ATTN = 1, CAT_OTHER = 2 };
struct ProfScope {
    hx_model* m; int cat; bool on;
    ProfScope(hx_model* mm, int c, bool active) : m(mm), cat(c), on(active) {
        if (!on) return;
        if (m->prof_n + 2 > m->prof_ev.size()) {
            for (int i = 0; i < 2; i++) { cudaEvent_t e; cudaEventCreate(&e); m->prof_ev.push_back(e); }
            m->prof_cat.push_back(cat);
        }
        m->prof_cat[m->prof_n / 2] = cat;
        cudaEventRecord(m->prof_ev[m->prof_n], m->st);
    }
    ~ProfScope() { if (on) { cudaEventRecord(m->prof_ev[m->prof_n + 1], m->st); m->prof_n += 2; } }
};

// Enqueue one token step on m->st.  from_prompt: the input token is d_prompt[*pos] and no logits are
// computed (prefill); otherwise the input token is *d_tok and the head + arg-max run.
// GPT-2 block sequencing (forward_layer_gpt2, helixc/runtime/gpt2_infer.c:1131-1193, with a KV cache): LayerNorm ->
// fused qkv (+bias) -> attention (scale 1/sqrt(DH), no RoPE, no QK norm) -> proj (+bias, residual) -> LayerNorm ->
// c_fc (+bias, gelu_new) -> proj (+bias, residual); ln_f and the tied lm_head at the end.  The embedding kernel has
// already added the learned position row.
int enqueue_step_gpt2(hx_model* m, bool from_prompt, bool with_head, bool prof) {
    (void)from_prompt;
    const hx_config& c = m->cfg;
    const int DH = c.head_dim, cap = m->kv_cap;
    const bool pdl = m->pdl && !prof;
    int rc;
    for (int L = 0; L < c.n_layers; L++) {
        Layer& ly = m->layers[L];
        HxLinear a = lin(ly.qkv, m->x, m->qkv, HX_EPI_STORE);
        a.norm = HX_NORM_LAYER; a.norm_g = ly.in_g; a.norm_b = ly.ln1_b; a.eps = c.norm_eps; a.bias = ly.b_qkv;
        { ProfScope ps(m, CAT_GEMV, prof); if ((rc = hx_launch_linear(a, m->st, pdl))) return rc; }
        HxAttn at = {};
        at.qkv = m->qkv; at.q_rot = m->q_rot;
        at.kc = m->kc + (size_t)L * c.n_kv_heads * cap * DH; at.vc = m->vc + (size_t)L * c.n_kv_heads * cap * DH;
        at.pos = m->d_pos; at.NH = c.n_heads; at.NKV = c.n_kv_heads; at.DH = DH; at.cap = cap;
        at.eps = c.norm_eps; at.scale = 1.0f / sqrtf((float)DH); at.nsplit = m->nsplit;
        at.part_m = m->part_m; at.part_l = m->part_l; at.part_acc = m->part_acc; at.counters = m->attn_cnt; at.ctx = m->ctx;
        { ProfScope ps(m, CAT_OTHER, prof); if ((rc = hx_launch_qk_prep(at, m->st, pdl))) return rc; }
        { ProfScope ps(m, CAT_ATTN, prof); if ((rc = hx_launch_attn(at, m->st, pdl))) return rc; }
        HxLinear o = lin(ly.o, m->ctx, m->x, HX_EPI_RESID); o.resid = m->x; o.bias = ly.b_o;
        { ProfScope ps(m, CAT_GEMV, prof); if ((rc = hx_launch_linear(o, m->st, pdl))) return rc; }
        HxLinear fc = lin(ly.gu, m->x, m->h, HX_EPI_GELU);
        fc.norm = HX_NORM_LAYER; fc.norm_g = ly.post_g; fc.norm_b = ly.ln2_b; fc.eps = c.norm_eps; fc.bias = ly.b_fc;
        { ProfScope ps(m, CAT_GEMV, prof); if ((rc = hx_launch_linear(fc, m->st, pdl))) return rc; }
        HxLinear dn = lin(ly.down, m->h, m->x, HX_EPI_RESID); dn.resid = m->x; dn.bias = ly.b_down;
        { ProfScope ps(m, CAT_GEMV, prof); if ((rc = hx_launch_linear(dn, m->st, pdl))) return rc; }
    }
    if (with_head) {
        HxLinear hd = lin(m->head, m->x, m->logits, HX_EPI_ARGMAX);
        hd.norm = HX_NORM_LAYER; hd.norm_g = m->final_g; hd.norm_b = m->final_b; hd.eps = c.norm_eps;
        hd.part_val = m->am_val; hd.part_idx = m->am_idx; hd.counter = m->am_cnt; hd.next_tok = m->d_tok; hd.pos_inc = m->d_pos;
        hd.hist = m->d_hist;
        { ProfScope ps(m, CAT_GEMV, prof); if ((rc = hx_launch_linear(hd, m->st, pdl))) return rc; }
    } else {
        k_advance<<<1, 32, 0, m->st>>>(m->d_pos);
        HX_COUNT_LAUNCH(1);
        HX_CUDA(cudaGetLastError());
    }
    return HX_OK;
}

int enqueue_step(hx_model* m, bool from_prompt, bool with_head, bool prof = false) {
    const hx_config& c = m->cfg;
    const int DM = c.d_model, DH = c.head_dim, cap = m->kv_cap;
    const bool pdl = m->pdl && !prof;
    int rc;
    {
        // the first kernel of a step follows the last kernel of the previous step
        const int* tok = from_prompt ? m->d_prompt : m->d_tok;
        ProfScope ps(m, CAT_OTHER, prof);
        rc = hx_launch_embed(m->emb, c.arch == 0 ? m->wpe : nullptr, tok, m->d_pos, from_prompt ? 1 : 0, m->x, DM, m->st, pdl);
        if (rc) return rc;
    }
    if (c.arch == 0) return enqueue_step_gpt2(m, from_prompt, with_head, prof);
    for (int L = 0; L < c.n_layers; L++) {
        Layer& ly = m->layers[L];
        HxLinear a = lin(ly.qkv, m->x, m->qkv, HX_EPI_STORE);
        a.norm = HX_NORM_RMS; a.norm_g = ly.in_g; a.eps = c.norm_eps;
        { ProfScope ps(m, CAT_GEMV, prof); if ((rc = hx_launch_linear(a, m->st, pdl))) return rc; }
        HxAttn at = {};
        at.qkv = m->qkv; at.q_rot = m->q_rot; at.qn_g = ly.qn_g; at.kn_g = ly.kn_g;
        at.cosT = m->cosT; at.sinT = m->sinT;
        at.kc = m->kc + (size_t)L * c.n_kv_heads * cap * DH; at.vc = m->vc + (size_t)L * c.n_kv_heads * cap * DH;
        at.pos = m->d_pos; at.NH = c.n_heads; at.NKV = c.n_kv_heads; at.DH = DH; at.cap = cap;
        at.eps = c.norm_eps; at.scale = 1.0f / sqrtf((float)DH); at.nsplit = m->nsplit;
        at.part_m = m->part_m; at.part_l = m->part_l; at.part_acc = m->part_acc; at.counters = m->attn_cnt; at.ctx = m->ctx;
        { ProfScope ps(m, CAT_OTHER, prof); if ((rc = hx_launch_qk_prep(at, m->st, pdl))) return rc; }
        { ProfScope ps(m, CAT_ATTN, prof); if ((rc = hx_launch_attn(at, m->st, pdl))) return rc; }
        HxLinear o = lin(ly.o, m->ctx, m->x, HX_EPI_RESID); o.resid = m->x;
        { ProfScope ps(m, CAT_GEMV, prof); if ((rc = hx_launch_linear(o, m->st, pdl))) return rc; }
        HxLinear gu = lin(ly.gu, m->x, m->h, HX_EPI_SWIGLU);
        gu.norm = HX_NORM_RMS; gu.norm_g = ly.post_g; gu.eps = c.norm_eps;
        { ProfScope ps(m, CAT_GEMV, prof); if ((rc = hx_launch_linear(gu, m->st, pdl))) return rc; }
        HxLinear dn = lin(ly.down, m->h, m->x, HX_EPI_RESID); dn.resid = m->x;
        { ProfScope ps(m, CAT_GEMV, prof); if ((rc = hx_launch_linear(dn, m->st, pdl))) return rc; }
    }
    if (with_head) {
        HxLinear hd = lin(m->head, m->x, m->logits, HX_EPI_ARGMAX);
        hd.norm = HX_NORM_RMS; hd.norm_g = m->final_g; hd.eps = c.norm_eps;
        hd.part_val = m->am_val; hd.part_idx = m->am_idx; hd.counter = m->am_cnt; hd.next_tok = m->d_tok; hd.pos_inc = m->d_pos;
        hd.hist = m->d_hist;
        { ProfScope ps(m, CAT_GEMV, prof); if ((rc = hx_launch_linear(hd, m->st, pdl))) return rc; }
    } else {
        k_advance<<<1, 32, 0, m->st>>>(m->d_pos);
        HX_COUNT_LAUNCH(1);
        HX_CUDA(cudaGetLastError());
    }
    return HX_OK;
}

int capture(hx_model* m, bool from_prompt, bool with_head, cudaGraphExec_t* out) {
    cudaGraph_t g = nullptr;
    HX_CUDA(cudaStreamBeginCapture(m->st, cudaStreamCaptureModeThreadLocal));
    const unsigned long long before = g_hx_launches;
    int rc = enqueue_step(m, from_prompt, with_head);
    cudaError_t e = cudaStreamEndCapture(m->st, &g);
    g_hx_launches = before;                       // captured, not launched
    if (rc) { if (g) cudaGraphDestroy(g); return rc; }
    if (e != cudaSuccess) return hx_fail(HX_ERR_CUDA, "graph capture: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(out, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return hx_fail(HX_ERR_CUDA, "graph instantiate: %s", cudaGetErrorString(e));
    return HX_OK;
}

int kernels_per_step(const hx_model* m, bool with_head) { (void)with_head; return 1 + 6 * m->cfg.n_layers + 1; }

// Phase table of one token for the persistent kernel: per layer qkv, attention, o_proj, gate+up, down;
// then (with_head) the lm_head.  from_prompt: layer 0 reads the token from the prompt array.
int build_phases(hx_model* m, bool from_prompt, bool with_head, HxPhase** out, int* nout) {
    const hx_config& c = m->cfg;
    const int DH = c.head_dim, cap = m->kv_cap;
    std::vector<HxPhase> v;
    auto linear = [&](const Fused& f, const float* x, float* y, int epi, int N) {
        HxPhase p = {};
        p.type = HX_PH_LINEAR; p.w = f.t16; p.ntiles = f.ntiles; p.KG = f.KG; p.unit = (epi == HX_EPI_SWIGLU) ? 2 : 1;
        if (m->use_tc) {
            p.type = HX_PH_LINEAR_TC; p.w = f.t128; p.ntiles = f.tiles128; p.ksteps = f.ksteps;
            int maxp = 1, maxrun = 1;
            if (m->use_df) {
                // per-CTA work split from a table (one per distinct tile grid, shared by the layers)
                const long long key = ((long long)p.ntiles << 32) | (unsigned)(p.ksteps / 4);
                size_t slot = 0;
                for (; slot < m->plan_keys.size(); slot++) if (m->plan_keys[slot] == key) break;
                std::vector<HxCtaPlan> tab((size_t)m->grid_persist);
                hx_df_plan(p.ntiles, p.ksteps / 4, m->grid_persist, tab.data(), &maxp, &maxrun);
                if (slot == m->plan_keys.size()) {
                    HxCtaPlan* d = nullptr;
                    if (dalloc(m, &d, tab.size()) == HX_OK && cudaMemcpy(d, tab.data(), tab.size() * sizeof(HxCtaPlan), cudaMemcpyHostToDevice) == cudaSuccess) {
                        m->plan_keys.push_back(key); m->plan_tabs.push_back(d);
                    }
                }
                p.plan = slot < m->plan_tabs.size() ? m->plan_tabs[slot] : nullptr;
            } else
            hx_tc_split(p.ntiles, p.ksteps / 4, m->grid_persist, &maxp, &maxrun);
            p.pieces = maxp;
            if ((size_t)p.ntiles * maxp > m->tc_units_max) m->tc_units_max = (size_t)p.ntiles * maxp;
            if (p.ntiles > m->tc_tiles_max) m->tc_tiles_max = p.ntiles;
            const int per_cell = m->use_df ? 3072 : 2048;       // digit cells (+ the staged input values of the dataflow engine)
            if (maxrun * per_cell > m->bdig_bytes) m->bdig_bytes = maxrun * per_cell;
        }
        p.N = N; p.x = x; p.K = f.K; p.norm = HX_NORM_NONE; p.epi = epi; p.y = y;
        p.ts[0] = f.ts[0]; p.ts[1] = f.ts[1]; p.ts[2] = f.ts[2]; p.bound0 = f.bound0; p.bound1 = f.bound1;
        return p;
    };
    int maxK = 0;
    // tensor parallel: o_proj and down leave per-rank partial sums; the next linear's prologue adds them to the residual
    // stream, which alternates between two buffers (a CTA must not overwrite what another still reads)
    const bool tp = m->tp_world > 1 && !m->use_df;
    float* xcur = m->x; int nbar = 0;
    if (m->use_df) {
        // Dataflow engine: the residual stream alternates between two pair buffers (xll[0] after o_proj, xll[1] after
        // down), every other vector has one buffer per producing phase of a layer; `*_dep` is the index of the phase
        // whose epoch tags an input.  With several ranks o_proj and down are row-split and their residual epilogue
        // exchanges the partial rows (tp_partial = slot + 1).
        const int ntile_dm = (c.d_model + 127) / 128;
        const bool dtp = m->tp_world > 1;
        int dep_x = -1;                                   // phase that produced the current residual stream (-1: the embedding row)
        for (int L = 0; L < c.n_layers; L++) {
            Layer& ly = m->layers[L];
            float* kcl = m->kc + (size_t)L * c.n_kv_heads * cap * DH; float* vcl = m->vc + (size_t)L * c.n_kv_heads * cap * DH;
            HxPhase a = linear(ly.qkv, nullptr, nullptr, HX_EPI_QKV, ly.qkv.N);
            a.norm = HX_NORM_RMS; a.g = ly.in_g; a.eps = c.norm_eps;
            if (dep_x < 0) { a.x = m->emb; a.tok = from_prompt ? m->d_prompt : m->d_tok; a.res_ld = c.d_model; }
            else { a.in_ll = m->xll[1]; a.in_stat = m->statll[1]; a.n_in_stat = ntile_dm; a.in_dep = dep_x; }
            a.qn_g = ly.qn_g; a.kn_g = ly.kn_g; a.cosT = m->cosT; a.sinT = m->sinT; a.kc = kcl; a.vc = vcl;
            a.NH = c.n_heads; a.NKV = c.n_kv_heads; a.DH = DH; a.cap = cap;
            a.out_ll = m->qll; a.kv_ll = m->kvll; a.part_ll = m->part_ll[0];
            const int i_qkv = (int)v.size(); v.push_back(a);
            HxPhase at = {};
            at.type = HX_PH_ATTN; at.epi = HX_EPI_QKV; at.kc = kcl; at.vc = vcl;
            at.NH = c.n_heads; at.NKV = c.n_kv_heads; at.DH = DH; at.cap = cap;
            at.nsplit = m->nsplit_persist; at.scale = 1.0f / sqrtf((float)DH); at.eps = c.norm_eps;
            at.in_ll = m->qll; at.kv_ll = m->kvll; at.in_dep = i_qkv;
            at.pacc_ll = m->pacc_ll; at.pml_ll = m->pml_ll; at.out_ll = m->ctxll;       // splits merged by one CTA per head
            const int i_att = (int)v.size(); v.push_back(at);
            HxPhase o = linear(ly.o, nullptr, nullptr, HX_EPI_RESID, ly.o.N);
            o.in_ll = m->ctxll; o.in_dep = i_att;
            {   // the CTA's K slice of the input is staged in shared memory behind its digit cells
                int maxp = 1, maxrun = 1;
                std::vector<HxCtaPlan> tab((size_t)m->grid_persist);
                hx_df_plan(o.ntiles, o.ksteps / 4, m->grid_persist, tab.data(), &maxp, &maxrun);
                if (maxrun * 3072 > m->bdig_bytes) m->bdig_bytes = maxrun * 3072;
            }
            if (dep_x < 0) { o.x = m->emb; o.tok = from_prompt ? m->d_prompt : m->d_tok; o.res_ld = c.d_model; }
            else { o.res_ll = m->xll[1]; o.res_dep = dep_x; }
            o.out_ll = m->xll[0]; o.out_stat = m->statll[0]; o.part_ll = m->part_ll[1];
            if (dtp) o.tp_partial = 1;
            const int i_o = (int)v.size(); v.push_back(o);
            HxPhase gu = linear(ly.gu, nullptr, nullptr, HX_EPI_SWIGLU, c.d_ff);
            gu.norm = HX_NORM_RMS; gu.g = ly.post_g; gu.eps = c.norm_eps;
            gu.in_ll = m->xll[0]; gu.in_stat = m->statll[0]; gu.n_in_stat = ntile_dm; gu.in_dep = i_o;
            gu.out_ll = m->hll; gu.part_ll = m->part_ll[2];
            const int i_gu = (int)v.size(); v.push_back(gu);
            HxPhase dn = linear(ly.down, nullptr, nullptr, HX_EPI_RESID, ly.down.N);
            dn.in_ll = m->hll; dn.in_dep = i_gu; dn.res_ll = m->xll[0]; dn.res_dep = i_o;
            dn.out_ll = m->xll[1]; dn.out_stat = m->statll[1]; dn.part_ll = m->part_ll[3];
            if (dtp) dn.tp_partial = 2;
            dep_x = (int)v.size(); v.push_back(dn);
        }
        if (with_head) {
            HxPhase hd = linear(m->head, nullptr, m->logits, HX_EPI_ARGMAX, m->head.N);
            hd.norm = HX_NORM_RMS; hd.g = m->final_g; hd.eps = c.norm_eps;
            if (dep_x < 0) { hd.x = m->emb; hd.tok = from_prompt ? m->d_prompt : m->d_tok; hd.res_ld = c.d_model; }
            else { hd.in_ll = m->xll[1]; hd.in_stat = m->statll[1]; hd.n_in_stat = ntile_dm; hd.in_dep = dep_x; }
            hd.part_ll = m->part_ll[4];
            v.push_back(hd);
        }
    } else
    for (int L = 0; L < c.n_layers; L++) {
        Layer& ly = m->layers[L];
        HxPhase a = linear(ly.qkv, xcur, m->qkv, HX_EPI_STORE, ly.qkv.N);
        a.norm = HX_NORM_RMS; a.g = ly.in_g; a.eps = c.norm_eps;
        if (L == 0) { a.x = m->emb; a.tok = from_prompt ? m->d_prompt : m->d_tok; a.x_out = m->x; xcur = m->x; }
        else if (tp) { a.tp_sum = 2; a.x_out = xcur == m->x ? m->x2 : m->x; xcur = a.x_out; }     // + down partials of the layer before
        // tensor-core path: the qkv epilogue norms and rotates q and k and writes k, v into the cache
        const bool fuse_qk = m->use_tc && (DH == 32 || DH == 64 || DH == 128);
        if (fuse_qk) {
            a.epi = HX_EPI_QKV; a.qn_g = ly.qn_g; a.kn_g = ly.kn_g; a.cosT = m->cosT; a.sinT = m->sinT;
            a.kc = m->kc + (size_t)L * c.n_kv_heads * cap * DH; a.vc = m->vc + (size_t)L * c.n_kv_heads * cap * DH;
            a.NH = c.n_heads; a.NKV = c.n_kv_heads; a.DH = DH; a.cap = cap;
        }
        v.push_back(a);
        HxPhase at = {};
        if (fuse_qk) at.epi = HX_EPI_QKV;          // q arrives prepared, the position's k and v are cached
        at.type = HX_PH_ATTN; at.qkv = m->qkv; at.qn_g = ly.qn_g; at.kn_g = ly.kn_g; at.cosT = m->cosT; at.sinT = m->sinT;
        at.kc = m->kc + (size_t)L * c.n_kv_heads * cap * DH; at.vc = m->vc + (size_t)L * c.n_kv_heads * cap * DH;
        at.ctx = m->ctx; at.NH = c.n_heads; at.NKV = c.n_kv_heads; at.DH = DH; at.cap = cap;
        at.nsplit = m->nsplit_persist; at.scale = 1.0f / sqrtf((float)DH); at.eps = c.norm_eps;
        v.push_back(at);
        HxPhase o = linear(ly.o, m->ctx, xcur, HX_EPI_RESID, ly.o.N);
        if (tp) { o.tp_partial = 1; o.tp_barrier = 1; o.tp_epoch = ++nbar; }
        // the o_proj prologue merges the attention splits itself (no merging CTA on the critical path)
        const bool defer_merge = fuse_qk && (size_t)c.n_heads * m->nsplit_persist <= 2304 && DH % 8 == 0;
        if (defer_merge) {
            v.back().pieces = 1;                       // attention phase: leave the partials unmerged
            o.norm = HX_NORM_ATTN; o.NH = c.n_heads; o.NKV = c.n_kv_heads; o.DH = DH; o.nsplit = m->nsplit_persist;
        }
        v.push_back(o);
        HxPhase gu = linear(ly.gu, xcur, m->h, HX_EPI_SWIGLU, c.d_ff);
        gu.norm = HX_NORM_RMS; gu.g = ly.post_g; gu.eps = c.norm_eps;
        if (tp) { gu.tp_sum = 1; gu.x_out = xcur == m->x ? m->x2 : m->x; xcur = gu.x_out; }                                   // + o partials
        v.push_back(gu);
        HxPhase dn = linear(ly.down, m->h, xcur, HX_EPI_RESID, ly.down.N);
        if (tp) { dn.tp_partial = 2; dn.tp_barrier = 1; dn.tp_epoch = ++nbar; }
        v.push_back(dn);
        if (ly.down.K > maxK) maxK = ly.down.K;
        if (ly.o.K > maxK) maxK = ly.o.K;
        if (ly.qkv.K > maxK) maxK = ly.qkv.K;
    }
    if (with_head && !m->use_df) {
        HxPhase hd = linear(m->head, xcur, m->logits, HX_EPI_ARGMAX, m->head.N);
        hd.norm = HX_NORM_RMS; hd.g = m->final_g; hd.eps = c.norm_eps;
        if (tp && c.n_layers > 0) { hd.tp_sum = 2; hd.x_out = xcur == m->x ? m->x2 : m->x; }
        v.push_back(hd);
    }
    m->tp_nbar = nbar;
    const int dig = 3 * hx_t16_kgroups(maxK) * HX_T16_KG * 2;
    if (dig > m->dig_bytes) m->dig_bytes = dig;
    HxPhase* d = nullptr;
    int rc = dalloc(m, &d, v.size()); if (rc) return rc;
    HX_CUDA(cudaMemcpy(d, v.data(), v.size() * sizeof(HxPhase), cudaMemcpyHostToDevice));
    *out = d; *nout = (int)v.size();
    return HX_OK;
}

int init_persist(hx_model* m) {
    int dev = 0, sms = 0, coop = 0;
    HX_CUDA(cudaGetDevice(&dev));
    HX_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    HX_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    if (!coop) return hx_fail(HX_ERR_CUDA, "device does not support cooperative launches");
    m->grid_persist = sms;
    m->nsplit_persist = sms / m->cfg.n_kv_heads; if (m->nsplit_persist < 1) m->nsplit_persist = 1;
    if (m->nsplit_persist > m->nsplit) m->nsplit_persist = m->nsplit;      // scratch is sized for nsplit
    if (const char* e = getenv("HX_ATT_SPLIT")) { const int v = atoi(e); if (v >= 1 && v <= m->nsplit_persist) m->nsplit_persist = v; }
    if (256 % m->cfg.head_dim) return hx_fail(HX_ERR_ARG, "persistent decode needs head_dim dividing 256");
    int rc;
    {   // the dataflow engine needs the fused qkv epilogue (whole heads per tile) and room for the split weights
        const hx_config& c = m->cfg;
        const char* sy = getenv("HX_SYNC");
        const bool fuse_qk = c.head_dim == 32 || c.head_dim == 64 || c.head_dim == 128;
        // (the prologue polls at most 64 per-tile sums of squares: d_model up to 8192)
        m->use_df = m->use_tc && fuse_qk && (size_t)c.n_heads * m->nsplit_persist <= 2304 && c.d_model <= 8192 && !(sy && strcmp(sy, "barrier") == 0);
    }
    if (m->tp_world > 1 && !m->use_df) m->pf_batched = false;       // the chunk exchange of a shard belongs to the pair engine
    if (m->use_df) {
        const hx_config& c = m->cfg;
        const int DH = c.head_dim, QD = m->QD, KVD = m->KVD, ntile_dm = (c.d_model + 127) / 128;
        auto ll = [&](unsigned long long** p, size_t n) -> int {
            int r = dalloc(m, p, n + 2); if (r) return r;
            HX_CUDA(cudaMemset(*p, 0, (n + 2) * 8));
            return HX_OK;
        };
        for (int i = 0; i < 2; i++) { if ((rc = ll(&m->xll[i], (size_t)ntile_dm * 128))) return rc; if ((rc = ll(&m->statll[i], (size_t)ntile_dm))) return rc; }
        if ((rc = ll(&m->qll, (size_t)QD + 128))) return rc;
        if ((rc = ll(&m->kvll, (size_t)2 * KVD + 128))) return rc;
        if ((rc = ll(&m->hll, (size_t)((c.d_ff + 63) / 64) * 64 + 128))) return rc;
        const size_t hs = (size_t)c.n_heads * m->nsplit_persist;
        if ((rc = ll(&m->pacc_ll, hs * DH))) return rc;
        if ((rc = ll(&m->pml_ll, hs * 2))) return rc;
        if ((rc = ll(&m->ctxll, (size_t)QD + 128))) return rc;
        auto parts = [&](const Fused& f) -> size_t {
            int maxp = 1, maxrun = 1;
            std::vector<HxCtaPlan> tab((size_t)m->grid_persist);
            hx_df_plan(f.tiles128, f.ksteps / 4, m->grid_persist, tab.data(), &maxp, &maxrun);
            return (size_t)f.tiles128 * maxp * 128;
        };
        size_t need[5] = {128, 128, 128, 128, parts(m->head)};
        for (auto& ly : m->layers) {
            const size_t v4[4] = {parts(ly.qkv), parts(ly.o), parts(ly.gu), parts(ly.down)};
            for (int i = 0; i < 4; i++) if (v4[i] > need[i]) need[i] = v4[i];
        }
        for (int i = 0; i < 5; i++) if ((rc = ll(&m->part_ll[i], need[i]))) return rc;
        if ((rc = dalloc(m, &m->done_cnt, (size_t)4))) return rc;
        HX_CUDA(cudaMemset(m->done_cnt, 0, 16));
        if ((rc = hx_decode_df_prepare())) return rc;
    }
    if (m->tp_world > 1) {
        if ((rc = dalloc(m, &m->x2, (size_t)m->cfg.d_model))) return rc;
        m->tp_buf_floats = (size_t)2 * m->tp_world * m->cfg.d_model + (size_t)4 * m->tp_world + 64;
        if (m->use_df) m->tp_buf_floats *= 2;            // the same layout in 8-byte (value, epoch) pairs
        // behind it: the exchange areas of the batched prefill, two buffers (used in turn) of one slot per rank
        m->tp_buf_floats = (m->tp_buf_floats + 3) & ~(size_t)3;
        m->tp_pf_off = m->tp_buf_floats / 2;                                       // in pairs
        m->tp_pf_area = (size_t)HX_PF_TB * m->cfg.d_model;                         // pairs per slot
        m->tp_buf_floats += (size_t)2 * 2 * m->tp_world * m->tp_pf_area;
        if ((rc = dalloc(m, &m->tp_buf, m->tp_buf_floats))) return rc;
        HX_CUDA(cudaMemset(m->tp_buf, 0, m->tp_buf_floats * 4));
        m->tp_peer[m->tp_rank] = m->tp_buf;
    }
    rc = build_phases(m, false, true, &m->ph_decode, &m->nph_decode); if (rc) return rc;
    rc = build_phases(m, true, false, &m->ph_prefill, &m->nph_prefill); if (rc) return rc;
    if ((rc = dalloc(m, &m->d_bar, (size_t)2))) return rc;
    if ((rc = dalloc(m, &m->d_err, (size_t)4))) return rc;
    HX_CUDA(cudaMemset(m->d_bar, 0, 16));
    HX_CUDA(cudaMemset(m->d_err, 0, 16));
    m->bar_count = 0;
#ifdef HX_DEBUG_STAMPS
    if (getenv("HX_PERSIST_DBG")) { if ((rc = dalloc(m, &m->d_dbg, (size_t)16 * (m->nph_decode + 4) + (size_t)8 * m->nph_decode * m->grid_persist))) return rc; }
#endif
    if (m->use_tc) {
        if ((rc = dalloc(m, &m->tc_partial, m->tc_units_max * 128 + 128))) return rc;
        if ((rc = dalloc(m, &m->tc_cnt, (size_t)m->tc_tiles_max + 8))) return rc;
        HX_CUDA(cudaMemset(m->tc_cnt, 0, ((size_t)m->tc_tiles_max + 8) * 4));
        if (m->use_df) { const int att = hx_decode_df_att_bytes(m->cfg.n_heads / m->cfg.n_kv_heads); if (att > m->bdig_bytes) m->bdig_bytes = att; }
        m->tc_ring = m->use_df ? hx_decode_df_ring(m->bdig_bytes) : hx_persist_tc_ring(m->bdig_bytes);
        if (const char* e = getenv("HX_TC_RING")) { const int r = atoi(e); if (r >= 3 && r < m->tc_ring) m->tc_ring = r; }
        if (m->tc_ring < 3)
            return hx_fail(HX_ERR_ARG, "tensor-core decode: K too large for shared memory (%zu bytes besides the ring)", hx_persist_tc_smem(m->bdig_bytes));
    } else if (hx_persist_smem(m->dig_bytes) > 227 * 1024)
        return hx_fail(HX_ERR_ARG, "persistent decode: K too large for shared memory (%zu bytes)", hx_persist_smem(m->dig_bytes));
    return HX_OK;
}

// One token through the persistent kernel.
int persist_step(hx_model* m, bool from_prompt, bool with_head) {
    HxPersist P = {};
    P.phases = from_prompt ? m->ph_prefill : m->ph_decode;
    P.nphases = from_prompt ? m->nph_prefill : m->nph_decode;
    (void)with_head;
    P.pos = m->d_pos; P.bar = m->d_bar; P.bar_base = m->bar_count; P.err = m->d_err;
    P.part_m = m->part_m; P.part_l = m->part_l; P.part_acc = m->part_acc; P.part_amax = m->part_amax; P.attn_cnt = m->attn_cnt;
    P.am_val = m->am_val; P.am_idx = m->am_idx; P.am_cnt = m->am_cnt; P.next_tok = m->d_tok; P.pos_inc = m->d_pos;
    P.hist = m->d_hist; P.logits = m->logits; P.dig_bytes = m->dig_bytes;
    P.tok_by_pos = from_prompt ? 1 : 0; P.advance_pos = from_prompt ? 1 : 0;
#ifdef HX_DEBUG_STAMPS
    P.dbg = m->d_dbg; P.dbg_all = m->d_dbg ? m->d_dbg + (size_t)16 * (m->nph_decode + 4) : nullptr; { const char* dc = getenv("HX_PERSIST_DBG"); P.dbg_cta = dc ? atoi(dc) - 1 : 0; if (P.dbg_cta < 0) P.dbg_cta = 0; }
#endif
    P.tc_partial = m->tc_partial; P.tc_cnt = m->tc_cnt; P.bdig_bytes = m->bdig_bytes; P.tc_ring = m->tc_ring;
    P.tp_world = m->tp_world; P.tp_rank = m->tp_rank; P.tp_dm = m->cfg.d_model; P.tp_vocab_off = m->tp_rank * m->cfg.vocab;
    if (m->tp_world > 1) {
        if (!m->tp_connected) return hx_fail(HX_ERR_STATE, "tensor parallel: call hx_model_tp_connect before the first step");
        for (int w = 0; w < m->tp_world; w++) P.tp_peer[w] = m->tp_peer[w];
        P.tp_epoch_base = m->tp_launches * 4096u;        // every rank launches the same sequence of steps
    }
    if (m->use_df) {
        if (m->ep_count > 0xFFF00000u) return hx_fail(HX_ERR_STATE, "epoch counter of the decode engine exhausted: rebuild the model");
        P.ep_base = m->ep_count;
        P.wait_limit = m->wait_limit; P.inject_stall = m->inject_stall; P.done_cnt = m->done_cnt;
        P.att_nkv = m->cfg.n_kv_heads; P.att_nsplit = m->nsplit_persist; P.att_dh = m->cfg.head_dim;
        for (int w = 0; w < m->tp_world; w++) P.tp_x[w] = reinterpret_cast<unsigned long long*>(m->tp_peer[w]);
        const int rc = hx_decode_df_launch(P, m->grid_persist, m->st);
        if (rc == HX_OK) m->ep_count += (unsigned)P.nphases + 2u;      // the counters move only with a launch that ran
        return rc;
    }
    const int rc = m->use_tc ? hx_persist_tc_launch(P, m->grid_persist, m->st) : hx_persist_launch(P, m->grid_persist, m->st);
    if (rc == HX_OK) {
        m->bar_count += (unsigned long long)m->grid_persist * (unsigned long long)(P.nphases - 1);
        if (m->tp_world > 1) m->tp_launches++;
    }
    return rc;
}

// Before the synchronize that ends a step: the two error words travel with the step's results, so that looking at
// them afterwards costs no round trip of its own.
static void flags_enqueue(hx_model* m) {
    if (!m->h_flags && cudaMallocHost((void**)&m->h_flags, 16) != cudaSuccess) { (void)cudaGetLastError(); m->h_flags = nullptr; return; }
    m->h_flags[0] = m->h_flags[1] = 0;
    if (m->pf_err) cudaMemcpyAsync(&m->h_flags[0], m->pf_err, 4, cudaMemcpyDeviceToHost, m->st);
    if (m->persist) cudaMemcpyAsync(&m->h_flags[1], m->d_err, 4, cudaMemcpyDeviceToHost, m->st);
    m->h_flags[2] = 1;       // fetched: valid after the next synchronize of the stream
}

// After a synchronize: did any bounded wait of the persistent kernel run out?
int persist_check(hx_model* m) {
    const bool fetched = m->h_flags && m->h_flags[2] == 1;
    if (fetched) m->h_flags[2] = 0;
    if (fetched && !m->h_flags[0] && !m->h_flags[1]) return HX_OK;
    if (m->pf_err) {
        int pe = 0;
        HX_CUDA(cudaMemcpy(&pe, m->pf_err, 4, cudaMemcpyDeviceToHost));
        if (pe) { cudaMemset(m->pf_err, 0, 4); return hx_fail(HX_ERR_TIMEOUT, "a bounded wait in the prefill GEMM ran out"); }
    }
    if (!m->persist) return HX_OK;
    int e = 0;
    HX_CUDA(cudaMemcpy(&e, m->d_err, 4, cudaMemcpyDeviceToHost));
    if (e) {
        // every counter a launch leaves behind goes back to its idle value, so the next step starts clean (the pair
        // buffers need nothing: epochs only grow)
        cudaMemset(m->d_err, 0, 16); cudaMemset(m->d_bar, 0, 8); m->bar_count = 0;
        cudaMemset(m->am_cnt, 0, 16); cudaMemset(m->attn_cnt, 0, (size_t)m->cfg.n_kv_heads * 4);
        if (m->tc_cnt) cudaMemset(m->tc_cnt, 0, ((size_t)m->tc_tiles_max + 8) * 4);
        if (m->done_cnt) cudaMemset(m->done_cnt, 0, 16);
        return hx_fail(HX_ERR_TIMEOUT, "a bounded wait in the persistent decode kernel ran out");
    }
    return HX_OK;
}

int finish_init(hx_model* m) {
    int rc = alloc_state(m); if (rc) return rc;
    const char* np = getenv("HX_NO_PDL");
    m->pdl = !(np && *np == '1');
    if (m->persist) {
        rc = init_persist(m);
        if (rc) return rc;
    }
    if (m->persist) return HX_OK;               // the per-op launch graphs belong to the graph engine alone
    rc = capture(m, false, true, &m->g_decode);
    if (rc && m->pdl) {     // programmatic edges not capturable on this driver: plain stream order
        m->pdl = false;
        rc = capture(m, false, true, &m->g_decode);
    }
    if (rc) return rc;
    return capture(m, true, false, &m->g_prefill);
}

// One decode / prefill token on the model's stream, whichever engine is selected.
int step_decode(hx_model* m) {
    if (m->persist) return persist_step(m, false, true);
    HX_CUDA(cudaGraphLaunch(m->g_decode, m->st));
    HX_COUNT_LAUNCH(kernels_per_step(m, true));
    return HX_OK;
}
int step_prefill(hx_model* m) {
    if (m->persist) return persist_step(m, true, false);
    HX_CUDA(cudaGraphLaunch(m->g_prefill, m->st));
    HX_COUNT_LAUNCH(kernels_per_step(m, false));
    return HX_OK;
}

int check_cfg(const hx_config& c, int kv_cap, int batch, int tp_rank, int tp_size) {
    if (c.arch != 1) return hx_fail(HX_ERR_ARG, "arch %d: only the Llama/Qwen3 family (1) is built", c.arch);
    if (c.n_layers <= 0 || c.d_model <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.head_dim <= 0 || c.d_ff <= 0 || c.vocab <= 0)
        return hx_fail(HX_ERR_ARG, "non-positive model dimension");
    if (c.n_heads % c.n_kv_heads) return hx_fail(HX_ERR_ARG, "n_heads %d not a multiple of n_kv_heads %d", c.n_heads, c.n_kv_heads);
    if (c.head_dim % 32 || c.head_dim > 256) return hx_fail(HX_ERR_ARG, "head_dim %d: need a multiple of 32 up to 256", c.head_dim);
    if (c.d_model % 4 || c.d_ff % 4) return hx_fail(HX_ERR_ARG, "d_model and d_ff must be multiples of 4");
    if (kv_cap <= 0) return hx_fail(HX_ERR_ARG, "kv_cap must be positive");
    if (batch < 1 || batch > 1024) return hx_fail(HX_ERR_ARG, "batch %d: 1 .. 1024 sequences per model instance", batch);
    if (tp_size < 1 || tp_size > 8 || tp_rank < 0 || tp_rank >= tp_size) return hx_fail(HX_ERR_ARG, "tensor parallel rank %d of %d", tp_rank, tp_size);
    if (tp_size > 1) {
        if (c.n_heads % tp_size || c.n_kv_heads % tp_size || c.d_ff % tp_size || c.vocab % tp_size)
            return hx_fail(HX_ERR_ARG, "tensor parallel %d: heads %d, kv heads %d, d_ff %d and vocab %d must be divisible", tp_size, c.n_heads, c.n_kv_heads, c.d_ff, c.vocab);
        if ((c.n_heads / tp_size * c.head_dim) % 16 || (c.d_ff / tp_size) % 16) return hx_fail(HX_ERR_ARG, "tensor parallel %d: shard widths must be multiples of 16", tp_size);
    }
    return HX_OK;
}

}  // namespace

HX_API int hx_model_free(hx_model* m) {
    if (!m) return HX_OK;
    if (m->g_decode) cudaGraphExecDestroy(m->g_decode);
    if (m->g_prefill) cudaGraphExecDestroy(m->g_prefill);
    if (m->g_pf_chunk) cudaGraphExecDestroy(m->g_pf_chunk);
    if (m->g_bstep) cudaGraphExecDestroy(m->g_bstep);
    if (m->ev0) cudaEventDestroy(m->ev0);
    if (m->ev1) cudaEventDestroy(m->ev1);
    for (int w = 0; w < 8; w++)                      // mappings of the peers' exchange buffers
        if (m->tp_peer[w] && w != m->tp_rank) cudaIpcCloseMemHandle(m->tp_peer[w]);
    for (void* p : m->allocs) cudaFree(p);
    if (m->h_flags) cudaFreeHost(m->h_flags);
    for (cudaEvent_t e : m->prof_ev) cudaEventDestroy(e);
    if (m->st) cudaStreamDestroy(m->st);
    delete m;
    return HX_OK;
}

HX_API int hx_model_synth(hx_model** out, const hx_config* cfg, uint64_t seed, int kv_cap, int batch,
                          int flags, int tp_rank, int tp_size) {
    HX_CHECK_ARG(out && cfg);
    int rc = check_cfg(*cfg, kv_cap, batch, tp_rank, tp_size); if (rc) return rc;
    hx_model* m = new hx_model();
        m->gcfg = *cfg; m->cfg = *cfg; m->tp_rank = tp_rank; m->tp_world = tp_size;
        if (tp_size > 1) { m->cfg.n_heads /= tp_size; m->cfg.n_kv_heads /= tp_size; m->cfg.d_ff /= tp_size; m->cfg.vocab /= tp_size; }
        m->QD = m->cfg.n_heads * m->cfg.head_dim; m->KVD = m->cfg.n_kv_heads * m->cfg.head_dim;
    m->kv_cap = kv_cap; m->batch = batch; m->flags = flags;
    { const char* dm = getenv("HX_DECODE"); const char* lm = getenv("HX_LINEAR");
      m->persist = !(dm && strcmp(dm, "graph") == 0);
      m->use_tc = m->persist && !(lm && strcmp(lm, "mma") == 0);
      m->want_t128 = m->use_tc;
      { const char* pf = getenv("HX_PREFILL"); m->pf_batched = !(pf && strcmp(pf, "token") == 0); }
      if (m->tp_world > 1) { m->persist = true; m->use_tc = true; m->want_t128 = true; } }
    cudaError_t e = cudaStreamCreateWithFlags(&m->st, cudaStreamNonBlocking);
    if (e != cudaSuccess) { delete m; return hx_fail(HX_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e)); }
    Source s; s.synth = true; s.seed = seed;
    rc = build(m, s);
    if (!rc) rc = finish_init(m);
    if (rc) { hx_model_free(m); return rc; }
    *out = m;
    return HX_OK;
}

// ---- GPT-2 (12 layers, d 768: the GPT-2-124M configuration) ---------------------------------------------
// The reference has no NVFP4 container for GPT-2 (its v3 packer matches Llama/Qwen3 tensor names only), so the
// weights come as host f32 arrays, every linear as [out][in] (the transpose of the Conv1D storage, so that the
// 16-element blocks run along K); the library quantizes them with the bit-exact quantizer.
static int gpt2_upload(hx_model* m, float** dst, const float* src, size_t n) {
    int rc = dalloc(m, dst, n); if (rc) return rc;
    HX_CUDA(cudaMemcpyAsync(*dst, src, n * 4, cudaMemcpyHostToDevice, m->st));
    return HX_OK;
}
static int gpt2_linear(hx_model* m, Fused& f, const float* w_host, int N, int K, float* stage, int32_t* wtmp, uint8_t* mtmp, float* tstmp) {
    int rc = alloc_fused(m, f, N, K); if (rc) return rc;
    HX_CUDA(cudaMemcpyAsync(stage, w_host, (size_t)N * K * 4, cudaMemcpyHostToDevice, m->st));
    if ((rc = hx_quantize_nvfp4(stage, N, K, wtmp, mtmp, nullptr, tstmp, m->st))) return rc;
    Committed c; c.rows = N; c.K = K; c.Kpad = hx_kpad(K); c.words = wtmp; c.micro = mtmp;
    HX_CUDA(cudaMemcpyAsync(&c.ts, tstmp, 4, cudaMemcpyDeviceToHost, m->st));
    HX_CUDA(cudaStreamSynchronize(m->st));
    put_rows(m, c, f, 1, 0);
    f.ts[0] = f.ts[1] = f.ts[2] = c.ts; f.bound0 = f.bound1 = N;
    HX_CUDA(cudaStreamSynchronize(m->st));
    return HX_OK;
}

HX_API int hx_model_gpt2(hx_model** out, const hx_config* cfg, const hx_gpt2_weights* w, int kv_cap) {
    HX_CHECK_ARG(out && cfg && w && w->wte && w->wpe && w->lnf_g && w->lnf_b && w->layers);
    const hx_config& c = *cfg;
    if (c.arch != 0) return hx_fail(HX_ERR_ARG, "hx_model_gpt2 builds arch 0 (GPT-2), got %d", c.arch);
    if (c.n_layers <= 0 || c.d_model <= 0 || c.n_heads <= 0 || c.d_ff <= 0 || c.vocab <= 0 || c.max_ctx <= 0)
        return hx_fail(HX_ERR_ARG, "non-positive model dimension");
    if (c.d_model % c.n_heads || c.head_dim != c.d_model / c.n_heads || c.n_kv_heads != c.n_heads)
        return hx_fail(HX_ERR_ARG, "GPT-2: head_dim must be d_model / n_heads and n_kv_heads == n_heads");
    if (c.head_dim % 32 || c.head_dim > 256 || c.d_model % 4 || c.d_ff % 4) return hx_fail(HX_ERR_ARG, "GPT-2: head_dim multiple of 32 (<= 256), widths multiples of 4");
    if (kv_cap <= 0 || kv_cap > c.max_ctx) return hx_fail(HX_ERR_ARG, "kv_cap %d outside 1..max_ctx %d", kv_cap, c.max_ctx);
    hx_model* m = new hx_model();
    m->cfg = c; m->gcfg = c; m->cfg.qk_norm = 0; m->QD = c.d_model; m->KVD = c.d_model;
    m->kv_cap = kv_cap; m->batch = 1; m->flags = 0;
    m->persist = false; m->use_tc = false; m->want_t128 = false; m->pf_batched = false;     // per-op kernels in one CUDA graph
    int rc = HX_OK;
    float* stage = nullptr; int32_t* wtmp = nullptr; uint8_t* mtmp = nullptr; float* tstmp = nullptr;
    do {
        cudaError_t e = cudaStreamCreateWithFlags(&m->st, cudaStreamNonBlocking);
        if (e != cudaSuccess) { rc = hx_fail(HX_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e)); break; }
        const int DM = c.d_model, DFF = c.d_ff, NV = c.vocab;
        size_t maxel = (size_t)NV * DM; if ((size_t)3 * DM * DM > maxel) maxel = (size_t)3 * DM * DM; if ((size_t)DFF * DM > maxel) maxel = (size_t)DFF * DM;
        const int kp = hx_kpad(DM > DFF ? DM : DFF);
        size_t maxrows = (size_t)NV; if ((size_t)3 * DM > maxrows) maxrows = 3 * DM; if ((size_t)DFF > maxrows) maxrows = DFF;
        if (cudaMalloc(&stage, maxel * 4) != cudaSuccess || cudaMalloc(&wtmp, maxrows * (kp / 7) * 4) != cudaSuccess ||
            cudaMalloc(&mtmp, maxrows * (kp / 16)) != cudaSuccess || cudaMalloc(&tstmp, 256) != cudaSuccess) { rc = hx_fail(HX_ERR_NOMEM, "GPT-2 staging"); break; }
        m->layers.resize(c.n_layers);
        for (int L = 0; L < c.n_layers && !rc; L++) {
            Layer& ly = m->layers[L]; const hx_gpt2_layer& hl = w->layers[L];
            if (!hl.ln1_g || !hl.ln1_b || !hl.w_qkv || !hl.b_qkv || !hl.w_proj || !hl.b_proj || !hl.ln2_g || !hl.ln2_b || !hl.w_fc || !hl.b_fc || !hl.w_proj2 || !hl.b_proj2) {
                rc = hx_fail(HX_ERR_ARG, "GPT-2 layer %d: null tensor", L); break; }
            if ((rc = gpt2_upload(m, &ly.in_g, hl.ln1_g, DM)) || (rc = gpt2_upload(m, &ly.ln1_b, hl.ln1_b, DM)) ||
                (rc = gpt2_upload(m, &ly.post_g, hl.ln2_g, DM)) || (rc = gpt2_upload(m, &ly.ln2_b, hl.ln2_b, DM)) ||
                (rc = gpt2_upload(m, &ly.b_qkv, hl.b_qkv, (size_t)3 * DM)) || (rc = gpt2_upload(m, &ly.b_o, hl.b_proj, DM)) ||
                (rc = gpt2_upload(m, &ly.b_fc, hl.b_fc, DFF)) || (rc = gpt2_upload(m, &ly.b_down, hl.b_proj2, DM))) break;
            if ((rc = gpt2_linear(m, ly.qkv, hl.w_qkv, 3 * DM, DM, stage, wtmp, mtmp, tstmp))) break;
            if ((rc = gpt2_linear(m, ly.o, hl.w_proj, DM, DM, stage, wtmp, mtmp, tstmp))) break;
            if ((rc = gpt2_linear(m, ly.gu, hl.w_fc, DFF, DM, stage, wtmp, mtmp, tstmp))) break;
            if ((rc = gpt2_linear(m, ly.down, hl.w_proj2, DM, DFF, stage, wtmp, mtmp, tstmp))) break;
        }
        if (rc) break;
        if ((rc = gpt2_upload(m, &m->emb, w->wte, (size_t)NV * DM)) || (rc = gpt2_upload(m, &m->wpe, w->wpe, (size_t)c.max_ctx * DM)) ||
            (rc = gpt2_upload(m, &m->final_g, w->lnf_g, DM)) || (rc = gpt2_upload(m, &m->final_b, w->lnf_b, DM))) break;
        if ((rc = gpt2_linear(m, m->head, w->wte, NV, DM, stage, wtmp, mtmp, tstmp))) break;       // tied lm_head
        HX_CUDA(cudaStreamSynchronize(m->st));
        rc = finish_init(m);
    } while (0);
    cudaFree(stage); cudaFree(wtmp); cudaFree(mtmp); cudaFree(tstmp);
    if (rc) { hx_model_free(m); return rc; }
    *out = m;
    return HX_OK;
}

HX_API int hx_model_load(hx_model** out, const char* path, int kv_cap, int batch, int flags,
                         int tp_rank, int tp_size) {
    HX_CHECK_ARG(out && path);
    int fd = open(path, O_RDONLY);
    if (fd < 0) return hx_fail(HX_ERR_IO, "cannot open %s", path);
    struct stat stt;
    if (fstat(fd, &stt) || stt.st_size < 64) { close(fd); return hx_fail(HX_ERR_FORMAT, "%s: too short for an HXGW header", path); }
    void* mp = mmap(nullptr, (size_t)stt.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (mp == MAP_FAILED) { close(fd); return hx_fail(HX_ERR_IO, "mmap %s failed", path); }
    const uint8_t* hb = (const uint8_t*)mp;
    const size_t len = (size_t)stt.st_size;
    auto u32 = [&](int off) { uint32_t v; memcpy(&v, hb + off, 4); return v; };
    auto f32 = [&](int off) { float v; memcpy(&v, hb + off, 4); return v; };
    int rc = HX_OK;
    hx_model* m = nullptr;
    do {
        if (u32(0) != HXGW_MAGIC) { rc = hx_fail(HX_ERR_FORMAT, "%s: bad magic 0x%08x", path, u32(0)); break; }
        if (u32(4) != 3u) { rc = hx_fail(HX_ERR_FORMAT, "%s: HXGW version %u, need 3", path, u32(4)); break; }
        if (u32(40) != 1u) { rc = hx_fail(HX_ERR_FORMAT, "%s: unknown arch %u", path, u32(40)); break; }
        hx_config c{};
        c.arch = 1; c.n_layers = (int)u32(8); c.d_model = (int)u32(12); c.n_heads = (int)u32(16); c.vocab = (int)u32(20);
        c.max_ctx = (int)u32(24); c.d_ff = (int)u32(28); c.n_kv_heads = (int)u32(44); c.rope_theta = f32(48);
        const float file_eps = f32(52);
        const int hd = (int)u32(56), nt = (int)u32(60);
        if (c.n_heads <= 0) { rc = hx_fail(HX_ERR_FORMAT, "%s: n_heads %d", path, c.n_heads); break; }
        c.head_dim = hd > 0 ? hd : c.d_model / c.n_heads;
        c.qk_norm = 1;
        // the reference's norm kernel bakes 1e-5 and the worker accepts the header's value with a note
        c.norm_eps = (flags & HX_LOAD_FILE_EPS) ? file_eps : 1e-5f;
        if ((rc = check_cfg(c, kv_cap, batch, tp_rank, tp_size))) break;
        if (nt != c.n_layers * T_PER_LAYER + 3) { rc = hx_fail(HX_ERR_FORMAT, "%s: %d tensors, expected %d", path, nt, c.n_layers * T_PER_LAYER + 3); break; }
        // descriptors must tile the file exactly
        uint64_t cur = 64 + (uint64_t)nt * 32;
        if (cur > len) { rc = hx_fail(HX_ERR_FORMAT, "%s: descriptor table past the end of the file", path); break; }
        const V3Desc* d = (const V3Desc*)(hb + 64);
        for (int i = 0; i < nt && !rc; i++) {
            if (d[i].data_off != cur) { rc = hx_fail(HX_ERR_FORMAT, "v3 desc %d data_off %llu != %llu", i, (unsigned long long)d[i].data_off, (unsigned long long)cur); break; }
            if (d[i].packed) {
                if (d[i].Kpad % 112) { rc = hx_fail(HX_ERR_FORMAT, "v3 desc %d Kpad %u not a multiple of 112", i, d[i].Kpad); break; }
                const uint64_t wb = (uint64_t)d[i].rows * (d[i].Kpad / 7) * 4;
                if (d[i].scale_off != cur + wb) { rc = hx_fail(HX_ERR_FORMAT, "v3 desc %d scale_off mismatch", i); break; }
                cur += wb + (uint64_t)d[i].rows * (d[i].Kpad / 16) + 4;
            } else cur += (uint64_t)d[i].rows * d[i].K * 4;
        }
        if (rc) break;
        if (cur != len) { rc = hx_fail(HX_ERR_FORMAT, "v3 layout %llu != file %zu", (unsigned long long)cur, len); break; }
        m = new hx_model();
        m->gcfg = c; m->cfg = c; m->tp_rank = tp_rank; m->tp_world = tp_size;
        if (tp_size > 1) { m->cfg.n_heads /= tp_size; m->cfg.n_kv_heads /= tp_size; m->cfg.d_ff /= tp_size; m->cfg.vocab /= tp_size; }
        m->QD = m->cfg.n_heads * m->cfg.head_dim; m->KVD = m->cfg.n_kv_heads * m->cfg.head_dim;
        m->kv_cap = kv_cap; m->batch = batch; m->flags = flags;
    { const char* dm = getenv("HX_DECODE"); const char* lm = getenv("HX_LINEAR");
      m->persist = !(dm && strcmp(dm, "graph") == 0);
      m->use_tc = m->persist && !(lm && strcmp(lm, "mma") == 0);
      m->want_t128 = m->use_tc;
      { const char* pf = getenv("HX_PREFILL"); m->pf_batched = !(pf && strcmp(pf, "token") == 0); }
      if (m->tp_world > 1) { m->persist = true; m->use_tc = true; m->want_t128 = true; } }
        cudaError_t e = cudaStreamCreateWithFlags(&m->st, cudaStreamNonBlocking);
        if (e != cudaSuccess) { rc = hx_fail(HX_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e)); break; }
        Source s; s.map = hb; s.maplen = len; s.desc = d;
        if ((rc = build(m, s))) break;
        rc = finish_init(m);
    } while (0);
    munmap(mp, len); close(fd);
    if (rc) { if (m) hx_model_free(m); return rc; }
    *out = m;
    return HX_OK;
}

HX_API int hx_model_config(const hx_model* m, hx_config* cfg) { HX_CHECK_ARG(m && cfg); *cfg = m->cfg; return HX_OK; }
HX_API int hx_model_weight_bytes(const hx_model* m, uint64_t* decode_layout, uint64_t* committed_layout) {
    HX_CHECK_ARG(m);
    if (decode_layout) *decode_layout = m->decode_bytes;
    if (committed_layout) *committed_layout = m->committed_bytes;
    return HX_OK;
}
HX_API int hx_model_reset(hx_model* m) { HX_CHECK_ARG(m); m->kv_len = 0; return HX_OK; }
HX_API int hx_model_last_stats(const hx_model* m, hx_step_stats* st) { HX_CHECK_ARG(m && st); *st = m->stats; return HX_OK; }
#ifdef HX_DEBUG_STAMPS
// Debug builds only: per-phase time stamps of one CTA from the last persistent launch (16 per phase, nanoseconds).
HX_API int hx_model_phase_stamps(hx_model* m, unsigned long long* out, int max_phases, int* nphases) {
    HX_CHECK_ARG(m && out && nphases);
    if (!m->d_dbg) return hx_fail(HX_ERR_STATE, "set HX_PERSIST_DBG=1 before creating the model");
    const int n = m->nph_decode < max_phases ? m->nph_decode : max_phases;
    HX_CUDA(cudaMemcpy(out, m->d_dbg, (size_t)n * 16 * 8, cudaMemcpyDeviceToHost));
    *nphases = n;
    return HX_OK;
}
// Debug: the time every CTA finished each phase's work in the last persistent launch: out[phase * grid + cta].
HX_API int hx_model_phase_stamps_all(hx_model* m, unsigned long long* out, size_t max_words, int* nphases, int* grid) {
    HX_CHECK_ARG(m && out && nphases && grid);
    if (!m->d_dbg) return hx_fail(HX_ERR_STATE, "set HX_PERSIST_DBG=1 before creating the model");
    const size_t n = (size_t)8 * m->nph_decode * m->grid_persist;      // eight events per CTA and phase
    HX_CHECK_ARG(n <= max_words);
    HX_CUDA(cudaMemcpy(out, m->d_dbg + (size_t)16 * (m->nph_decode + 4), n * 8, cudaMemcpyDeviceToHost));
    *nphases = m->nph_decode; *grid = m->grid_persist;
    return HX_OK;
}
#endif
// ---- tensor parallel: exchange-buffer handles ----------------------------------------------------------
// The caller moves the 64-byte handles between the ranks' processes by any channel it has.
HX_API int hx_model_tp_handle(hx_model* m, uint8_t handle[64]) {
    HX_CHECK_ARG(m && handle);
    if (m->tp_world < 2 || !m->tp_buf) return hx_fail(HX_ERR_STATE, "not a tensor-parallel shard");
    cudaIpcMemHandle_t h;
    HX_CUDA(cudaIpcGetMemHandle(&h, m->tp_buf));
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle, &h, 64);
    return HX_OK;
}
HX_API int hx_model_tp_connect(hx_model* m, const uint8_t* handles, int world) {
    HX_CHECK_ARG(m && handles);
    if (world != m->tp_world || m->tp_world < 2) return hx_fail(HX_ERR_ARG, "tensor parallel: %d handles for a group of %d", world, m->tp_world);
    if (m->tp_connected) return hx_fail(HX_ERR_STATE, "tensor parallel: the group is already connected");
    if (m->tp_nbar >= 4095) return hx_fail(HX_ERR_ARG, "tensor parallel: too many layers for the barrier numbering");
    for (int w = 0; w < world; w++) {
        if (w == m->tp_rank) continue;
        cudaIpcMemHandle_t h; memcpy(&h, handles + (size_t)w * 64, 64);
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return hx_fail(HX_ERR_COMM, "cudaIpcOpenMemHandle(rank %d): %s", w, cudaGetErrorString(e));
        m->tp_peer[w] = (float*)p;
    }
    m->tp_connected = true;
    return HX_OK;
}

// Which decode engine this model runs: "persistent-tcgen05", "persistent-mma" or "graph".
HX_API const char* hx_model_engine(const hx_model* m) {
    if (!m) return "";
    if (!m->persist) return "graph";
    if (m->use_df) return "persistent-tcgen05-dataflow";
    return m->use_tc ? "persistent-tcgen05" : "persistent-mma";
}
// Test hook of the bounded waits: polls before a device-side wait gives up (0 = the default) and, with
// inject_stall != 0, a wait at the start of every launch on a word that nothing writes.
HX_API int hx_model_debug_waits(hx_model* m, unsigned wait_limit, int inject_stall) {
    HX_CHECK_ARG(m);
    m->wait_limit = wait_limit ? wait_limit : (1u << 24);
    m->inject_stall = inject_stall;
    return HX_OK;
}
HX_API int hx_model_set_profile(hx_model* m, int on) { HX_CHECK_ARG(m); m->profile = on != 0; return HX_OK; }

// ---- HXGW v3 image ---------------------------------------------------------------------------------
namespace {
struct ImgEntry { bool packed; const Committed* c; const float* dense; size_t n; };
int image_plan(const hx_model* m, std::vector<ImgEntry>& ents) {
    if (!(m->flags & HX_LOAD_KEEP_COMMITTED)) return hx_fail(HX_ERR_STATE, "model was built without HX_LOAD_KEEP_COMMITTED");
    const hx_config& c = m->cfg;
    for (int L = 0; L < c.n_layers; L++) {
        const Layer& ly = m->layers[L];
        ents.push_back({false, nullptr, ly.in_g, (size_t)c.d_model});
        ents.push_back({true, &ly.c[T_Q], nullptr, 0});
        ents.push_back({false, nullptr, ly.qn_g, (size_t)c.head_dim});
        ents.push_back({true, &ly.c[T_K], nullptr, 0});
        ents.push_back({false, nullptr, ly.kn_g, (size_t)c.head_dim});
        ents.push_back({true, &ly.c[T_V], nullptr, 0});
        ents.push_back({true, &ly.c[T_O], nullptr, 0});
        ents.push_back({false, nullptr, ly.post_g, (size_t)c.d_model});
        ents.push_back({true, &ly.c[T_GATE], nullptr, 0});
        ents.push_back({true, &ly.c[T_UP], nullptr, 0});
        ents.push_back({true, &ly.c[T_DOWN], nullptr, 0});
    }
    ents.push_back({false, nullptr, m->emb, (size_t)c.vocab * c.d_model});
    ents.push_back({false, nullptr, m->final_g, (size_t)c.d_model});
    ents.push_back({true, &m->head_c, nullptr, 0});
    return HX_OK;
}
uint64_t entry_bytes(const ImgEntry& e) {
    if (!e.packed) return (uint64_t)e.n * 4;
    return (uint64_t)e.c->rows * (e.c->Kpad / 7) * 4 + (uint64_t)e.c->rows * (e.c->Kpad / 16) + 4;
}
}  // namespace

HX_API int hx_model_v3_size(const hx_model* m, uint64_t* bytes) {
    HX_CHECK_ARG(m && bytes);
    std::vector<ImgEntry> ents; int rc = image_plan(m, ents); if (rc) return rc;
    uint64_t cur = 64 + 32 * (uint64_t)ents.size();
    for (auto& e : ents) cur += entry_bytes(e);
    *bytes = cur;
    return HX_OK;
}

HX_API int hx_model_v3_export(const hx_model* m, void* host_buf, uint64_t bytes) {
    HX_CHECK_ARG(m && host_buf);
    std::vector<ImgEntry> ents; int rc = image_plan(m, ents); if (rc) return rc;
    uint64_t need = 0; hx_model_v3_size(m, &need);
    if (bytes < need) return hx_fail(HX_ERR_ARG, "buffer of %llu bytes, image needs %llu", (unsigned long long)bytes, (unsigned long long)need);
    uint8_t* o = (uint8_t*)host_buf;
    const hx_config& c = m->cfg;
    memset(o, 0, 64);
    const uint32_t h32[8] = {HXGW_MAGIC, 3u, (uint32_t)c.n_layers, (uint32_t)c.d_model, (uint32_t)c.n_heads, (uint32_t)c.vocab,
                             (uint32_t)c.max_ctx, (uint32_t)c.d_ff};
    memcpy(o, h32, 32);
    const uint32_t arch = 1u, nkv = (uint32_t)c.n_kv_heads, hd = (uint32_t)c.head_dim, nt = (uint32_t)ents.size();
    const float eps_hdr = 1e-6f;    // what a Qwen3 config states; the kernels use cfg.norm_eps
    memcpy(o + 40, &arch, 4); memcpy(o + 44, &nkv, 4); memcpy(o + 48, &c.rope_theta, 4); memcpy(o + 52, &eps_hdr, 4);
    memcpy(o + 56, &hd, 4); memcpy(o + 60, &nt, 4);
    V3Desc* d = (V3Desc*)(o + 64);
    uint64_t cur = 64 + 32 * (uint64_t)ents.size();
    for (size_t i = 0; i < ents.size(); i++) {
        const ImgEntry& e = ents[i];
        if (e.packed) {
            const uint64_t wb = (uint64_t)e.c->rows * (e.c->Kpad / 7) * 4, mb = (uint64_t)e.c->rows * (e.c->Kpad / 16);
            d[i] = {1u, (uint32_t)e.c->rows, (uint32_t)e.c->K, (uint32_t)e.c->Kpad, cur, cur + wb};
            HX_CUDA(cudaMemcpy(o + cur, e.c->words, wb, cudaMemcpyDeviceToHost));
            HX_CUDA(cudaMemcpy(o + cur + wb, e.c->micro, mb, cudaMemcpyDeviceToHost));
            memcpy(o + cur + wb + mb, &e.c->ts, 4);
        } else {
            d[i] = {0u, 1u, (uint32_t)e.n, (uint32_t)e.n, cur, 0};
            HX_CUDA(cudaMemcpy(o + cur, e.dense, e.n * 4, cudaMemcpyDeviceToHost));
        }
        cur += entry_bytes(e);
    }
    return HX_OK;
}

HX_API int hx_model_v3_save(const hx_model* m, const char* path) {
    HX_CHECK_ARG(m && path);
    uint64_t n = 0; int rc = hx_model_v3_size(m, &n); if (rc) return rc;
    void* buf = malloc(n);
    if (!buf) return hx_fail(HX_ERR_NOMEM, "malloc(%llu)", (unsigned long long)n);
    rc = hx_model_v3_export(m, buf, n);
    if (!rc) {
        FILE* f = fopen(path, "wb");
        if (!f) rc = hx_fail(HX_ERR_IO, "cannot write %s", path);
        else { if (fwrite(buf, 1, n, f) != n) rc = hx_fail(HX_ERR_IO, "short write %s", path); fclose(f); }
    }
    free(buf);
    return rc;
}

HX_API int hx_model_sha256(const hx_model* m, char hex[65]) {
    HX_CHECK_ARG(m && hex);
    uint64_t n = 0; int rc = hx_model_v3_size(m, &n); if (rc) return rc;
    void* buf = malloc(n);
    if (!buf) return hx_fail(HX_ERR_NOMEM, "malloc(%llu)", (unsigned long long)n);
    rc = hx_model_v3_export(m, buf, n);
    if (!rc) rc = hx_sha256_hex(buf, n, hex);
    free(buf);
    return rc;
}

// ---- stepping ------------------------------------------------------------------------------------
static int set_pos_tok(hx_model* m, int pos, const int32_t* tok) {
    HX_CUDA(cudaMemcpyAsync(m->d_pos, &pos, 4, cudaMemcpyHostToDevice, m->st));
    if (tok) HX_CUDA(cudaMemcpyAsync(m->d_tok, tok, 4, cudaMemcpyHostToDevice, m->st));
    return HX_OK;
}

HX_API int hx_decode_step(hx_model* m, const int32_t* ids, int pos, int32_t* next_ids, float* logits) {
    HX_CHECK_ARG(m && ids);
    if (pos < 0 || pos >= m->kv_cap) return hx_fail(HX_ERR_STATE, "position %d outside the KV capacity %d", pos, m->kv_cap);
    if (ids[0] < 0 || ids[0] >= m->gcfg.vocab) return hx_fail(HX_ERR_ARG, "token %d outside the vocabulary", ids[0]);
    int rc = set_pos_tok(m, pos, ids); if (rc) return rc;
    if ((rc = step_decode(m))) return rc;
    if (next_ids) HX_CUDA(cudaMemcpyAsync(next_ids, m->d_tok, 4, cudaMemcpyDeviceToHost, m->st));
    if (logits) HX_CUDA(cudaMemcpyAsync(logits, m->logits, (size_t)m->cfg.vocab * 4, cudaMemcpyDeviceToHost, m->st));
    flags_enqueue(m);
    HX_CUDA(cudaStreamSynchronize(m->st));
    if ((rc = persist_check(m))) return rc;
    m->kv_len = pos + 1;
    return HX_OK;
}

// ---- batched prefill ---------------------------------------------------------------------------------
static_assert(HX_PF_TB <= HX_TC_MAX_GROUPS * HX_TC_MAX_TOK && HX_PF_TB <= HX_TC_NTOK, "a chunk fits the token groups of the GEMM");
// K pieces of a linear in the chunk GEMM: pieces small enough for their digit cells to stay in shared memory, and
// with few row tiles enough of them for about one unit per SM.
static int pf_pieces(const Fused& f) {
    const int kcells = f.ksteps / 4;
    int P = (kcells + HX_TC_RES_CELLS - 1) / HX_TC_RES_CELLS;
    if (2 * f.tiles128 <= 148) {
        int q = 148 / f.tiles128; if (q > kcells) q = kcells;
        if (q > 148 / HX_TC_MAX_GROUPS) q = 148 / HX_TC_MAX_GROUPS;      // pieces x token groups is the least grid
        if (q > P) P = q;
    }
    return P < 1 ? 1 : P;
}

static int pf_alloc(hx_model* m) {
    if (m->pf_x) return HX_OK;
    { const int prc = hx_gemm_tc_prepare(); if (prc) return prc; }
    const hx_config& c = m->cfg;
    int maxK = c.d_model > m->QD ? c.d_model : m->QD; if (c.d_ff > maxK) maxK = c.d_ff;
    const size_t cells = (size_t)((maxK + 255) / 256) * HX_TC_MAX_GROUPS * (HX_TC_GROUP_COLS * 128);
    m->pf_gu_ld = m->layers.empty() ? 64 : m->layers[0].gu.tiles128 * 64;      // hidden size rounded up to whole tiles
    int rc;
    if ((rc = dalloc(m, &m->pf_x, (size_t)HX_PF_TB * c.d_model))) return rc;
    if ((rc = dalloc(m, &m->pf_qkv, (size_t)HX_PF_TB * (m->QD + 2 * m->KVD)))) return rc;
    if ((rc = dalloc(m, &m->pf_ctx, (size_t)HX_PF_TB * m->QD))) return rc;
    if ((rc = dalloc(m, &m->pf_gu, (size_t)HX_PF_TB * m->pf_gu_ld))) return rc;
    if ((rc = dalloc(m, &m->pf_scale, (size_t)HX_PF_TB))) return rc;
    if ((rc = dalloc(m, &m->pf_cells, cells))) return rc;
    if (m->tp_world > 1 && (rc = dalloc(m, &m->pf_part, (size_t)HX_PF_TB * c.d_model))) return rc;
    if ((rc = dalloc(m, &m->pf_err, (size_t)4))) return rc;
    if ((rc = dalloc(m, &m->d_pf_pos, (size_t)4))) return rc;
    if ((rc = dalloc(m, &m->pf_att_part, hx_pf_attn_scratch(HX_PF_TB, c.n_heads, c.n_kv_heads, c.head_dim)))) return rc;
    if ((rc = dalloc(m, &m->pf_att_tickets, (size_t)HX_PF_TB * c.n_kv_heads))) return rc;
    HX_CUDA(cudaMemsetAsync(m->pf_att_tickets, 0, (size_t)HX_PF_TB * c.n_kv_heads * 4, m->st));
    HX_CUDA(cudaMemsetAsync(m->pf_err, 0, 16, m->st));
    {   // partial sums [tile][piece][token][128] of the most demanding linear, tickets per tile
        size_t need = 0; int maxt = m->head.tiles128;
        auto acc = [&](const Fused& f) { const size_t v = (size_t)f.tiles128 * pf_pieces(f) * HX_PF_TB * 128; if (v > need) need = v; if (f.tiles128 > maxt) maxt = f.tiles128; };
        for (auto& ly : m->layers) { acc(ly.qkv); acc(ly.o); acc(ly.gu); acc(ly.down); }
        acc(m->head);
        m->pf_partial_n = need;
        if ((rc = dalloc(m, &m->pf_partial, need))) return rc;
        const size_t ntk = (size_t)maxt * HX_TC_MAX_GROUPS + 8;
        if ((rc = dalloc(m, &m->pf_tickets, ntk))) return rc;
        HX_CUDA(cudaMemsetAsync(m->pf_tickets, 0, ntk * 4, m->st));
    }
    return HX_OK;
}

// one linear of a chunk: digits of `src` -> GEMM against f -> out (token-major)
static int pf_linear(hx_model* m, const Fused& f, const float* src, int ld_src, int n, int swiglu, const float* g,
                     float* out, int ld_out, int rows, int resid, int pair64) {
    hx_pf_digits(src, ld_src, n, f.K, 0, g, m->cfg.norm_eps, m->pf_cells, m->pf_scale, m->st);
    HxGemmTC q = {};
    q.a = f.t128; q.b = m->pf_cells; q.rows = rows; q.ntiles = f.tiles128; q.ksteps = f.ksteps; q.ntok = n; q.stage_ksteps = 4;
    q.err = m->pf_err; q.digit_mode = 1; q.col_scale = m->pf_scale; q.out = out; q.ld_out = ld_out; q.resid = resid;
    q.ts[0] = f.ts[0]; q.ts[1] = f.ts[1]; q.ts[2] = f.ts[2]; q.bound0 = f.bound0; q.bound1 = f.bound1; q.pair64 = pair64; q.swiglu = swiglu;
    const int P = pf_pieces(f);
    if (P > 148) return hx_fail(HX_ERR_ARG, "prefill: %d input columns are more than the chunk GEMM cuts into pieces", f.K);
    q.ksplit = P; q.partial = m->pf_partial; q.tickets = m->pf_tickets; q.b_resident = 1;
    if ((size_t)f.tiles128 * P * HX_PF_TB * 128 > m->pf_partial_n) return hx_fail(HX_ERR_ARG, "prefill: partial-sum buffer too small");
    return hx_gemm_tc_launch(q, m->st);
}

// Tensor-parallel shard: pf_part (this rank's partial rows of a row-split linear for the n tokens of the chunk) summed over
// the ranks into pf_x.  Every rank issues the same sequence of exchanges, so the epoch and the buffer (two, in turn: a
// rank cannot be two exchanges ahead of a peer it has to read from) agree without any negotiation.
static int pf_tp_reduce(hx_model* m, int n) {
    if (!m->tp_connected) return hx_fail(HX_ERR_STATE, "tensor parallel: call hx_model_tp_connect before the first step");
    if (m->tp_pf_ep > 0xFFFFFF00u) return hx_fail(HX_ERR_STATE, "epoch counter of the prefill exchange exhausted: rebuild the model");
    const unsigned ep = ++m->tp_pf_ep;
    unsigned long long* areas[8] = {nullptr};
    for (int w = 0; w < m->tp_world; w++)
        areas[w] = reinterpret_cast<unsigned long long*>(m->tp_peer[w]) + m->tp_pf_off + (size_t)(ep & 1u) * m->tp_world * m->tp_pf_area;
    hx_pf_tp_reduce(m->pf_part, m->pf_x, areas, m->tp_rank, m->tp_world, n * m->cfg.d_model, m->tp_pf_area, ep, m->wait_limit, m->pf_err, m->st);
    return HX_OK;
}

// The launches of the layers for one chunk of n tokens (ids[t] / wh say which token, position and sequence each is).
static int pf_enqueue_layers(hx_model* m, int n, const int* ids, HxPfWhere wh) {
    const hx_config& c = m->cfg;
    const int DH = c.head_dim, DM = c.d_model, QD = m->QD, KVD = m->KVD, cap = m->kv_cap;
    const int ldq = QD + 2 * KVD;
    const float att_scale = 1.0f / sqrtf((float)DH);
    int rc;
    hx_pf_embed(ids, wh, m->emb, m->pf_x, n, DM, m->st);
    for (int L = 0; L < c.n_layers; L++) {
        Layer& ly = m->layers[L];
        float* kc = m->kc + (size_t)L * c.n_kv_heads * cap * DH; float* vc = m->vc + (size_t)L * c.n_kv_heads * cap * DH;
        if ((rc = pf_linear(m, ly.qkv, m->pf_x, DM, n, 0, ly.in_g, m->pf_qkv, ldq, ly.qkv.N, 0, 0))) return rc;
        hx_pf_qkpost(m->pf_qkv, ldq, n, wh, c.n_heads, c.n_kv_heads, DH, ly.qn_g, ly.kn_g, c.norm_eps, m->cosT, m->sinT, kc, vc, cap, m->st);
        if ((rc = hx_pf_attn(m->pf_qkv, ldq, n, wh, c.n_heads, c.n_kv_heads, DH, kc, vc, cap, att_scale, m->pf_ctx, QD, m->pf_att_part, m->pf_att_tickets, m->pf_err, m->st))) return rc;
        if (m->tp_world > 1) {
            if ((rc = pf_linear(m, ly.o, m->pf_ctx, QD, n, 0, nullptr, m->pf_part, DM, ly.o.N, 0, 0))) return rc;
            if ((rc = pf_tp_reduce(m, n))) return rc;
        } else if ((rc = pf_linear(m, ly.o, m->pf_ctx, QD, n, 0, nullptr, m->pf_x, DM, ly.o.N, 1, 0))) return rc;
        if ((rc = pf_linear(m, ly.gu, m->pf_x, DM, n, 1, ly.post_g, m->pf_gu, m->pf_gu_ld, c.d_ff, 0, 1))) return rc;       // SwiGLU in the epilogue
        if (m->tp_world > 1) {
            if ((rc = pf_linear(m, ly.down, m->pf_gu, m->pf_gu_ld, n, 0, nullptr, m->pf_part, DM, ly.down.N, 0, 0))) return rc;
            if ((rc = pf_tp_reduce(m, n))) return rc;
        } else if ((rc = pf_linear(m, ly.down, m->pf_gu, m->pf_gu_ld, n, 0, nullptr, m->pf_x, DM, ly.down.N, 1, 0))) return rc;
    }
    return HX_OK;
}

// One prefill chunk of n tokens whose first position is *d_pf_pos; ends by advancing that position.
static int pf_enqueue_chunk(hx_model* m, int n) {
    const hx_config& c = m->cfg;
    HxPfWhere wh = {m->d_pf_pos, nullptr, nullptr, (size_t)c.n_layers * c.n_kv_heads * m->kv_cap * c.head_dim, m->d_pf_pos + 1};
    int rc = pf_enqueue_layers(m, n, m->d_prompt, wh); if (rc) return rc;
    hx_pf_advance(m->d_pf_pos, n, m->st);
    return HX_OK;
}

// ---- batched decode: n_seq independent sequences, one token each, in chunks of HX_PF_TB ----------------
static int bd_alloc(hx_model* m) {
    int rc = pf_alloc(m); if (rc) return rc;
    if (m->d_bids) return HX_OK;
    m->b_cap = ((m->batch + HX_PF_TB - 1) / HX_PF_TB) * HX_PF_TB;
    if ((rc = dalloc(m, &m->d_bids, (size_t)m->b_cap))) return rc;
    if ((rc = dalloc(m, &m->d_bpos, (size_t)m->b_cap))) return rc;
    if ((rc = dalloc(m, &m->d_bseq, (size_t)m->b_cap))) return rc;
    if ((rc = dalloc(m, &m->d_bnext, (size_t)m->b_cap))) return rc;
    if (!m->pf_logits && (rc = dalloc(m, &m->pf_logits, (size_t)HX_PF_TB * m->cfg.vocab))) return rc;
    std::vector<int> seq(m->b_cap);
    for (int i = 0; i < m->b_cap; i++) seq[i] = i;
    HX_CUDA(cudaMemcpy(m->d_bseq, seq.data(), (size_t)m->b_cap * 4, cudaMemcpyHostToDevice));
    return HX_OK;
}

// One decode step of sequences 0..n_seq-1: tokens d_bids, positions d_bpos (advanced by one), next tokens to d_bnext and
// back into d_bids.
static int bd_enqueue_step(hx_model* m, int n_seq) {
    const hx_config& c = m->cfg;
    const size_t seq_stride = (size_t)c.n_layers * c.n_kv_heads * m->kv_cap * c.head_dim;
    int rc;
    for (int c0 = 0; c0 < n_seq; c0 += HX_PF_TB) {
        const int n = n_seq - c0 < HX_PF_TB ? n_seq - c0 : HX_PF_TB;
        HxPfWhere wh = {nullptr, m->d_bpos + c0, m->d_bseq + c0, seq_stride, nullptr};
        if ((rc = pf_enqueue_layers(m, n, m->d_bids + c0, wh))) return rc;
        if ((rc = pf_linear(m, m->head, m->pf_x, c.d_model, n, 0, m->final_g, m->pf_logits, c.vocab, m->head.N, 0, 0))) return rc;
        if (m->tp_world > 1) {
            // every rank holds a slice of the vocabulary: local first maximum, then the best over the ranks
            if (!m->tp_connected) return hx_fail(HX_ERR_STATE, "tensor parallel: call hx_model_tp_connect before the first step");
            const unsigned ep = ++m->tp_pf_ep;
            unsigned long long* areas[8] = {nullptr};
            for (int w = 0; w < m->tp_world; w++)
                areas[w] = reinterpret_cast<unsigned long long*>(m->tp_peer[w]) + m->tp_pf_off + (size_t)(ep & 1u) * m->tp_world * m->tp_pf_area;
            hx_pf_tp_argmax_rows(m->pf_logits, c.vocab, c.vocab, n, m->tp_rank * c.vocab, areas, m->tp_rank, m->tp_world, m->tp_pf_area, ep,
                                 m->wait_limit, m->pf_err, m->d_bnext + c0, m->d_bpos + c0, m->st);
        } else hx_pf_argmax_rows(m->pf_logits, c.vocab, c.vocab, n, m->d_bnext + c0, m->d_bpos + c0, m->st);
    }
    HX_CUDA(cudaMemcpyAsync(m->d_bids, m->d_bnext, (size_t)n_seq * 4, cudaMemcpyDeviceToDevice, m->st));
    return HX_OK;
}

// Prompt positions [0, T) in chunks of HX_PF_TB tokens; ends like the token-by-token path: KV rows written,
// logits of the last position in m->logits, its arg-max in d_tok / d_hist[T], *d_pos = T.
// Full chunks replay one captured CUDA graph (the position lives in device memory); the last, shorter chunk
// and the lm_head are launched directly.
static int run_prefill_batched(hx_model* m, int T, int seq) {
    const hx_config& c = m->cfg;
    int rc = pf_alloc(m); if (rc) return rc;
    const int ps[2] = {0, seq};                      // first position of the chunk, KV slot of the sequence
    HX_CUDA(cudaMemcpyAsync(m->d_pf_pos, ps, 8, cudaMemcpyHostToDevice, m->st));
    const int nfull = T / HX_PF_TB, rem = T - nfull * HX_PF_TB;
    if (nfull > 1 && !m->g_pf_chunk && !m->pf_graph_failed) {
        cudaGraph_t g = nullptr;
        HX_CUDA(cudaStreamBeginCapture(m->st, cudaStreamCaptureModeThreadLocal));
        const unsigned long long before = g_hx_launches;
        rc = pf_enqueue_chunk(m, HX_PF_TB);
        cudaError_t e = cudaStreamEndCapture(m->st, &g);
        g_hx_launches = before;
        if (rc) { if (g) cudaGraphDestroy(g); return rc; }
        if (e == cudaSuccess) e = cudaGraphInstantiate(&m->g_pf_chunk, g, 0);
        if (g) cudaGraphDestroy(g);
        if (e != cudaSuccess) { (void)cudaGetLastError(); m->g_pf_chunk = nullptr; m->pf_graph_failed = true; }
        m->pf_chunk_launches = 2 + 11 * c.n_layers;
    }
    for (int i = 0; i < nfull; i++) {
        if (m->g_pf_chunk) { HX_CUDA(cudaGraphLaunch(m->g_pf_chunk, m->st)); HX_COUNT_LAUNCH(m->pf_chunk_launches); }
        else if ((rc = pf_enqueue_chunk(m, HX_PF_TB))) return rc;
    }
    if (rem && (rc = pf_enqueue_chunk(m, rem))) return rc;
    const int nlast = rem ? rem : HX_PF_TB;
    if ((rc = pf_linear(m, m->head, m->pf_x + (size_t)(nlast - 1) * c.d_model, c.d_model, 1, 0, m->final_g, m->logits, 0, m->head.N, 0, 0))) return rc;
    hx_pf_argmax(m->logits, c.vocab, m->d_tok, m->d_hist, m->d_pos, T - 1, m->st);
    HX_CUDA(cudaGetLastError());
    return HX_OK;
}

static int run_prefill(hx_model* m, const int32_t* ids, int T, int seq = 0) {
    // positions 0..T-2 without the head, position T-1 with it
    HX_CUDA(cudaMemcpyAsync(m->d_prompt, ids, (size_t)T * 4, cudaMemcpyHostToDevice, m->st));
    if (m->tp_world > 1 && m->use_tc && m->pf_batched && m->head.t128 && m->use_df) {
        // a shard: positions [0, T-1) in chunks (the exchanges are epoch-numbered kernel arguments, so no graph replay),
        // the last position through the decode kernel, which holds the arg-max over the ranks' vocabulary slices
        int rc = pf_alloc(m); if (rc) return rc;
        const hx_config& c = m->cfg;
        const bool slot = seq != 0 || m->batch > 1;       // a slot of a batch: everything through the chunk path
        const int Tc = slot ? T : T - 1;
        const int ps[2] = {0, seq};
        HX_CUDA(cudaMemcpyAsync(m->d_pf_pos, ps, 8, cudaMemcpyHostToDevice, m->st));
        int nlast = 0;
        for (int t0 = 0; t0 < Tc; t0 += HX_PF_TB) {
            nlast = Tc - t0 < HX_PF_TB ? Tc - t0 : HX_PF_TB;
            if ((rc = pf_enqueue_chunk(m, nlast))) return rc;
        }
        if (slot) {
            // the head on the last position, then the first maximum over the ranks' vocabulary slices
            if ((rc = pf_linear(m, m->head, m->pf_x + (size_t)(nlast - 1) * c.d_model, c.d_model, 1, 0, m->final_g, m->logits, 0, m->head.N, 0, 0))) return rc;
            const unsigned ep = ++m->tp_pf_ep;
            unsigned long long* areas[8] = {nullptr};
            for (int w = 0; w < m->tp_world; w++)
                areas[w] = reinterpret_cast<unsigned long long*>(m->tp_peer[w]) + m->tp_pf_off + (size_t)(ep & 1u) * m->tp_world * m->tp_pf_area;
            hx_pf_tp_argmax_rows(m->logits, c.vocab, c.vocab, 1, m->tp_rank * c.vocab, areas, m->tp_rank, m->tp_world, m->tp_pf_area, ep,
                                 m->wait_limit, m->pf_err, m->d_tok, nullptr, m->st);
            HX_CUDA(cudaGetLastError());
            return HX_OK;
        }
        if ((rc = set_pos_tok(m, T - 1, nullptr))) return rc;
        HX_CUDA(cudaMemcpyAsync(m->d_tok, m->d_prompt + (T - 1), 4, cudaMemcpyDeviceToDevice, m->st));
        return step_decode(m);
    }
    if (m->use_tc && m->pf_batched && m->head.t128) return run_prefill_batched(m, T, seq);
    if (seq != 0) return hx_fail(HX_ERR_STATE, "prefill into KV slot %d needs the batched prefill path", seq);
    int rc = set_pos_tok(m, 0, nullptr); if (rc) return rc;
    for (int s = 0; s < T - 1; s++) if ((rc = step_prefill(m))) return rc;
    HX_CUDA(cudaMemcpyAsync(m->d_tok, m->d_prompt + (T - 1), 4, cudaMemcpyDeviceToDevice, m->st));
    return step_decode(m);
}

HX_API int hx_prefill(hx_model* m, const int32_t* ids, int T, int32_t* next_ids, float* logits) {
    HX_CHECK_ARG(m && ids && T > 0);
    if (T > m->kv_cap) return hx_fail(HX_ERR_STATE, "prompt of %d tokens exceeds the KV capacity %d", T, m->kv_cap);
    for (int i = 0; i < T; i++) if (ids[i] < 0 || ids[i] >= m->gcfg.vocab) return hx_fail(HX_ERR_ARG, "token %d outside the vocabulary", ids[i]);
    int rc = run_prefill(m, ids, T); if (rc) return rc;
    if (next_ids) HX_CUDA(cudaMemcpyAsync(next_ids, m->d_tok, 4, cudaMemcpyDeviceToHost, m->st));
    if (logits) HX_CUDA(cudaMemcpyAsync(logits, m->logits, (size_t)m->cfg.vocab * 4, cudaMemcpyDeviceToHost, m->st));
    HX_CUDA(cudaStreamSynchronize(m->st));
    if ((rc = persist_check(m))) return rc;
    m->kv_len = T;
    return HX_OK;
}

// Prefill one sequence of a batch into its own KV slot (the batched decode then continues all slots together).
HX_API int hx_prefill_seq(hx_model* m, int seq, const int32_t* ids, int T, int32_t* next_id, float* logits) {
    HX_CHECK_ARG(m && ids && T > 0);
    if (seq < 0 || seq >= m->batch) return hx_fail(HX_ERR_ARG, "sequence %d outside the batch of %d", seq, m->batch);
    if (T > m->kv_cap) return hx_fail(HX_ERR_STATE, "prompt of %d tokens exceeds the KV capacity %d", T, m->kv_cap);
    for (int i = 0; i < T; i++) if (ids[i] < 0 || ids[i] >= m->gcfg.vocab) return hx_fail(HX_ERR_ARG, "token %d outside the vocabulary", ids[i]);
    int rc = run_prefill(m, ids, T, seq); if (rc) return rc;
    if (next_id) HX_CUDA(cudaMemcpyAsync(next_id, m->d_tok, 4, cudaMemcpyDeviceToHost, m->st));
    if (logits) HX_CUDA(cudaMemcpyAsync(logits, m->logits, (size_t)m->cfg.vocab * 4, cudaMemcpyDeviceToHost, m->st));
    HX_CUDA(cudaStreamSynchronize(m->st));
    return persist_check(m);
}

HX_API int hx_decode_loop(hx_model* m, const int32_t* ids, int pos0, int n_steps, int32_t* out_ids, float* ms) {
    HX_CHECK_ARG(m && n_steps > 0);
    if (pos0 < 0 || pos0 + n_steps > m->kv_cap) return hx_fail(HX_ERR_STATE, "steps %d..%d outside the KV capacity %d", pos0, pos0 + n_steps, m->kv_cap);
    int rc = set_pos_tok(m, pos0, ids); if (rc) return rc;
    HX_CUDA(cudaEventRecord(m->ev0, m->st));
    if (m->profile && !m->persist) {
        // eager launches with an event pair around each kernel: per-kernel device time by category
        m->stats.ms_gemv = m->stats.ms_attn = m->stats.ms_other = 0.0f;
        for (int s = 0; s < n_steps; s++) {
            m->prof_n = 0;
            if ((rc = enqueue_step(m, false, true, true))) return rc;
            HX_CUDA(cudaStreamSynchronize(m->st));
            for (size_t i = 0; i < m->prof_n; i += 2) {
                float t = 0.0f; cudaEventElapsedTime(&t, m->prof_ev[i], m->prof_ev[i + 1]);
                const int cat = m->prof_cat[i / 2];
                (cat == CAT_GEMV ? m->stats.ms_gemv : cat == CAT_ATTN ? m->stats.ms_attn : m->stats.ms_other) += t;
            }
        }
    } else {
        for (int s = 0; s < n_steps; s++) if ((rc = step_decode(m))) return rc;
    }
    HX_CUDA(cudaEventRecord(m->ev1, m->st));
    if (out_ids) HX_CUDA(cudaMemcpyAsync(out_ids, m->d_hist + pos0 + 1, (size_t)n_steps * 4, cudaMemcpyDeviceToHost, m->st));
    HX_CUDA(cudaStreamSynchronize(m->st));
    float t = 0.0f; HX_CUDA(cudaEventElapsedTime(&t, m->ev0, m->ev1));
    m->stats.ms_total = t; m->stats.kernel_launches = (uint32_t)(m->persist ? n_steps : n_steps * kernels_per_step(m, true));
    if (ms) *ms = t;
    if ((rc = persist_check(m))) return rc;
    m->kv_len = pos0 + n_steps;
    return HX_OK;
}

HX_API int hx_generate_greedy(hx_model* m, const int32_t* prompt, int T, int n_new, int32_t* out_ids,
                              float* ms_prefill, float* ms_decode) {
    HX_CHECK_ARG(m && prompt && T > 0 && n_new > 0 && out_ids);
    if (T + n_new - 1 > m->kv_cap) return hx_fail(HX_ERR_STATE, "%d prompt + %d new tokens exceed the KV capacity %d", T, n_new, m->kv_cap);
    for (int i = 0; i < T; i++) if (prompt[i] < 0 || prompt[i] >= m->gcfg.vocab) return hx_fail(HX_ERR_ARG, "token %d outside the vocabulary", prompt[i]);
    cudaEvent_t e0, e1, e2;
    HX_CUDA(cudaEventCreate(&e0)); HX_CUDA(cudaEventCreate(&e1)); HX_CUDA(cudaEventCreate(&e2));
    HX_CUDA(cudaEventRecord(e0, m->st));
    int rc = run_prefill(m, prompt, T);            // leaves token #1 in d_tok / d_hist[T], *d_pos = T
    if (!rc) {
        cudaEventRecord(e1, m->st);
        for (int s = 1; s < n_new && !rc; s++) rc = step_decode(m);
        cudaEventRecord(e2, m->st);
        cudaMemcpyAsync(out_ids, m->d_hist + T, (size_t)n_new * 4, cudaMemcpyDeviceToHost, m->st);
        cudaError_t e = cudaStreamSynchronize(m->st);
        if (e != cudaSuccess) rc = hx_fail(HX_ERR_CUDA, "generate: %s", cudaGetErrorString(e));
        else if ((rc = persist_check(m))) {}
        else if (!rc) {
            float a = 0, b = 0; cudaEventElapsedTime(&a, e0, e1); cudaEventElapsedTime(&b, e1, e2);
            if (ms_prefill) *ms_prefill = a;
            if (ms_decode) *ms_decode = b;
            m->stats.ms_total = a + b;
            m->stats.kernel_launches = (uint32_t)((T - 1) * kernels_per_step(m, false) + n_new * kernels_per_step(m, true));
            m->kv_len = T + n_new - 1;
        }
    }
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaEventDestroy(e2);
    return rc;
}

// ---- prompt-lookup speculative decode ------------------------------------------------------------------
// The drafter of the reference (pld_draft, gpt2_infer.c:2972-2994): the longest suffix ids[T-k..T), k from k_max
// down to k_min, is looked up backwards in ids[0..T-1); the tokens following the most recent match (at most m
// of them, those before T) are the draft.  A match with nothing after it keeps the scan going.  Host only.
HX_API int hx_pld_draft(const int32_t* ids, int T, int k_min, int k_max, int m, int32_t* draft) {
    if (!ids || !draft || T < k_min + 1 || k_min < 1) return 0;
    if (m > HX_SPEC_DRAFT_MAX) m = HX_SPEC_DRAFT_MAX;
    if (m < 1) return 0;
    if (k_max > T - 1) k_max = T - 1;
    for (int k = k_max; k >= k_min; k--) {
        const int32_t* suffix = ids + (T - k);
        for (int start = T - k - 1; start >= 0; start--) {
            if (memcmp(ids + start, suffix, (size_t)k * sizeof(int32_t)) != 0) continue;
            int n = 0;
            for (int src = start + k; n < m && src < T; src++) draft[n++] = ids[src];
            if (n > 0) return n;
        }
    }
    return 0;
}

static int spec_alloc(hx_model* m) {
    if (!m->use_tc || !m->pf_batched || !m->head.t128 || m->tp_world > 1 || m->cfg.arch == 0)
        return hx_fail(HX_ERR_STATE, "speculative decode needs the tensor-core engine with batched prefill on one GPU");
    int rc = pf_alloc(m); if (rc) return rc;
    if (!m->pf_logits && (rc = dalloc(m, &m->pf_logits, (size_t)HX_PF_TB * m->cfg.vocab))) return rc;
    if (!m->sp_next && (rc = dalloc(m, &m->sp_next, (size_t)HX_PF_TB))) return rc;
    if (!m->sp_margin && (rc = dalloc(m, &m->sp_margin, (size_t)HX_PF_TB))) return rc;
    return HX_OK;
}

// The verify forward (forward_verify, gpt2_infer.c:3011-3074): the n window tokens sit at positions pos..pos+n-1
// behind the resident prefix [0, pos); their K/V rows go into the cache at those positions, every row attends
// [0, its own position], and every row gets its logits.  Here that is one prefill chunk that starts at `pos`
// plus the head on all n rows; the arg-max and its margin over the runner-up are taken on the device.
static int spec_verify(hx_model* m, const int32_t* win, int n, int pos, int32_t* a, float* margin) {
    const hx_config& c = m->cfg;
    const int ps[2] = {pos, 0};
    if (pos < 0 || pos + n > m->kv_cap) return hx_fail(HX_ERR_STATE, "verify window [%d, %d) outside the KV capacity %d", pos, pos + n, m->kv_cap);
    // the chunk kernels index the token buffer by position, as the prompt is laid out: the window goes to its positions
    HX_CUDA(cudaMemcpyAsync(m->d_prompt + pos, win, (size_t)n * 4, cudaMemcpyHostToDevice, m->st));
    HX_CUDA(cudaMemcpyAsync(m->d_pf_pos, ps, 8, cudaMemcpyHostToDevice, m->st));
    HxPfWhere wh = {m->d_pf_pos, nullptr, nullptr, (size_t)c.n_layers * c.n_kv_heads * m->kv_cap * c.head_dim, m->d_pf_pos + 1};
    int rc = pf_enqueue_layers(m, n, m->d_prompt, wh); if (rc) return rc;
    if ((rc = pf_linear(m, m->head, m->pf_x, c.d_model, n, 0, m->final_g, m->pf_logits, c.vocab, m->head.N, 0, 0))) return rc;
    hx_pf_top2_rows(m->pf_logits, c.vocab, c.vocab, n, m->sp_next, m->sp_margin, m->st);
    HX_CUDA(cudaMemcpyAsync(a, m->sp_next, (size_t)n * 4, cudaMemcpyDeviceToHost, m->st));
    HX_CUDA(cudaMemcpyAsync(margin, m->sp_margin, (size_t)n * 4, cudaMemcpyDeviceToHost, m->st));
    HX_CUDA(cudaStreamSynchronize(m->st));
    return persist_check(m);
}

// One plain decode step of token `tok` at position `pos`; the next token comes back to the host.
static int spec_single(hx_model* m, int32_t tok, int pos, int32_t* next) {
    int rc = set_pos_tok(m, pos, &tok); if (rc) return rc;
    if ((rc = step_decode(m))) return rc;
    HX_CUDA(cudaMemcpyAsync(next, m->d_tok, 4, cudaMemcpyDeviceToHost, m->st));
    HX_CUDA(cudaStreamSynchronize(m->st));
    return persist_check(m);
}

// Greedy generation with prompt-lookup drafts (run_generate's HX_SPEC path and spec_step, gpt2_infer.c:3076-3118,
// 3150-3161).  The output is the plain greedy sequence: a draft is accepted only where it equals the model's own
// arg-max.  The verify rows come from the batched GEMM path, whose sums are ordered differently from the decode
// kernel's, so an arg-max of a verify row is only used when it leads the runner-up by more than `min_margin`
// (a near tie is left to the plain decode step, which then decides exactly as hx_generate_greedy does).
HX_API int hx_generate_spec(hx_model* m, const int32_t* prompt, int T, int n_new, const hx_spec_config* cfg_in,
                            int32_t* out_ids, hx_spec_stats* stats_out, float* ms_prefill, float* ms_decode) {
    HX_CHECK_ARG(m && prompt && T > 0 && n_new > 0 && out_ids);
    if (T + n_new - 1 > m->kv_cap) return hx_fail(HX_ERR_STATE, "%d prompt + %d new tokens exceed the KV capacity %d", T, n_new, m->kv_cap);
    for (int i = 0; i < T; i++) if (prompt[i] < 0 || prompt[i] >= m->gcfg.vocab) return hx_fail(HX_ERR_ARG, "token %d outside the vocabulary", prompt[i]);
    hx_spec_config cfg = {3, 1, 6, 1e-3f};                       // the reference's defaults (HX_SPEC_K, HX_SPEC_KMIN, HX_SPEC_M)
    if (cfg_in) cfg = *cfg_in;
    HX_CHECK_ARG(cfg.k_min >= 1 && cfg.k_max >= cfg.k_min && cfg.m >= 1 && cfg.min_margin >= 0.0f);
    int rc = spec_alloc(m); if (rc) return rc;
    const int m_cap = 15 < HX_SPEC_DRAFT_MAX ? 15 : HX_SPEC_DRAFT_MAX;   // window = last token + drafts: sixteen rows at most, one token group of the GEMM
    const int M = cfg.m < m_cap ? cfg.m : m_cap;
    hx_spec_stats stt = {0, 0, 0, 0, 0, 0, 0, 0};
    std::vector<int32_t> ids(prompt, prompt + T);
    ids.reserve((size_t)T + n_new);
    cudaEvent_t e0, e1, e2;
    HX_CUDA(cudaEventCreate(&e0)); HX_CUDA(cudaEventCreate(&e1)); HX_CUDA(cudaEventCreate(&e2));
    cudaEventRecord(e0, m->st);
    int32_t first = 0;
    rc = run_prefill(m, prompt, T);
    if (!rc) {
        cudaMemcpyAsync(&first, m->d_tok, 4, cudaMemcpyDeviceToHost, m->st);
        cudaEventRecord(e1, m->st);
        if (cudaStreamSynchronize(m->st) != cudaSuccess) rc = hx_fail(HX_ERR_CUDA, "generate: %s", cudaGetErrorString(cudaGetLastError()));
        else rc = persist_check(m);
    }
    if (!rc) ids.push_back(first);
    int emitted = 1;
    while (!rc && emitted < n_new) {
        const int Tc = (int)ids.size(), pos = Tc - 1;            // ids[pos] is confirmed, its K/V row is not written yet
        int32_t draft[HX_SPEC_DRAFT_MAX], a[HX_PF_TB]; float margin[HX_PF_TB];
        int dn = hx_pld_draft(ids.data(), Tc, cfg.k_min, cfg.k_max, M, draft);
        if (Tc >= cfg.k_min + 1) stt.steps++;                     // counted where the reference's drafter counts
        if (dn > 0) { stt.hits++; stt.drafted += dn; }
        if (pos + dn >= m->kv_cap) { dn = m->kv_cap - 1 - pos; if (dn < 0) dn = 0; }
        int commit = 0;
        if (dn > 0) {
            int32_t win[HX_PF_TB];
            win[0] = ids[pos];
            for (int i = 0; i < dn; i++) win[1 + i] = draft[i];
            if ((rc = spec_verify(m, win, dn + 1, pos, a, margin))) break;
            stt.forwards++;
            if (margin[0] > cfg.min_margin) {
                commit = 1;
                for (int i = 1; i <= dn; i++) {
                    if (draft[i - 1] != a[i - 1]) break;
                    if (!(margin[i] > cfg.min_margin)) { stt.near_ties++; break; }
                    commit = i + 1;
                }
                if (commit > n_new - emitted) commit = n_new - emitted;
                stt.accepted += commit - 1; stt.emitted += commit;     // counted like the reference: verify steps only
            } else stt.near_ties++;
        }
        if (commit == 0) {                                        // no draft, or the first verify row was a near tie
            if ((rc = spec_single(m, ids[pos], pos, &a[0]))) break;
            stt.single_steps++;
            commit = 1;
        }
        for (int i = 0; i < commit; i++) ids.push_back(a[i]);
        emitted += commit;
    }
    if (!rc) {
        cudaEventRecord(e2, m->st);
        cudaEventSynchronize(e2);
        float p = 0, d = 0; cudaEventElapsedTime(&p, e0, e1); cudaEventElapsedTime(&d, e1, e2);
        if (ms_prefill) *ms_prefill = p;
        if (ms_decode) *ms_decode = d;
        memcpy(out_ids, ids.data() + T, (size_t)n_new * 4);
        if (stats_out) *stats_out = stt;
        m->kv_len = T + n_new - 1;
        // leave the device-side cursor where hx_generate_greedy leaves it: last token, next position
        const int32_t last = ids.back();
        rc = set_pos_tok(m, T + n_new - 1, &last);
        if (!rc && cudaStreamSynchronize(m->st) != cudaSuccess) rc = hx_fail(HX_ERR_CUDA, "generate: %s", cudaGetErrorString(cudaGetLastError()));
    }
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaEventDestroy(e2);
    return rc;
}

static int bd_check(hx_model* m, int n_seq) {
    if (!m->use_tc || !m->head.t128 || (m->tp_world > 1 && !(m->use_df && m->pf_batched)))
        return hx_fail(HX_ERR_STATE, "batched decode needs the tensor-core engine (and, in a tensor-parallel group, the pair engine)");
    if (n_seq < 1 || n_seq > m->batch) return hx_fail(HX_ERR_ARG, "%d sequences, the model was created for %d", n_seq, m->batch);
    return bd_alloc(m);
}

HX_API int hx_decode_batch(hx_model* m, const int32_t* ids, const int32_t* pos, int n_seq, int32_t* next_ids) {
    HX_CHECK_ARG(m && ids && pos && next_ids);
    int rc = bd_check(m, n_seq); if (rc) return rc;
    for (int i = 0; i < n_seq; i++) {
        if (ids[i] < 0 || ids[i] >= m->gcfg.vocab) return hx_fail(HX_ERR_ARG, "token %d outside the vocabulary", ids[i]);
        if (pos[i] < 0 || pos[i] >= m->kv_cap) return hx_fail(HX_ERR_STATE, "position %d outside the KV capacity %d", pos[i], m->kv_cap);
    }
    HX_CUDA(cudaMemcpyAsync(m->d_bids, ids, (size_t)n_seq * 4, cudaMemcpyHostToDevice, m->st));
    HX_CUDA(cudaMemcpyAsync(m->d_bpos, pos, (size_t)n_seq * 4, cudaMemcpyHostToDevice, m->st));
    if ((rc = bd_enqueue_step(m, n_seq))) return rc;
    HX_CUDA(cudaMemcpyAsync(next_ids, m->d_bnext, (size_t)n_seq * 4, cudaMemcpyDeviceToHost, m->st));
    HX_CUDA(cudaStreamSynchronize(m->st));
    return persist_check(m);
}

HX_API int hx_decode_batch_loop(hx_model* m, const int32_t* ids, int pos0, int n_seq, int n_steps, int32_t* out_ids, float* ms) {
    HX_CHECK_ARG(m && ids && n_steps > 0);
    int rc = bd_check(m, n_seq); if (rc) return rc;
    if (pos0 < 0 || pos0 + n_steps > m->kv_cap) return hx_fail(HX_ERR_STATE, "steps %d..%d outside the KV capacity %d", pos0, pos0 + n_steps, m->kv_cap);
    std::vector<int> p((size_t)n_seq, pos0);
    HX_CUDA(cudaMemcpyAsync(m->d_bids, ids, (size_t)n_seq * 4, cudaMemcpyHostToDevice, m->st));
    HX_CUDA(cudaMemcpyAsync(m->d_bpos, p.data(), (size_t)n_seq * 4, cudaMemcpyHostToDevice, m->st));
    HX_CUDA(cudaStreamSynchronize(m->st));
    // one step captured once per batch size and replayed (tokens and positions live in device memory)
    if (n_steps > 1 && m->tp_world == 1 && (!m->g_bstep || m->g_bstep_n != n_seq)) {       // (a shard's exchanges carry epoch arguments)
        if (m->g_bstep) { cudaGraphExecDestroy(m->g_bstep); m->g_bstep = nullptr; }
        cudaGraph_t g = nullptr;
        HX_CUDA(cudaStreamBeginCapture(m->st, cudaStreamCaptureModeThreadLocal));
        const unsigned long long before = g_hx_launches;
        rc = bd_enqueue_step(m, n_seq);
        cudaError_t e = cudaStreamEndCapture(m->st, &g);
        m->pf_chunk_launches = (int)(g_hx_launches - before);
        g_hx_launches = before;
        if (rc) { if (g) cudaGraphDestroy(g); return rc; }
        if (e == cudaSuccess) e = cudaGraphInstantiate(&m->g_bstep, g, 0);
        if (g) cudaGraphDestroy(g);
        if (e != cudaSuccess) { (void)cudaGetLastError(); m->g_bstep = nullptr; }
        m->g_bstep_n = n_seq;
    }
    HX_CUDA(cudaEventRecord(m->ev0, m->st));
    for (int s = 0; s < n_steps; s++) {
        if (m->g_bstep && m->g_bstep_n == n_seq) { HX_CUDA(cudaGraphLaunch(m->g_bstep, m->st)); HX_COUNT_LAUNCH(m->pf_chunk_launches); }
        else if ((rc = bd_enqueue_step(m, n_seq))) return rc;
        if (out_ids) HX_CUDA(cudaMemcpyAsync(out_ids + (size_t)s * n_seq, m->d_bnext, (size_t)n_seq * 4, cudaMemcpyDeviceToHost, m->st));
    }
    HX_CUDA(cudaEventRecord(m->ev1, m->st));
    HX_CUDA(cudaStreamSynchronize(m->st));
    float t = 0.0f; HX_CUDA(cudaEventElapsedTime(&t, m->ev0, m->ev1));
    if (ms) *ms = t;
    return persist_check(m);
}

HX_API int hx_model_fill_kv(hx_model* m, int T, uint64_t seed) {
    HX_CHECK_ARG(m && T >= 0 && T <= m->kv_cap);
    const hx_config& c = m->cfg;
    // whole cache gets values; only positions below the running length are ever read
    const size_t n = (size_t)c.n_layers * c.n_kv_heads * m->kv_cap * c.head_dim * (size_t)m->batch;
    int rc = hx_launch_fill_normal(m->kc, n, 1.0f, seed * 2 + 1, m->st); if (rc) return rc;
    rc = hx_launch_fill_normal(m->vc, n, 1.0f, seed * 2 + 2, m->st); if (rc) return rc;
    HX_CUDA(cudaStreamSynchronize(m->st));
    m->kv_len = T;
    return HX_OK;
}

// Copy n cached positions [pos0, pos0 + n) of one (sequence, layer, kv head) between the cache and host arrays
// of n * head_dim floats (K after QK-norm and RoPE, as the reference caches it).
static int kv_span(hx_model* m, int seq, int layer, int kv_head, int pos0, int n, size_t* off) {
    const hx_config& c = m->cfg;
    if (seq < 0 || seq >= m->batch || layer < 0 || layer >= c.n_layers || kv_head < 0 || kv_head >= c.n_kv_heads)
        return hx_fail(HX_ERR_ARG, "kv rows: sequence %d, layer %d, kv head %d outside the model", seq, layer, kv_head);
    if (pos0 < 0 || n < 0 || pos0 + n > m->kv_cap) return hx_fail(HX_ERR_STATE, "kv rows %d..%d outside the KV capacity %d", pos0, pos0 + n, m->kv_cap);
    const size_t seq_stride = (size_t)c.n_layers * c.n_kv_heads * m->kv_cap * c.head_dim;
    *off = seq * seq_stride + (((size_t)layer * c.n_kv_heads + kv_head) * m->kv_cap + pos0) * c.head_dim;
    return HX_OK;
}
HX_API int hx_model_kv_read(hx_model* m, int seq, int layer, int kv_head, int pos0, int n, float* k, float* v) {
    HX_CHECK_ARG(m && k && v);
    size_t off = 0; int rc = kv_span(m, seq, layer, kv_head, pos0, n, &off); if (rc) return rc;
    HX_CUDA(cudaStreamSynchronize(m->st));
    HX_CUDA(cudaMemcpy(k, m->kc + off, (size_t)n * m->cfg.head_dim * 4, cudaMemcpyDeviceToHost));
    HX_CUDA(cudaMemcpy(v, m->vc + off, (size_t)n * m->cfg.head_dim * 4, cudaMemcpyDeviceToHost));
    return HX_OK;
}
HX_API int hx_model_kv_write(hx_model* m, int seq, int layer, int kv_head, int pos0, int n, const float* k, const float* v) {
    HX_CHECK_ARG(m && k && v);
    size_t off = 0; int rc = kv_span(m, seq, layer, kv_head, pos0, n, &off); if (rc) return rc;
    HX_CUDA(cudaStreamSynchronize(m->st));
    HX_CUDA(cudaMemcpy(m->kc + off, k, (size_t)n * m->cfg.head_dim * 4, cudaMemcpyHostToDevice));
    HX_CUDA(cudaMemcpy(m->vc + off, v, (size_t)n * m->cfg.head_dim * 4, cudaMemcpyHostToDevice));
    return HX_OK;
}

// ---- single-matrix round trip: quantize W, then y = dequant(W) x, host buffers in and out ---------------
HX_API int hx_roundtrip_host(const float* w, int rows, int K, const float* x, float* y, int* kpad_out) {
    HX_CHECK_ARG(w && x && y && rows > 0 && K > 0 && K % 4 == 0);
    const int Kpad = hx_kpad(K), Kd = hx_kd(K);
    float *dw = nullptr, *dx = nullptr, *dy = nullptr, *dts = nullptr; int32_t* dq = nullptr; uint8_t *dm = nullptr, *dc = nullptr, *ds = nullptr;
    int rc = HX_OK;
    auto fr = [&]() { cudaFree(dw); cudaFree(dx); cudaFree(dy); cudaFree(dts); cudaFree(dq); cudaFree(dm); cudaFree(dc); cudaFree(ds); };
#define RT(call) do { cudaError_t _e = (call); if (_e != cudaSuccess) { fr(); return hx_fail(HX_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(_e)); } } while (0)
    RT(cudaMalloc(&dw, (size_t)rows * K * 4)); RT(cudaMalloc(&dx, (size_t)Kd * 4)); RT(cudaMalloc(&dy, (size_t)rows * 4));
    RT(cudaMalloc(&dts, 4)); RT(cudaMalloc(&dq, (size_t)rows * (Kpad / 7) * 4)); RT(cudaMalloc(&dm, (size_t)rows * (Kpad / 16)));
    RT(cudaMalloc(&dc, (size_t)rows * (Kd / 2))); RT(cudaMalloc(&ds, (size_t)rows * (Kd / 16)));
    RT(cudaMemcpy(dw, w, (size_t)rows * K * 4, cudaMemcpyHostToDevice));
    RT(cudaMemset(dx, 0, (size_t)Kd * 4));
    RT(cudaMemcpy(dx, x, (size_t)K * 4, cudaMemcpyHostToDevice));
    rc = hx_quantize_nvfp4(dw, rows, K, dq, dm, nullptr, dts, nullptr);
    if (!rc) rc = hx_repack_d16(dq, dm, rows, K, Kpad, dc, ds, nullptr);
    if (!rc) rc = hx_gemv_d16(dx, dc, ds, dts, dy, rows, Kd, nullptr);
    if (rc) { fr(); return rc; }
    RT(cudaMemcpy(y, dy, (size_t)rows * 4, cudaMemcpyDeviceToHost));
#undef RT
    fr();
    if (kpad_out) *kpad_out = Kpad;
    return HX_OK;
}
