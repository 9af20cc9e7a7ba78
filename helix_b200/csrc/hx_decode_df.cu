// hx_decode_df.cu -- the persistent decode-step kernel without grid barriers ("dataflow" engine).
//
// One cooperative CTA per SM runs the whole token as a list of phases (per layer qkv | attention | o_proj |
// gate+up | down, then lm_head + arg-max), the weights streaming through a shared-memory ring of T128 cells
// into tcgen05.mma kind::mxf4nvf4 exactly as in hx_persist_tc.cu (digit-sliced activations, TMEM
// accumulators, a producer thread that runs ahead of the consumers).  What differs is how the CTAs hand
// results to one another.  There is no grid-wide barrier: every vector that crosses CTAs (residual stream,
// q, the position's k and v, attention partials, the SwiGLU hidden vector, split-K partial sums, per-tile
// sums of squares) is stored as 8-byte (value, epoch) pairs with one 64-bit store per element, and the
// reader polls the data itself until the epoch of the producing phase shows up.  An 8-byte store is
// single-copy atomic, so a matching epoch proves the value beside it; no fence, flag or ticket travels
// separately, and a hand-over costs one store-to-load latency instead of release + barrier + load.
//
//  * A linear phase cuts its cells over the CTAs like hx_persist_tc.cu (tc_plan).  The CTA that holds
//    piece 0 of a tile is its merger: the other pieces store their partial rows as pairs, the merger polls
//    them, adds them in piece order (results do not depend on timing) and runs the epilogue.
//  * RMSNorm needs the sum of squares of the whole input: the residual epilogue that produces a tile of x
//    also publishes that tile's sum of squares, and every CTA of the consuming phase adds the per-tile
//    sums in tile order.  Polling them also keeps the CTAs in step: nobody enters a norm phase before all
//    tiles of the previous residual phase are final, which is what makes the reuse of the pair buffers
//    one layer later safe.  The digit scale is taken over the CTA's own K slice.
//  * Tensor parallel: the merger of a row-split linear stores its partial rows as pairs into every
//    rank's exchange buffer (plain NVLink stores, 8-byte atomic) and adds the ranks' rows in rank order,
//    so the all-reduce is one more hand-over of the same kind.
//
// Every wait is bounded (HxPersist::wait_limit polls).  A wait that runs out latches an abort flag; code
// between two phase boundaries never changes its barrier pattern because of it (waits return at once,
// the arithmetic runs on whatever is there) and the phase boundary decides with a barrier-wide OR, so all
// threads leave together through the common exit, which waits for the CTA's own bulk copies in flight
// and frees its tensor memory.  The host reports HX_ERR_TIMEOUT.
#define HX_TC_MAX_RING 10
#define RING_SLOTS ((uint32_t)P.tc_ring)
#ifndef NCW
#define NCW 8
#endif
#define NCT (NCW * 32)
#define PT (NCT + 64)               // + producer warp (16) + MMA warp (17)
// mbar_wait (hx_persist_common.cuh) reads its limit from the word after the abort flag it is given
#define WAIT_LIMIT (reinterpret_cast<volatile unsigned*>(abort_flag)[1])
#include "hx_persist.cuh"
#include "hx_persist_common.cuh"
#include "hx_gemm_tc.cuh"

#define TC_NDIG 16
#define TM_COLS 256
#define TM_D0 0                     // two accumulators of TC_NDIG columns
#define TM_SFB 32                   // constant unit scales for the digit columns
#define TM_SFA 64                   // + slot * 16 + K step * 4
#define EPI_WARPS 4                 // warps 0..3 own TMEM lanes 0..127 = the rows of a tile
#define DRAIN_LIMIT (1u << 22)

typedef unsigned long long u64;

// per-phase time stamps of one CTA, debug builds only (-DHX_DEBUG_STAMPS)
#ifdef HX_DEBUG_STAMPS
#define DF_STAMP(i) do { if (P.dbg && cta == P.dbg_cta && tid == 0) { unsigned long long _t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t)); P.dbg[pi * 16 + (i)] = _t; } } while (0)
#define DF_MARK(ev) do { if (P.dbg_all && tid == 0) { unsigned long long _t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t)); P.dbg_all[((size_t)pi * gridDim.x + blockIdx.x) * 8 + (ev)] = _t; } } while (0)
#define DF_GT(v) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v))
#define DF_MMA_T0() unsigned long long _w0; DF_GT(_w0)
#define DF_MMA_T1() do { unsigned long long _w1; DF_GT(_w1); dbg_wait += _w1 - _w0; } while (0)
#define DF_MMA_OUT() do { if (P.dbg_all) { unsigned long long _t; DF_GT(_t); P.dbg_all[((size_t)pi * gridDim.x + blockIdx.x) * 8 + 7] = _t; P.dbg_all[((size_t)pi * gridDim.x + blockIdx.x) * 8 + 6] = dbg_wait; } } while (0)
#else
#define DF_STAMP(i) do { } while (0)
#define DF_MARK(ev) do { } while (0)
#define DF_MMA_T0() do { } while (0)
#define DF_MMA_T1() do { } while (0)
#define DF_MMA_OUT() do { } while (0)
#endif

namespace {

__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout = 0) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) |
           (1ull << 46) | ((uint64_t)layout << 61);
}
#define TC_SW128 2u
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" :: "r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                 :: "r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 2, %0;" :: "n"(EPI_WARPS * 32) : "memory"); }
// consumer barrier that also ORs a flag over the consumer threads: every thread gets the same answer
__device__ __forceinline__ bool consumer_sync_any(int flag) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbar.red.or.pred q, 1, %2, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(r) : "r"(flag), "n"(NCT) : "memory");
    return r != 0;
}

struct SmemDf {
    uint64_t full[HX_TC_MAX_RING];
    uint64_t empty[HX_TC_MAX_RING];
    uint64_t acc_full[2], acc_empty[2], b_ready;
    float red[NCW * 2];
    float att_m[8], att_l[8], att_r[8];
    float wgt[2304];                // merge weights of the attention splits, [head][split] (o_proj prologue)
    float bv[NCW]; int bi[NCW];
    float swi[128];
    HxPhase ph[2];
    AttPlan ap; int att_ns, ap_tile_rows, ap_ntiles;      // attention work split of this launch (depends on the position only)
    int tile_off[8], tile_slot[8];                        // ring slots of the attention tile in flight (K: 0.., V: 4..)
    unsigned ticket;
    uint32_t tmem_base;
    volatile int abort_flag; unsigned wait_limit;      // adjacent: bounded waits read the limit at (&abort_flag)[1]
};

// ---- (value, epoch) pairs ----
__device__ __forceinline__ void ll_st(u64* p, float v, unsigned ep) {
    const u64 w = ((u64)ep << 32) | (u64)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" :: "l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void ll_st_sys(u64* p, float v, unsigned ep) {
    const u64 w = ((u64)ep << 32) | (u64)__float_as_uint(v);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ u64 ll_ld(const u64* p) {
    u64 w; asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory"); return w;
}
__device__ __forceinline__ u64 ll_ld_sys(const u64* p) {
    u64 w; asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory"); return w;
}
__device__ __forceinline__ void ll_ld2(const u64* p, u64& a, u64& b) {
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ float ll_val(u64 w) { return __uint_as_float((unsigned)w); }
__device__ __forceinline__ bool ll_ok(u64 w, unsigned ep) { return (unsigned)(w >> 32) == ep; }
__device__ __forceinline__ bool df_gave_up(SmemDf& S, const HxPersist& P) {
    return S.abort_flag != 0 || *reinterpret_cast<volatile int*>(P.err) != 0;
}
__device__ __forceinline__ void df_fail(SmemDf& S, const HxPersist& P) { S.abort_flag = 1; *P.err = 1; }

// One pair.  After an abort the wait returns at once with whatever is there.
template <bool SYS = false>
__device__ __forceinline__ float df_wait1(const u64* p, unsigned ep, SmemDf& S, const HxPersist& P) {
    const unsigned lim = S.abort_flag ? 1u : S.wait_limit;
    u64 w = 0;
    for (unsigned i = 0; i < lim; i++) {
        w = SYS ? ll_ld_sys(p) : ll_ld(p);
        if (ll_ok(w, ep)) return ll_val(w);
        if ((i & 63u) == 63u && df_gave_up(S, P)) break;
    }
    df_fail(S, P);
    return ll_val(w);
}
// Up to four pairs `stride` apart, all in flight together; returns their values added to `acc` in index order.
__device__ __forceinline__ float df_wait_add4(const u64* p, size_t stride, int n, unsigned ep, float acc, SmemDf& S, const HxPersist& P) {
    const unsigned lim = S.abort_flag ? 1u : S.wait_limit;
    u64 w[4] = {0, 0, 0, 0};
    bool ok = false;
    for (unsigned i = 0; i < lim && !ok; i++) {
        ok = true;
#pragma unroll
        for (int c = 0; c < 4; c++) if (c < n) w[c] = ll_ld(p + (size_t)c * stride);
#pragma unroll
        for (int c = 0; c < 4; c++) if (c < n) ok = ok && ll_ok(w[c], ep);
        if (!ok && (i & 63u) == 63u && df_gave_up(S, P)) break;
    }
    if (!ok) df_fail(S, P);
#pragma unroll
    for (int c = 0; c < 4; c++) if (c < n) acc += ll_val(w[c]);
    return acc;
}
// Two pairs at a 16-byte aligned address.
__device__ __forceinline__ void df_wait2(const u64* p, unsigned ep, float& a, float& b, SmemDf& S, const HxPersist& P) {
    const unsigned lim = S.abort_flag ? 1u : S.wait_limit;
    u64 x = 0, y = 0;
    for (unsigned i = 0; i < lim; i++) {
        ll_ld2(p, x, y);
        if (ll_ok(x, ep) && ll_ok(y, ep)) { a = ll_val(x); b = ll_val(y); return; }
        if ((i & 63u) == 63u && df_gave_up(S, P)) break;
    }
    df_fail(S, P);
    a = ll_val(x); b = ll_val(y);
}
// Eight consecutive pairs at a 16-byte aligned address (one item of the digit prologue).
__device__ __forceinline__ void df_wait8(const u64* p, unsigned ep, float (&v)[8], SmemDf& S, const HxPersist& P) {
    const unsigned lim = S.abort_flag ? 1u : S.wait_limit;
    u64 w[8];
#pragma unroll
    for (int e = 0; e < 8; e++) w[e] = 0;
    bool ok = false;
    for (unsigned i = 0; i < lim && !ok; i++) {
#pragma unroll
        for (int e = 0; e < 8; e += 2) ll_ld2(p + e, w[e], w[e + 1]);
        ok = true;
#pragma unroll
        for (int e = 0; e < 8; e++) ok = ok && ll_ok(w[e], ep);
        if (!ok && (i & 63u) == 63u && df_gave_up(S, P)) break;
    }
    if (!ok) df_fail(S, P);
#pragma unroll
    for (int e = 0; e < 8; e++) v[e] = ll_val(w[e]);
}

// ---- attention work split: the number of splits follows the context length (about 64 positions each) ----
__device__ __noinline__ AttPlan att_plan_df(const HxPersist& P, int cta, int pos, int nring, int* ns_out, int* tile_rows, int* ntiles) {
#ifndef DF_SPLIT_ROWS_LOG2
#define DF_SPLIT_ROWS_LOG2 4          // about 16 cached positions per attention split while CTAs are left (measured best: 8..16)
#endif
    int ns = (pos + (1 << DF_SPLIT_ROWS_LOG2)) >> DF_SPLIT_ROWS_LOG2;
    ns = ns < 1 ? 1 : (ns > P.att_nsplit ? P.att_nsplit : ns);
    struct { int NKV, DH; } ph = {P.att_nkv, P.att_dh};
    AttPlan a;
    a.active = cta < ph.NKV * ns;
    a.kv = cta / ns; a.split = cta % ns;
    const int T = pos + 1, chunk = (T + ns - 1) / ns;
    a.t0 = a.split * chunk; a.t1 = min(T, a.t0 + chunk);
    if (!a.active || a.t0 >= a.t1) { a.t0 = a.t1 = 0; a.n_old = 0; a.has_new = 0; }
    else { a.has_new = (pos >= a.t0 && pos < a.t1); a.n_old = (a.t1 - a.t0) - a.has_new; }
    a.rows_per_slot = HX_RING_SLOT / (ph.DH * 4);
    a.nslots = (a.n_old + a.rows_per_slot - 1) / a.rows_per_slot;      // K slots == V slots
    const AttPlan2 a2 = att_plan2(a, nring);
    *ns_out = ns; *tile_rows = a2.tile_rows; *ntiles = a2.ntiles;
    return a;
}

// ------------------------------------------------------------------------------------------------
// Attention phase of one CTA: (kv head, split of the cached positions); the split of the work depends on the
// position only and is worked out once per launch (SmemDf::ap).  q (normed, rotated) and this position's k and v
// arrive as pairs from the qkv epilogue; older rows stream through the ring from the cache.
//  * scores: eight threads per (row, head), each holding its DH/8 query dimensions in registers, one shuffle
//    tree per row;
//  * soft-max statistics (online, m seeded -1e8 like the reference, fused_decode_attn_kernel.hx:74-102): one warp
//    per head;
//  * P*V: a thread owns four output dimensions of ALL heads of the group over a subset of the rows (a V row is read
//    once, not once per head); the subsets are folded through shared memory.
// The split's partial output and (max, sum) leave as pairs; the o_proj prologue merges the splits.
// The phase runs once per layer from a cold instruction cache: loops stay rolled and waits have one site each.
// ------------------------------------------------------------------------------------------------
#define ATT_GP 8                       // stride of a row's probabilities (one float per head of the group, GRP <= 8)
__device__ __forceinline__ void ring_adv(uint32_t& slot, uint32_t& par, uint32_t n, uint32_t nring) {
    slot += n;
    while (slot >= nring) { slot -= nring; par ^= 1u; }
}
// The splits of a head merged into the attention output, by one CTA per head: the CTA of (kv head, split s) takes
// the heads s, s + ns, ... of its group once its own partial is out.  out[d] = sum_s w_s acc_s[d] with
// w_s = exp(m_s - M) / sum_s l_s exp(m_s - M); splits are added in split order, so the result does not depend on
// timing.  The o_proj phase then reads a plain vector.
__device__ __noinline__ void attention_merge_df(const HxPersist& P, const HxPhase& ph, SmemDf& S, int kv, int split, int ns, int grp, unsigned ep) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int DH = ph.DH;
    float* wm = S.wgt; float* wl = S.wgt + 1152;                  // ns <= 1152 (the host checks heads * splits <= 2304)
    #pragma unroll 1
    for (int i = split; i < grp; i += ns) {
        const int h = kv * grp + i;
        if (warp == 0) {
            const u64* pml = ph.pml_ll + 2 * (size_t)h * ns;
            float M = -INFINITY;
            #pragma unroll 1
            for (int s = lane; s < ns; s += 32) { float m, l; df_wait2(pml + 2 * s, ep, m, l, S, P); wm[s] = m; wl[s] = l; M = fmaxf(M, m); }
            M = hx_warp_max(M);
            float L = 0.0f;
            #pragma unroll 1
            for (int s = lane; s < ns; s += 32) { const float w = __expf(wm[s] - M); wm[s] = w; L = fmaf(wl[s], w, L); }
            L = hx_warp_sum(L);
            #pragma unroll 1
            for (int s = lane; s < ns; s += 32) wm[s] = wm[s] / L;
        }
        consumer_sync();
        constexpr int SB = 12;
        #pragma unroll 1
        for (int d2 = tid; d2 < (DH >> 1); d2 += NCT) {
            const u64* pa = ph.pacc_ll + (size_t)h * ns * DH + 2 * d2;
            float o0 = 0.0f, o1 = 0.0f;
            #pragma unroll 1
            for (int s0 = 0; s0 < ns; s0 += SB) {
                const int n = min(SB, ns - s0);
                u64 w[SB][2];
                const unsigned lim = S.abort_flag ? 1u : S.wait_limit;
                bool ok = false;
                #pragma unroll 1
                for (unsigned t = 0; t < lim && !ok; t++) {
#pragma unroll
                    for (int c = 0; c < SB; c++) { w[c][0] = w[c][1] = 0; if (c < n) ll_ld2(pa + (size_t)(s0 + c) * DH, w[c][0], w[c][1]); }
                    ok = true;
#pragma unroll
                    for (int c = 0; c < SB; c++) if (c < n) ok = ok && ll_ok(w[c][0], ep) && ll_ok(w[c][1], ep);
                    if (!ok && (t & 63u) == 63u && df_gave_up(S, P)) break;
                }
                if (!ok) df_fail(S, P);
#pragma unroll
                for (int c = 0; c < SB; c++) if (c < n) { const float wg = wm[s0 + c]; o0 = fmaf(ll_val(w[c][0]), wg, o0); o1 = fmaf(ll_val(w[c][1]), wg, o1); }
            }
            ll_st(ph.out_ll + (size_t)h * DH + 2 * d2, o0, ep);
            ll_st(ph.out_ll + (size_t)h * DH + 2 * d2 + 1, o1, ep);
        }
        consumer_sync();                                            // the weights are reused by the next head
    }
}

template <int GRP>
__device__ __noinline__ void attention_df(const HxPersist& P, const HxPhase& ph, SmemDf& S, uint8_t* ring, uint8_t* digb,
                                          uint32_t& cslot, uint32_t& cpar, int pi, int pos) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, cta = blockIdx.x;
    (void)cta;
    const int ns = S.att_ns;
    const AttPlan ap = S.ap;
    const int tr_rows = S.ap_tile_rows, ntiles = S.ap_ntiles;
    const unsigned ep = P.ep_base + (unsigned)pi + 1u, in_ep = P.ep_base + (unsigned)ph.in_dep + 1u;
    const int DH = ph.DH, rps = ap.rows_per_slot, KVD = ph.NKV * DH;
    const uint32_t nring = RING_SLOTS;
    float* sq = reinterpret_cast<float*>(digb);                 // [GRP][DH] queries
    float* knew = sq + 8 * 256;                                  // [DH] current k
    float* vnew = knew + 256;                                    // [DH] current v
    float* sp = vnew + 256;                                      // [160 rows][ATT_GP] scores / probabilities
    float* accx = sp + 160 * ATT_GP;                             // [row subset][GRP][DH] partial outputs
    const float* ringf = reinterpret_cast<const float*>(ring);
    const int HD = GRP * DH;
    // score pass: thread = (row group, head, part of 8)
    constexpr int TPR = GRP * 8, NRG = NCT / TPR;
    const int a_rg = tid / TPR, a_i = (tid >> 3) % GRP, a_p = tid & 7;
    const int CPT = DH >> 5;                                     // float4 chunks of a row per score thread
    // P*V pass: thread = (row subset, float4 chunk of the head dimension), all heads of the group
    const int CH4 = DH >> 2, NSUB = NCT / CH4;
    const int c_sub = tid / CH4, c_c = tid - c_sub * CH4;
    if (!ap.active) return;
    if (ap.t1 <= ap.t0) {
        // empty split: neutral partial
        for (int i = tid; i < GRP; i += NCT) {
            const int hs = (ap.kv * GRP + i) * ns + ap.split;
            ll_st(ph.pml_ll + 2 * hs, -100000000.0f, ep); ll_st(ph.pml_ll + 2 * hs + 1, 0.0f, ep);
        }
        for (int i = tid; i < HD; i += NCT) {
            const int hs = (ap.kv * GRP + i / DH) * ns + ap.split;
            ll_st(ph.pacc_ll + (size_t)hs * DH + i % DH, 0.0f, ep);
        }
        attention_merge_df(P, ph, S, ap.kv, ap.split, ns, GRP, ep);
        return;
    }
    float4 acc[GRP];
#pragma unroll
    for (int i = 0; i < GRP; i++) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    {
        // q of the group, and k, v of this position when it falls into the split: one polling site
        const int nq = HD >> 1, nkv = ap.has_new ? DH >> 1 : 0;
        #pragma unroll 1
        for (int i = tid; i < nq + 2 * nkv; i += NCT) {
            const u64* src; float* dst;
            if (i < nq) { src = ph.in_ll + (size_t)ap.kv * HD + 2 * i; dst = sq + 2 * i; }
            else if (i < nq + nkv) { src = ph.kv_ll + (size_t)ap.kv * DH + 2 * (i - nq); dst = knew + 2 * (i - nq); }
            else { src = ph.kv_ll + (size_t)KVD + (size_t)ap.kv * DH + 2 * (i - nq - nkv); dst = vnew + 2 * (i - nq - nkv); }
            df_wait2(src, in_ep, dst[0], dst[1], S, P);
        }
    }
    if (tid < 8) { S.att_m[tid] = -100000000.0f; S.att_l[tid] = 0.0f; }
    consumer_sync();
    DF_STAMP(7); DF_MARK(1);
    float4 qf[4];
#pragma unroll
    for (int c = 0; c < 4; c++) qf[c] = (c < CPT && a_rg < NRG) ? *reinterpret_cast<const float4*>(sq + a_i * DH + (a_p + 8 * c) * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    const int ntile = ntiles + ((ap.has_new && ap.n_old % tr_rows == 0) ? 1 : 0);
    #pragma unroll 1
    for (int s = 0; s < ntile; s++) {
        const bool ring_tile = s < ntiles;
        const int nr = ring_tile ? min(tr_rows, ap.n_old - s * tr_rows) : 0;
        const int nsl = (nr + rps - 1) / rps;                       // ring slots of this tile (K, then as many of V)
        const bool add_new = ap.has_new && (s == ntile - 1);       // the current position rides on the last tile
        const int ntot = nr + (add_new ? 1 : 0);
        // one thread per ring slot waits for the rows and publishes where they are: K slots 0.., V slots 4..
        if (tid < 2 * nsl) {
            uint32_t sl = cslot, pr = cpar;
            ring_adv(sl, pr, (uint32_t)tid, nring);
            mbar_wait(&S.full[sl], pr, &S.abort_flag);
            S.tile_off[tid < nsl ? tid : 4 + tid - nsl] = (int)(sl * (HX_RING_SLOT / 4));
            S.tile_slot[tid] = (int)sl;
        }
        ring_adv(cslot, cpar, (uint32_t)(2 * nsl), nring);
        consumer_sync();
        if (s == 0) { DF_STAMP(8); DF_MARK(2); }
        // scores
        const int nk = (ntot + NRG - 1) / NRG;
        #pragma unroll 3
        for (int k = 0; k < nk; k++) {
            const int r = a_rg + k * NRG;
            const bool valid = a_rg < NRG && r < ntot;
            const int j = (r >= rps) + (r >= 2 * rps) + (r >= 3 * rps);
            const float* kr = (valid && r < nr) ? ringf + S.tile_off[j] + (r - j * rps) * DH : knew;
            float d0 = 0.0f, d1 = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; c++) if (c < CPT) {
                const float4 k4 = *reinterpret_cast<const float4*>(kr + (a_p + 8 * c) * 4);
                d0 = fmaf(qf[c].x, k4.x, d0); d1 = fmaf(qf[c].y, k4.y, d1); d0 = fmaf(qf[c].z, k4.z, d0); d1 = fmaf(qf[c].w, k4.w, d1);
            }
            float d = d0 + d1;
            d += __shfl_xor_sync(0xffffffffu, d, 1); d += __shfl_xor_sync(0xffffffffu, d, 2); d += __shfl_xor_sync(0xffffffffu, d, 4);
            if (valid && a_p == 0) sp[r * ATT_GP + a_i] = d * ph.scale;
        }
        consumer_sync();
        if (s == 0) DF_STAMP(9);
        if (tid < nsl) mbar_arrive(&S.empty[S.tile_slot[tid]]);
        // online softmax state per head
        if (warp < GRP) {
            const int i = warp;
            float tm = -INFINITY;
            for (int r = lane; r < ntot; r += 32) tm = fmaxf(tm, sp[r * ATT_GP + i]);
            tm = hx_warp_max(tm);
            const float mo = S.att_m[i], mn = fmaxf(mo, tm);
            float ls = 0.0f;
            for (int r = lane; r < ntot; r += 32) { const float pr = __expf(sp[r * ATT_GP + i] - mn); sp[r * ATT_GP + i] = pr; ls += pr; }
            ls = hx_warp_sum(ls);
            if (lane == 0) { const float rr = __expf(mo - mn); S.att_r[i] = rr; S.att_l[i] = S.att_l[i] * rr + ls; S.att_m[i] = mn; }
        }
        consumer_sync();
        if (s == 0) DF_STAMP(10);
        // P*V
        {
#pragma unroll
            for (int i = 0; i < GRP; i++) { const float rr = S.att_r[i]; acc[i].x *= rr; acc[i].y *= rr; acc[i].z *= rr; acc[i].w *= rr; }
            #pragma unroll 2
            for (int r = c_sub; r < ntot; r += NSUB) {
                const int j = (r >= rps) + (r >= 2 * rps) + (r >= 3 * rps);
                const float* vr = (r < nr) ? ringf + S.tile_off[4 + j] + (r - j * rps) * DH : vnew;
                const float4 v4 = *reinterpret_cast<const float4*>(vr + c_c * 4);
                const float4 pa = *reinterpret_cast<const float4*>(sp + r * ATT_GP);
                const float4 pb = GRP > 4 ? *reinterpret_cast<const float4*>(sp + r * ATT_GP + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float pw[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
                for (int i = 0; i < GRP; i++) {
                    acc[i].x = fmaf(pw[i], v4.x, acc[i].x); acc[i].y = fmaf(pw[i], v4.y, acc[i].y);
                    acc[i].z = fmaf(pw[i], v4.z, acc[i].z); acc[i].w = fmaf(pw[i], v4.w, acc[i].w);
                }
            }
        }
        consumer_sync();
        if (tid < nsl) mbar_arrive(&S.empty[S.tile_slot[nsl + tid]]);
    }
    DF_STAMP(11); DF_MARK(3);
    // fold the row subsets and hand the split's partial over
#pragma unroll
    for (int i = 0; i < GRP; i++) *reinterpret_cast<float4*>(accx + (c_sub * GRP + i) * DH + c_c * 4) = acc[i];
    consumer_sync();
    #pragma unroll 1
    for (int hd = tid; hd < HD; hd += NCT) {
        const int i = hd / DH, d = hd - i * DH;
        float O = 0.0f;
        for (int u = 0; u < NSUB; u++) O += accx[(u * GRP + i) * DH + d];
        const int hs = (ap.kv * GRP + i) * ns + ap.split;
        ll_st(ph.pacc_ll + (size_t)hs * DH + d, O, ep);
        if (d == 0) { ll_st(ph.pml_ll + 2 * hs, S.att_m[i], ep); ll_st(ph.pml_ll + 2 * hs + 1, S.att_l[i], ep); }
    }
    DF_MARK(4);
    attention_merge_df(P, ph, S, ap.kv, ap.split, ns, GRP, ep);
}

template <bool TP>
__global__ void __launch_bounds__(PT, 1) k_decode_df(const __grid_constant__ HxPersist P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    SmemDf& S = *reinterpret_cast<SmemDf*>(smem_raw);
    // swizzled operands need 1024-byte aligned cells (the swizzle is a function of the shared-memory address)
    uint8_t* sfb1 = smem_raw + ((sizeof(SmemDf) + 15) & ~(size_t)15);    // 512 bytes of 0x38 (scale 1.0)
    uint8_t* ring = smem_raw + (((smem_u32(smem_raw) + (uint32_t)sizeof(SmemDf) + 16u + 512u + 1023u) & ~1023u) - smem_u32(smem_raw));
    uint8_t* digb = ring + (size_t)P.tc_ring * HX_RING_SLOT;              // digit columns / attention scratch (1024-aligned)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, grid = gridDim.x;
    const int pos = *P.pos;
    const uint32_t nring = (uint32_t)P.tc_ring;

    if (tid == 0) {
        for (int i = 0; i < HX_TC_MAX_RING; i++) { mbar_init(&S.full[i], 1); mbar_init(&S.empty[i], 1); }
        mbar_init(&S.acc_full[0], 1); mbar_init(&S.acc_full[1], 1);
        mbar_init(&S.acc_empty[0], EPI_WARPS); mbar_init(&S.acc_empty[1], EPI_WARPS);
        mbar_init(&S.b_ready, 1);
        S.abort_flag = 0; S.wait_limit = P.wait_limit;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 128) reinterpret_cast<uint32_t*>(sfb1)[tid] = 0x38383838u;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == NCW + 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&S.tmem_base)), "n"(TM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = S.tmem_base;

    if (warp == NCW) {
        // =========================== producer ===========================
        if (lane == 0) {
            uint32_t slot = 0, par = 0, npush = 0;
            bool first_round = true;
            auto push = [&](const void* src, uint32_t bytes) -> bool {
                if (!first_round && !mbar_wait(&S.empty[slot], par, &S.abort_flag)) return false;
                mbar_expect_tx(&S.full[slot], bytes);
                bulk_g2s(ring + (size_t)slot * HX_RING_SLOT, src, bytes, &S.full[slot]);
                npush++;
                if (++slot == nring) { slot = 0; if (first_round) first_round = false; else par ^= 1u; }
                return true;
            };
            bool ok = true;
            int a_ns, a_trows, a_ntiles;
            const AttPlan ap = att_plan_df(P, cta, pos, (int)nring, &a_ns, &a_trows, &a_ntiles);
            HxPhase nxt = P.phases[0];
#pragma unroll 1
            for (int pi = 0; pi < P.nphases && ok; pi++) {
                const HxPhase ph = nxt;
                if (pi + 1 < P.nphases) {
                    nxt = P.phases[pi + 1];
                    // one CTA per phase pulls the small vectors of the next phase into L2 (a token's worth of weights
                    // has evicted them since their last use)
                    if (cta == (pi % grid)) {
                        const HxPhase& q = P.phases[pi + 1];
                        if (q.type == HX_PH_LINEAR_TC) {
                            if (q.norm == HX_NORM_RMS && q.g) l2_prefetch(q.g, (uint32_t)q.K * 4u);
                            if (q.epi == HX_EPI_QKV) {
                                if (q.qn_g) l2_prefetch(q.qn_g, (uint32_t)q.DH * 4u);
                                if (q.kn_g) l2_prefetch(q.kn_g, (uint32_t)q.DH * 4u);
                                if (q.cosT) { l2_prefetch(q.cosT + (size_t)pos * (q.DH >> 1), (uint32_t)q.DH * 2u); l2_prefetch(q.sinT + (size_t)pos * (q.DH >> 1), (uint32_t)q.DH * 2u); }
                            }
                        }
                    }
                }
                if (ph.type == HX_PH_LINEAR_TC) {
                    const int b0 = ph.plan[cta].b0, b1 = ph.plan[cta].b1;
                    const uint8_t* src = ph.w + (size_t)b0 * HX_T128_CELL;
#pragma unroll 1
                    for (int g = b0; g < b1 && ok; g++, src += HX_T128_CELL) ok = push(src, HX_T128_CELL);
                } else if (ph.type == HX_PH_ATTN) {
                    const size_t rowb = (size_t)ph.DH * 4;
                    // tiles of up to tr slots of K rows followed by as many of V rows (attention_df)
#pragma unroll 1
                    for (int t = 0; t < a_ntiles && ok; t++) {
                        const int r0 = ap.t0 + t * a_trows, nrt = min(a_trows, ap.t0 + ap.n_old - r0);
#pragma unroll 1
                        for (int kv2 = 0; kv2 < 2 && ok; kv2++) {
#pragma unroll 1
                            for (int r = 0; r < nrt && ok; r += ap.rows_per_slot) {
                                const size_t off = ((size_t)ap.kv * ph.cap + r0 + r) * ph.DH;
                                ok = push((kv2 ? ph.vc : ph.kc) + off, (uint32_t)(min(ap.rows_per_slot, nrt - r) * rowb));
                            }
                        }
                    }
                }
            }
            // the CTA must not end with a bulk copy of its own in flight: wait for the last copy into every slot
            const uint32_t first = npush > nring ? npush - nring : 0u;
            for (uint32_t j = first; j < npush; j++) {
                const uint32_t s = j % nring, pr = (j / nring) & 1u;
                for (uint32_t i = 0; i < DRAIN_LIMIT; i++) if (mbar_try(&S.full[s], pr)) break;
            }
        }
    } else if (warp == NCW + 1) {
        // =========================== MMA issuer ===========================
        if (lane == 0) {
            tc_cp_sf(tmem + TM_SFB, tc_desc(smem_u32(sfb1), 16, 128));
            const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(TC_NDIG >> 3) << 17) | (8u << 24);
            const uint64_t a_ring = tc_desc(smem_u32(ring), 16, 1024, TC_SW128);    // 8-row groups 1024 B apart, 128-byte swizzle
            const uint64_t sf_ring = tc_desc(smem_u32(ring) + 16384, 16, 128);
            const uint64_t b_base = tc_desc(smem_u32(digb), 16, 1024, TC_SW128);
            uint32_t slot = 0, par = 0, uc = 0, tcph = 0;
            bool ok = true;
            int a_ns, a_trows, a_ntiles;
            const AttPlan ap = att_plan_df(P, cta, pos, (int)nring, &a_ns, &a_trows, &a_ntiles);
#pragma unroll 1
            for (int pi = 0; pi < P.nphases && ok; pi++) {
                const HxPhase& ph = P.phases[pi];
                if (ph.type == HX_PH_LINEAR_TC) {
                    const HxCtaPlan tp = ph.plan[cta];
                    ok = mbar_wait(&S.b_ready, tcph & 1, &S.abort_flag);        // digit columns of this phase are in place
                    tcph++;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    unsigned long long dbg_wait = 0; (void)dbg_wait;
                    int kc = tp.k0, dp = 0;              // K cell of the tile, its position among the digit cells
                    bool fresh = true;
                    uint32_t dcol = 0;
#pragma unroll 1
                    for (int g = tp.b0; g < tp.b1 && ok; g++) {
                        if (fresh) {
                            const uint32_t buf = uc & 1u;
                            if (uc >= 2) ok = mbar_wait(&S.acc_empty[buf], ((uc >> 1) - 1) & 1, &S.abort_flag);
                            if (!ok) break;
                            dcol = tmem + TM_D0 + buf * TC_NDIG;
                        }
                        { DF_MMA_T0(); ok = mbar_wait(&S.full[slot], par, &S.abort_flag); DF_MMA_T1(); }
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        // descriptors advance in 16-byte units: a K step is 32 B of a swizzled row, a scale chunk 512 B
                        const uint64_t a_slot = a_ring + (uint64_t)(slot * (HX_RING_SLOT >> 4));
                        const uint64_t sf_slot = sf_ring + (uint64_t)(slot * (HX_RING_SLOT >> 4));
                        const uint64_t b_cell = b_base + (uint64_t)(dp * 128);
                        const uint32_t tsf = tmem + TM_SFA + slot * 16;
#pragma unroll
                        for (int e = 0; e < 4; e++) tc_cp_sf(tsf + e * 4, sf_slot + (uint64_t)(e * 32));
#pragma unroll
                        for (int e = 0; e < 4; e++)
                            tc_mma(dcol, a_slot + (uint64_t)(e * 2), b_cell + (uint64_t)(e * 2), idesc, tsf + e * 4, tmem + TM_SFB,
                                   (fresh && e == 0) ? 0u : 1u);
                        tc_commit(&S.empty[slot]);
                        fresh = false;
                        if (++slot == nring) { slot = 0; par ^= 1u; }
                        if (++dp == tp.C) dp = 0;
                        if (++kc == tp.C || g + 1 == tp.b1) {          // last cell of this tile's piece
                            tc_commit(&S.acc_full[uc & 1u]);
                            uc++; kc = 0; fresh = true;
                        }
                    }
                    DF_MMA_OUT();
                } else if (ph.type == HX_PH_ATTN) {
                    ring_adv(slot, par, 2u * (uint32_t)ap.nslots, nring);         // ring slots the consumers use for K and V rows
                }
            }
        }
    } else {
        // =============================== consumers ===============================
        uint32_t cslot = 0, cpar = 0, uc = 0;                 // ring cursor of the consumers (attention rows), accumulator use count
        float best_v = -INFINITY; int best_i = INT_MAX;
        if (tid == 0) S.ap = att_plan_df(P, cta, pos, (int)nring, &S.att_ns, &S.ap_tile_rows, &S.ap_ntiles);

        constexpr int PH_CHUNKS = (int)(sizeof(HxPhase) / 16);
        if (tid < PH_CHUNKS) reinterpret_cast<uint4*>(&S.ph[0])[tid] = __ldg(reinterpret_cast<const uint4*>(P.phases) + tid);
        if (P.inject_stall && tid == 0) (void)df_wait1(reinterpret_cast<const u64*>(P.err) + 1, 0xFFFFFFFFu, S, P);   // nothing ever writes this epoch
        if (consumer_sync_any(S.abort_flag)) goto aborted;
#pragma unroll 1
        for (int pi = 0; pi < P.nphases; pi++) {
            const HxPhase& ph = S.ph[pi & 1];
            const unsigned ep = P.ep_base + (unsigned)pi + 1u;
            DF_STAMP(0); DF_MARK(0);
            // the next descriptor travels to shared memory while this phase runs (its slot was last read a phase ago)
            if (pi + 1 < P.nphases && tid < PH_CHUNKS)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_u32(reinterpret_cast<uint4*>(&S.ph[(pi + 1) & 1]) + tid)),
                             "l"(reinterpret_cast<const uint4*>(P.phases + pi + 1) + tid) : "memory");
            if (ph.type == HX_PH_LINEAR_TC) {
                // ---------- prologue: x -> (norm) -> sixteen base-4 digit columns in operand layout ----------
                // Pass 1 stages the CTA's K slice of the input (times the norm gain) in shared memory behind the digit
                // cells and finds its largest magnitude; pass 2 turns the staged values into digit words.  The code runs
                // once per phase from a cold instruction cache, so it is kept small: one polling site, one digit site.
                const int K = ph.K;
                const HxCtaPlan tp = ph.plan[cta];
                const unsigned in_ep = P.ep_base + (unsigned)ph.in_dep + 1u;
                const bool rms = ph.norm == HX_NORM_RMS;
                // layer 0: the embedding row of the token is the input of qkv and the residual of o_proj
                const float* xrow = ph.tok ? ph.x + (size_t)(ph.tok[P.tok_by_pos ? pos : 0]) * (size_t)ph.res_ld : ph.x;
                const int nitems = tp.run * 32;
                float* xs = reinterpret_cast<float*>(digb + (size_t)tp.run * 2048);
                float ss = 0.0f, mx = 0.0f;
                {
                    // Sum of squares of the whole input: per-tile sums published by the producing epilogue, added in tile
                    // order (every CTA gets the same bits); layer 0 reads the embedding row itself.
                    if (rms && !ph.in_stat) {
                        #pragma unroll 1
                        for (int k = tid * 4; k < K; k += NCT * 4) {
                            const float4 a = __ldcg(reinterpret_cast<const float4*>(xrow + k));
                            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
                        }
                    }
                    // A unit is two consecutive elements (one 16-byte load), so a warp's load is 512 contiguous bytes.  UI
                    // units per thread and round are in flight together, with the norm gains fetched before the wait and,
                    // in the first round of warp 0, the per-tile sums of squares polled in the same breath.
                    constexpr int UI = 8;
                    const int nunits = nitems * 4;
                    #pragma unroll 1
                    for (int u0 = tid; u0 < nunits; u0 += UI * NCT) {
                        int kk[UI]; float2 gg[UI]; u64 w[UI][2];
#pragma unroll
                        for (int j = 0; j < UI; j++) {
                            const int u = u0 + j * NCT;
                            int kc = tp.k0 + (u >> 7); if (kc >= tp.C) kc -= tp.C;
                            const int k = kc * 256 + (u & 127) * 2;
                            kk[j] = (u < nunits && k < K) ? k : -1;
                            gg[j] = (rms && kk[j] >= 0) ? *reinterpret_cast<const float2*>(ph.g + k) : make_float2(1.0f, 1.0f);
                            w[j][0] = w[j][1] = 0;
                        }
                        const bool stat_round = rms && ph.in_stat != nullptr && warp == 0 && u0 == tid;
                        const bool st_a = stat_round && lane < ph.n_in_stat, st_b = stat_round && lane + 32 < ph.n_in_stat;
                        u64 sa = 0, sb = 0;
                        if (ph.in_ll) {
                            const unsigned lim = S.abort_flag ? 1u : S.wait_limit;
                            bool ok = false;
                            #pragma unroll 1
                            for (unsigned t = 0; t < lim && !ok; t++) {
#pragma unroll
                                for (int j = 0; j < UI; j++) if (kk[j] >= 0) ll_ld2(ph.in_ll + kk[j], w[j][0], w[j][1]);
                                if (st_a) sa = ll_ld(ph.in_stat + lane);
                                if (st_b) sb = ll_ld(ph.in_stat + lane + 32);
                                ok = (!st_a || ll_ok(sa, in_ep)) && (!st_b || ll_ok(sb, in_ep));
#pragma unroll
                                for (int j = 0; j < UI; j++) if (kk[j] >= 0) ok = ok && ll_ok(w[j][0], in_ep) && ll_ok(w[j][1], in_ep);
                                if (!ok && (t & 63u) == 63u && df_gave_up(S, P)) break;
                            }
                            if (!ok) df_fail(S, P);
                        } else {
#pragma unroll
                            for (int j = 0; j < UI; j++) if (kk[j] >= 0) {
                                const float2 a = __ldcg(reinterpret_cast<const float2*>(xrow + kk[j]));
                                w[j][0] = __float_as_uint(a.x); w[j][1] = __float_as_uint(a.y);
                            }
                        }
                        if (st_a) ss += ll_val(sa);
                        if (st_b) ss += ll_val(sb);
#pragma unroll
                        for (int j = 0; j < UI; j++) {
                            const int u = u0 + j * NCT;
                            if (u >= nunits) continue;
                            const float v0 = kk[j] >= 0 ? ll_val(w[j][0]) * gg[j].x : 0.0f, v1 = kk[j] >= 0 ? ll_val(w[j][1]) * gg[j].y : 0.0f;
                            mx = fmaxf(mx, fmaxf(fabsf(v0), fabsf(v1)));
                            *reinterpret_cast<float2*>(xs + u * 2) = make_float2(v0, v1);
                        }
                    }
                }
                DF_MARK(1);
                ss = hx_warp_sum(ss); mx = hx_warp_max(mx);
                if (lane == 0) { S.red[warp] = ss; S.red[NCW + warp] = mx; }
                consumer_sync();
                float inv = 1.0f, Sg = 1.0f;
                {
                    float tss = 0.0f, tmx = 0.0f;
#pragma unroll
                    for (int i = 0; i < NCW; i++) { tss += S.red[i]; tmx = fmaxf(tmx, S.red[NCW + i]); }
                    if (rms) inv = rsqrtf(tss / (float)K + ph.eps);
                    const float vmax = tmx * inv * 1.0000005f;            // margin for the rounding of x*g*inv
                    if (vmax > 0.0f && vmax < INFINITY) Sg = __uint_as_float(__float_as_uint(vmax) & 0x7F800000u);   // vmax/Sg in [1,2)
                }
                DF_STAMP(14);
                const float mul = (inv / Sg) * 2147483648.0f;             // |x_n| / Sg * 2^31 < 2^32
                #pragma unroll 1
                for (int it = tid; it < nitems; it += NCT) {
                    const float4 va = *reinterpret_cast<const float4*>(xs + it * 8), vb = *reinterpret_cast<const float4*>(xs + it * 8 + 4);
                    const float v[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
                    uint32_t M[8]; uint32_t sg = 0u;
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        M[e] = __float2uint_rn(fabsf(v[e]) * mul);
                        sg |= (v[e] < 0.0f ? 8u : 0u) << (4 * e);
                    }
                    // digit n of element e is bits 31-2n, 30-2n of M[e]; it lands on bits 4e+1, 4e of the word of row n
                    const int j = (it >> 2) & 7, w = it & 3;               // 16-byte chunk and word of this item in its cell
                    uint8_t* dst = digb + (size_t)(it >> 5) * 2048 + w * 4;
                    uint32_t rowv[16];
                    hx_digit_rows(M, sg, rowv);
#pragma unroll
                    for (int n = 0; n < TC_NDIG; n++) *reinterpret_cast<uint32_t*>(dst + n * 128 + ((j ^ (n & 7)) << 4)) = rowv[n];
                }
                DF_STAMP(15);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                consumer_sync();
                if (tid == 0) mbar_arrive(&S.b_ready);
                DF_STAMP(1); DF_MARK(2);

                // ---------- pieces of tiles: accumulator -> digits recombined -> merge -> epilogue ----------
                ring_adv(cslot, cpar, (uint32_t)(tp.b1 - tp.b0), nring);
                const int t_first = tp.t_first, t_last = tp.t_last;
                if (warp < EPI_WARPS) {
                    const float out_scale = Sg;       // x_n = Sg * sum_j 4^-j * (digit_j / 2), and digit/2 is the E2M1 value
                    const int rl = warp * 32 + lane;
                    const unsigned res_ep = P.ep_base + (unsigned)ph.res_dep + 1u;
#pragma unroll 1
                    for (int tile = t_first; tile <= t_last; tile++) {
                        const uint32_t buf = uc & 1u;
                        // the CTA holding a tile's first cell merges it (see HxCtaPlan)
                        const bool merger = tile > t_first || tp.first_merger;
                        const int others = tile == t_last ? tp.last_others : 0;
                        // operands of the epilogue that are final already travel while the MMAs of this piece run
                        float yres = 0.0f;
                        if (merger && ph.epi == HX_EPI_RESID && tile * 128 + rl < ph.N)
                            yres = ph.res_ll ? df_wait1(ph.res_ll + tile * 128 + rl, res_ep, S, P) : __ldcg(xrow + tile * 128 + rl);
                        float pre_g = 1.0f, pre_cs = 1.0f, pre_sn = 0.0f;
                        if (merger && ph.epi == HX_EPI_QKV) {
                            const int row = tile * 128 + rl, e = row % ph.DH, half = ph.DH >> 1;
                            const int sec = row < ph.NH * ph.DH ? 0 : (row < (ph.NH + ph.NKV) * ph.DH ? 1 : 2);
                            const float* gg = sec == 0 ? ph.qn_g : (sec == 1 ? ph.kn_g : nullptr);
                            if (gg) pre_g = gg[e];
                            if (ph.cosT) { pre_cs = ph.cosT[(size_t)pos * half + (e < half ? e : e - half)]; pre_sn = ph.sinT[(size_t)pos * half + (e < half ? e : e - half)]; }
                        }
                        mbar_wait(&S.acc_full[buf], (uc >> 1) & 1, &S.abort_flag);
                        uc++;
                        if (tile == t_last) DF_MARK(3);
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        uint32_t r[16];
                        const uint32_t ta = tmem + ((uint32_t)(warp * 32) << 16) + TM_D0 + buf * TC_NDIG;
                        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                                       "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                                     : "r"(ta));
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&S.acc_empty[buf]);
                        float v = 0.0f;
#pragma unroll
                        for (int j = TC_NDIG - 1; j >= 0; j--) v = fmaf(v, 0.25f, __uint_as_float(r[j]));
                        v *= out_scale;
                        if (!merger) {            // pieces 1.. hand their rows to the merger
                            ll_st(ph.part_ll + ((size_t)tile * ph.pieces + (size_t)tp.first_piece) * 128 + rl, v, ep);
                            continue;
                        }
                        #pragma unroll 1
                        for (int q = 0; q < others; q += 4)
                            v = df_wait_add4(ph.part_ll + ((size_t)tile * ph.pieces + (size_t)q) * 128 + rl, 128, min(4, others - q), ep, v, S, P);
                        if (tile == t_last) DF_MARK(4);
                        if (ph.epi == HX_EPI_QKV) {
                            // A tile holds 128 / DH whole heads (DH is 32, 64 or 128).  Per-head RMSNorm and rotate_half
                            // RoPE on q and k; q leaves as pairs, k and v as pairs and into the cache row of this position.
                            const int DH = ph.DH, half = DH >> 1, QD = ph.NH * DH, KVD = ph.NKV * DH;
                            const int row = tile * 128 + rl;
                            const bool valid = row < ph.N;
                            const int sec = row < QD ? 0 : (row < QD + KVD ? 1 : 2);
                            const int e = row % DH;
                            v = valid ? v * ph.ts[sec] : 0.0f;
                            const float* gg = sec == 0 ? ph.qn_g : (sec == 1 ? ph.kn_g : nullptr);
                            float ssq = hx_warp_sum(v * v);
                            if (DH > 32) {
                                if (lane == 0) S.swi[warp] = ssq;
                                epi_sync();
                                const int w0 = (rl / DH) * (DH >> 5);
                                ssq = 0.0f;
                                for (int j = 0; j < (DH >> 5); j++) ssq += S.swi[w0 + j];
                                epi_sync();
                            }
                            if (gg) v = pre_g * (v * rsqrtf(ssq / (float)DH + ph.eps));
                            if (ph.cosT) {                       // every thread meets the barriers, v rows keep their value
                                S.swi[rl] = v;
                                epi_sync();
                                const float other = S.swi[e < half ? rl + half : rl - half];
                                if (sec < 2) v = e < half ? v * pre_cs - other * pre_sn : v * pre_cs + other * pre_sn;
                                epi_sync();
                            }
                            if (valid) {
                                if (sec == 0) ll_st(ph.out_ll + row, v, ep);
                                else {
                                    const int hrow = row - QD - (sec == 2 ? KVD : 0);
                                    float* dst = sec == 1 ? ph.kc : ph.vc;
                                    dst[((size_t)(hrow / DH) * ph.cap + pos) * DH + e] = v;
                                    ll_st(ph.kv_ll + (sec == 2 ? KVD : 0) + hrow, v, ep);
                                }
                            }
                        } else if (ph.epi == HX_EPI_SWIGLU) {
                            // rows 0..63 of a tile are gate rows, 64..127 the matching up rows
                            S.swi[rl] = v * (rl < 64 ? ph.ts[0] : ph.ts[1]);
                            epi_sync();
                            const int hi = tile * 64 + rl;
                            if (rl < 64 && hi < ph.N) ll_st(ph.out_ll + hi, pz_silu_mul(S.swi[rl], S.swi[rl + 64]), ep);
                            epi_sync();
                        } else {
                            const int row = tile * 128 + rl;
                            const bool valid = row < ph.N;
                            v *= (row < ph.bound0) ? ph.ts[0] : (row < ph.bound1 ? ph.ts[1] : ph.ts[2]);
                            if (ph.epi == HX_EPI_RESID) {
                                if (TP && ph.tp_partial) {
                                    // row-split linear: this rank's partial row goes to every rank's exchange buffer, then the
                                    // ranks' rows are added in rank order -- the same bits on every rank
                                    const size_t o = ((size_t)(ph.tp_partial - 1) * P.tp_world) * P.tp_dm + row;
                                    if (valid) for (int w = 0; w < P.tp_world; w++)
                                        if (w != P.tp_rank) ll_st_sys(P.tp_x[w] + o + (size_t)P.tp_rank * P.tp_dm, v, ep);
                                    float sum = 0.0f;
                                    if (valid) for (int w = 0; w < P.tp_world; w++)
                                        sum += (w == P.tp_rank) ? v : df_wait1<true>(P.tp_x[P.tp_rank] + o + (size_t)w * P.tp_dm, ep, S, P);
                                    v = sum;
                                }
                                v = valid ? yres + v : 0.0f;
                                if (valid) ll_st(ph.out_ll + row, v, ep);
                                // this tile's share of the next norm's sum of squares
                                const float ssq = hx_warp_sum(v * v);
                                if (lane == 0) S.swi[warp] = ssq;
                                epi_sync();
                                if (rl == 0) ll_st(ph.out_stat + tile, (S.swi[0] + S.swi[1]) + (S.swi[2] + S.swi[3]), ep);
                                epi_sync();
                            } else if (valid) {
                                ph.y[row] = v;
                                if (ph.epi == HX_EPI_ARGMAX && pz_better(v, row, best_v, best_i)) { best_v = v; best_i = row; }
                            }
                        }
                    }
                } else uc += (uint32_t)(t_last - t_first + 1);
                if (ph.epi == HX_EPI_ARGMAX) {
                    // per-CTA best (held by warps 0-3), then the last CTA to arrive folds all of them
#pragma unroll
                    for (int d = 16; d >= 1; d >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, best_v, d);
                        const int oi = __shfl_xor_sync(0xffffffffu, best_i, d);
                        if (pz_better(ov, oi, best_v, best_i)) { best_v = ov; best_i = oi; }
                    }
                    if (lane == 0) { S.bv[warp] = best_v; S.bi[warp] = best_i; }
                    consumer_sync();
                    if (tid == 0) {
                        float bv = S.bv[0]; int bi = S.bi[0];
                        for (int i = 1; i < 4; i++) if (pz_better(S.bv[i], S.bi[i], bv, bi)) { bv = S.bv[i]; bi = S.bi[i]; }
                        P.am_val[cta] = bv; P.am_idx[cta] = bi;
                        S.ticket = S.abort_flag ? 0u : ticket_acq_rel(P.am_cnt);       // an aborting CTA never finishes the token
                    }
                    consumer_sync();
                    if (S.ticket == (unsigned)grid - 1 && warp == 0) {
                        float bv = -INFINITY; int bi = INT_MAX;
                        for (int i = lane; i < grid; i += 32) {
                            const float ov = __ldcg(P.am_val + i); const int oi = __ldcg(P.am_idx + i);
                            if (pz_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
                        }
#pragma unroll
                        for (int d = 16; d >= 1; d >>= 1) {
                            const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
                            const int oi = __shfl_xor_sync(0xffffffffu, bi, d);
                            if (pz_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
                        }
                        if (TP && lane == 0 && P.tp_world > 1) {
                            // vocabulary split over the ranks: exchange (value, global index) and take the best of all
                            const size_t ao = (size_t)2 * P.tp_world * P.tp_dm;
                            const int gi = bi == INT_MAX ? INT_MAX : bi + P.tp_vocab_off;
                            for (int w = 0; w < P.tp_world; w++) if (w != P.tp_rank) {
                                ll_st_sys(P.tp_x[w] + ao + 2 * P.tp_rank, bv, ep);
                                ll_st_sys(P.tp_x[w] + ao + 2 * P.tp_rank + 1, __int_as_float(gi), ep);
                            }
                            float fv = bv; int fi = gi;
                            for (int w = 0; w < P.tp_world; w++) if (w != P.tp_rank) {
                                const float ov = df_wait1<true>(P.tp_x[P.tp_rank] + ao + 2 * w, ep, S, P);
                                const int oi = __float_as_int(df_wait1<true>(P.tp_x[P.tp_rank] + ao + 2 * w + 1, ep, S, P));
                                if (pz_better(ov, oi, fv, fi)) { fv = ov; fi = oi; }
                            }
                            bv = fv; bi = fi;
                        }
                        if (lane == 0) {
                            const int nt = (bi == INT_MAX) ? 0 : bi;
                            *P.next_tok = nt;
                            *P.pos_inc = pos + 1;
                            if (P.hist) P.hist[pos + 1] = nt;
                            *P.am_cnt = 0u;
                        }
                    }
                }
            } else if (ph.type == HX_PH_ATTN) {
                switch (ph.NH / ph.NKV) {
                    case 1: attention_df<1>(P, ph, S, ring, digb, cslot, cpar, pi, pos); break;
                    case 2: attention_df<2>(P, ph, S, ring, digb, cslot, cpar, pi, pos); break;
                    case 3: attention_df<3>(P, ph, S, ring, digb, cslot, cpar, pi, pos); break;
                    case 4: attention_df<4>(P, ph, S, ring, digb, cslot, cpar, pi, pos); break;
                    case 5: attention_df<5>(P, ph, S, ring, digb, cslot, cpar, pi, pos); break;
                    case 6: attention_df<6>(P, ph, S, ring, digb, cslot, cpar, pi, pos); break;
                    case 7: attention_df<7>(P, ph, S, ring, digb, cslot, cpar, pi, pos); break;
                    default: attention_df<8>(P, ph, S, ring, digb, cslot, cpar, pi, pos); break;
                }
            }
            DF_STAMP(2); DF_MARK(5);
            // ---------- phase boundary: the digit columns and the attention scratch are free again ----------
            asm volatile("cp.async.wait_all;" ::: "memory");
            if (consumer_sync_any(S.abort_flag)) goto aborted;
            DF_STAMP(3);
        }
        if (P.advance_pos && tid == 0) {
            // no lm_head in this launch: the last CTA to finish advances the position
            if (ticket_acq_rel(P.done_cnt) == (unsigned)grid - 1) { *P.pos_inc = pos + 1; *P.done_cnt = 0u; }
        }
        goto done;
aborted:
        if (tid == 0) { S.abort_flag = 1; *P.err = 1; }
done:   ;
    }
    // every role meets here; the MMA warp then releases the tensor memory
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == NCW + 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "n"(TM_COLS) : "memory");
}

size_t df_smem_fixed(int bdig_bytes) {
    return ((sizeof(SmemDf) + 15) & ~(size_t)15) + 512 + 1024 + (size_t)bdig_bytes;      // + ring slots
}

}  // namespace

// Shared-memory scratch of the attention phase for a group of `grp` query heads per kv head (queries, the position's k
// and v, probabilities, partial outputs of the row subsets); the digit columns share the space.
int hx_decode_df_att_bytes(int grp) { return (8 * 256 + 256 + 256 + 160 * ATT_GP + NCT * 4 * grp) * 4; }

// Ring depth that fits beside the digit columns (0 = does not fit).
int hx_decode_df_ring(int bdig_bytes) {
    const size_t fixed = df_smem_fixed(bdig_bytes);
    if (fixed + 3 * (size_t)HX_RING_SLOT > 227 * 1024) return 0;
    size_t n = (227 * 1024 - fixed) / HX_RING_SLOT;
    return (int)(n > HX_TC_MAX_RING ? HX_TC_MAX_RING : n);
}

int hx_decode_df_prepare() {
    HX_CUDA(cudaFuncSetAttribute(k_decode_df<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    HX_CUDA(cudaFuncSetAttribute(k_decode_df<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    return HX_OK;
}

int hx_decode_df_launch(const HxPersist& p, int grid, cudaStream_t st) {
    if (p.tc_ring < 3 || p.tc_ring > HX_TC_MAX_RING) return hx_fail(HX_ERR_ARG, "dataflow decode: ring depth %d", p.tc_ring);
    const size_t smem = df_smem_fixed(p.bdig_bytes) + (size_t)p.tc_ring * HX_RING_SLOT;
    if (smem > 227 * 1024) return hx_fail(HX_ERR_ARG, "dataflow decode needs %zu bytes of shared memory", smem);
    void* args[] = {(void*)&p};
    void* fn = p.tp_world > 1 ? (void*)k_decode_df<true> : (void*)k_decode_df<false>;
    HX_CUDA(cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(PT), args, smem, st));
    HX_COUNT_LAUNCH(1);
    return HX_OK;
}
