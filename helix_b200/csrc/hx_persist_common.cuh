// hx_persist_common.cuh -- pieces shared by the persistent decode kernels: mbarrier / bulk-copy helpers,
// the attention work split and the attention phase.  The including file defines RING_SLOTS (ring depth), NCW (consumer warps),
// NCT (consumer threads), WAIT_LIMIT and a shared-memory struct with the members used below.
#pragma once
#include "hx_persist.cuh"
#include "hx_kernels.cuh"
#include <cuda_fp16.h>
#include <limits.h>

// ------------------------------------------------------------------------------------------------
// PTX helpers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* b, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait; returns false (and latches *abort) when the limit is hit or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
        if (mbar_try(b, parity)) return true;
        if ((i & 1023) == 1023 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// asks L2 to fetch [p, p+bytes): p 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void l2_prefetch(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(p), "r"(bytes) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" :: "n"(NCT) : "memory"); }

__device__ __forceinline__ float pz_silu_mul(float g, float u) {
    const float sgn = g < 0.0f ? -1.0f : 1.0f;
    const float e = __expf(-(sgn * g));
    const float th = sgn * ((1.0f - e) / (1.0f + e));
    return g * (0.5f * (1.0f + th)) * u;
}
__device__ __forceinline__ bool pz_better(float av, int ai, float bv, int bi) { return av > bv || (av == bv && ai < bi); }

// Digit rows of eight consecutive elements.  M[e] = |x_e| / S * 2^31 (32 bits = sixteen base-4 digits, most significant
// first), sg = sign bits (bit 4e+3 set when x_e < 0).  row[n] = the 32-bit word of digit row n: nibble e holds digit n of
// element e as an E2M1 code (value digit/2), with the sign bit on non-zero digits.  Each halfword is spread to one digit
// per nibble, then an 8 x 8 nibble transpose turns "element-major" into "digit-major".
__device__ __forceinline__ void hx_digit_rows(const uint32_t (&M)[8], uint32_t sg, uint32_t (&row)[16]) {
    uint32_t hi[8], lo[8];
#pragma unroll
    for (int e = 0; e < 8; e++) {
        uint32_t a = M[e] >> 16, b = M[e] & 0xFFFFu;
        a = (a | (a << 8)) & 0x00FF00FFu; b = (b | (b << 8)) & 0x00FF00FFu;
        a = (a | (a << 4)) & 0x0F0F0F0Fu; b = (b | (b << 4)) & 0x0F0F0F0Fu;
        hi[e] = (a | (a << 2)) & 0x33333333u; lo[e] = (b | (b << 2)) & 0x33333333u;
    }
    auto transpose = [](uint32_t (&a)[8]) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) { const uint32_t t = ((a[i] >> 4) ^ a[i + 1]) & 0x0F0F0F0Fu; a[i + 1] ^= t; a[i] ^= t << 4; }
#pragma unroll
        for (int q = 0; q < 4; q++) { const int i = (q & 1) + (q >> 1) * 4; const uint32_t t = ((a[i] >> 8) ^ a[i + 2]) & 0x00FF00FFu; a[i + 2] ^= t; a[i] ^= t << 8; }
#pragma unroll
        for (int i = 0; i < 4; i++) { const uint32_t t = ((a[i] >> 16) ^ a[i + 4]) & 0x0000FFFFu; a[i + 4] ^= t; a[i] ^= t << 16; }
    };
    transpose(hi); transpose(lo);
#pragma unroll
    for (int n = 0; n < 16; n++) {
        uint32_t w = n < 8 ? hi[7 - n] : lo[15 - n];
        const uint32_t nz = (w | (w >> 1)) & 0x11111111u;       // a zero digit carries no sign
        row[n] = w | (sg & (nz << 3));
    }
}

struct AttPlan { int active, kv, split, t0, t1, n_old, rows_per_slot, nslots, has_new; };
__device__ __forceinline__ AttPlan att_plan(const HxPhase& ph, int cta, int pos) {
    AttPlan a;
    a.active = cta < ph.NKV * ph.nsplit;
    a.kv = cta / ph.nsplit; a.split = cta % ph.nsplit;
    const int T = pos + 1, chunk = (T + ph.nsplit - 1) / ph.nsplit;
    a.t0 = a.split * chunk; a.t1 = min(T, a.t0 + chunk);
    if (!a.active || a.t0 >= a.t1) { a.t0 = a.t1 = 0; a.n_old = 0; a.has_new = 0; }
    else { a.has_new = (pos >= a.t0 && pos < a.t1); a.n_old = (a.t1 - a.t0) - a.has_new; }
    a.rows_per_slot = HX_RING_SLOT / (ph.DH * 4);
    a.nslots = (a.n_old + a.rows_per_slot - 1) / a.rows_per_slot;      // K slots == V slots
    return a;
}

#ifdef HX_DEBUG_STAMPS
#define STAMP_ALL() do { if (P.dbg_all && tid == 0) { unsigned long long _t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t)); P.dbg_all[(size_t)pi * gridDim.x + blockIdx.x] = _t; } } while (0)
#define STAMP(i) do { if (P.dbg && cta == P.dbg_cta && tid == 0) { unsigned long long _t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t)); P.dbg[pi * 16 + (i)] = _t; } } while (0)
#else
#define STAMP_ALL() do { } while (0)
#define STAMP(i) do { } while (0)
#endif

// ------------------------------------------------------------------------------------------------
// Attention phase of one CTA: (kv head, split of the cached positions); the GRP query heads of the kv
// head share the K and V rows.  Kept out of line and specialised per group size so that only the
// variant in use occupies the instruction cache.
// ------------------------------------------------------------------------------------------------
template <int GRP, int ARR, class SM>
__device__ __noinline__ bool attention_phase(const HxPersist& P, const HxPhase& ph, SM& S, uint8_t* ring, uint8_t* digb,
                                             uint32_t& ctr, int pi, int pos) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, cta = blockIdx.x;
    const AttPlan ap = att_plan(ph, cta, pos);
    const int DH = ph.DH, half = DH >> 1;
    float* sq = reinterpret_cast<float*>(digb);                 // [GRP][DH] rotated queries
    float* knew = sq + 8 * 256;                                  // [DH] current k (normed, rotated)
    float* vnew = knew + 256;                                    // [DH]
    float* sp = vnew + 256;                                      // [GRP][rows_per_slot + 1] scores / probabilities
    float* accx = sp + 8 * 160;                                  // [nsub][GRP][DH] partial outputs
    const int spitch = ap.rows_per_slot + 1;
    const int nsub = NCT / DH;                                   // threads per output dimension
    const int d = tid % DH, sub = tid / DH;
    float acc[GRP];
#pragma unroll
    for (int i = 0; i < GRP; i++) acc[i] = 0.0f;
    if (ap.active && ap.t1 > ap.t0) {
        // q (GRP heads) and, where the current position falls in this split, k and v:
        // per-head RMSNorm then rotate_half RoPE with table row pos (all loads of a lane first)
        const int nvec = GRP + (ap.has_new ? 2 : 0);
        #pragma unroll 1
        for (int v = warp; v < nvec; v += NCW) {
            const bool isq = v < GRP, isv = v == GRP + 1;
            const float* src = isq ? ph.qkv + (size_t)(ap.kv * GRP + v) * DH
                                   : ph.qkv + (size_t)ph.NH * DH + (size_t)(isv ? ph.NKV : 0) * DH + (size_t)ap.kv * DH;
            const float* gg = isv ? nullptr : (isq ? ph.qn_g : ph.kn_g);
            float* dst = isq ? sq + v * DH : (isv ? vnew : knew);
            float xv[8];
            float ssq = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++) { const int e = lane + 32 * j; xv[j] = e < DH ? __ldcg(src + e) : 0.0f; ssq = fmaf(xv[j], xv[j], ssq); }
            ssq = hx_warp_sum(ssq);
            const float inv = gg ? rsqrtf(ssq / (float)DH + ph.eps) : 1.0f;
#pragma unroll
            for (int j = 0; j < 8; j++) { const int e = lane + 32 * j; if (e < DH) dst[e] = gg ? gg[e] * (xv[j] * inv) : xv[j]; }
            __syncwarp();
            if (ph.cosT && !isv) {
                for (int e = lane; e < half; e += 32) {
                    const float lo = dst[e], hi = dst[e + half];
                    const float cs = ph.cosT[(size_t)pos * half + e], sn = ph.sinT[(size_t)pos * half + e];
                    dst[e] = lo * cs - hi * sn; dst[e + half] = hi * cs + lo * sn;
                }
            }
        }
        if (tid < 8) { S.att_m[tid] = -100000000.0f; S.att_l[tid] = 0.0f; }
        consumer_sync();
        STAMP(4);
        if (ap.has_new) {        // append to the cache for the tokens to come
            const size_t o = ((size_t)ap.kv * ph.cap + pos) * DH;
            for (int e = tid; e < DH; e += NCT) { ph.kc[o + e] = knew[e]; ph.vc[o + e] = vnew[e]; }
        }
        const int ntile = ap.nslots + ((ap.has_new && ap.n_old % ap.rows_per_slot == 0) ? 1 : 0);
        #pragma unroll 1
        for (int s = 0; s < ntile; s++) {
            const bool ring_tile = s < ap.nslots;
            int nr = ring_tile ? min(ap.rows_per_slot, ap.n_old - s * ap.rows_per_slot) : 0;
            // the current position rides on the last tile (room is guaranteed: spitch = rows + 1)
            const bool add_new = ap.has_new && (s == ntile - 1);
            uint32_t kslot = 0, vslot = 0;
            const float* kt = nullptr; const float* vt = nullptr;
            if (ring_tile) {
                kslot = ctr % RING_SLOTS; const uint32_t kround = ctr / RING_SLOTS; ctr++;
                if (!mbar_wait(&S.full[kslot], kround & 1, &S.abort_flag)) return false;
                kt = reinterpret_cast<const float*>(ring + (size_t)kslot * HX_RING_SLOT);
            }
            if (s == 0) STAMP(8);
            const int ntot = nr + (add_new ? 1 : 0);
            // scores: a warp per position, lanes over the head dimension
            #pragma unroll 1
            for (int r = warp; r < ntot; r += NCW) {
                const float* kr = (r < nr) ? kt + (size_t)r * DH : knew;
                float dot[GRP];
#pragma unroll
                for (int i = 0; i < GRP; i++) dot[i] = 0.0f;
                #pragma unroll 1
                for (int e = lane * 4; e < DH; e += 128) {
                    const float4 k4 = *reinterpret_cast<const float4*>(kr + e);
#pragma unroll
                    for (int i = 0; i < GRP; i++) {
                        const float4 q4 = *reinterpret_cast<const float4*>(sq + i * DH + e);
                        dot[i] = fmaf(q4.x, k4.x, dot[i]); dot[i] = fmaf(q4.y, k4.y, dot[i]);
                        dot[i] = fmaf(q4.z, k4.z, dot[i]); dot[i] = fmaf(q4.w, k4.w, dot[i]);
                    }
                }
#pragma unroll
                for (int i = 0; i < GRP; i++) {
                    const float sc = hx_warp_sum(dot[i]);
                    if (lane == 0) sp[i * spitch + r] = sc * ph.scale;
                }
            }
            __syncwarp();
            if (ARR != 1 && ring_tile && lane == 0) mbar_arrive(&S.empty[kslot]);
            consumer_sync();
            if (ARR == 1 && ring_tile && tid == 0) mbar_arrive(&S.empty[kslot]);
            if (s == 0) STAMP(9);
            // online softmax state per head (fused_decode_attn_kernel.hx:74-102)
            #pragma unroll 1
            for (int i = warp; i < GRP; i += NCW) {
                float tm = -INFINITY;
                for (int r = lane; r < ntot; r += 32) tm = fmaxf(tm, sp[i * spitch + r]);
                tm = hx_warp_max(tm);
                const float mo = S.att_m[i], mn = fmaxf(mo, tm);
                float ls = 0.0f;
                for (int r = lane; r < ntot; r += 32) { const float pr = __expf(sp[i * spitch + r] - mn); sp[i * spitch + r] = pr; ls += pr; }
                ls = hx_warp_sum(ls);
                if (lane == 0) { const float rr = __expf(mo - mn); S.att_r[i] = rr; S.att_l[i] = S.att_l[i] * rr + ls; S.att_m[i] = mn; }
            }
            consumer_sync();
            if (ring_tile) {
                vslot = ctr % RING_SLOTS; const uint32_t vround = ctr / RING_SLOTS; ctr++;
                if (!mbar_wait(&S.full[vslot], vround & 1, &S.abort_flag)) return false;
                vt = reinterpret_cast<const float*>(ring + (size_t)vslot * HX_RING_SLOT);
            }
            if (s == 0) STAMP(10);
#pragma unroll
            for (int i = 0; i < GRP; i++) acc[i] *= S.att_r[i];
            #pragma unroll 1
            for (int r = sub; r < ntot; r += nsub) {
                const float vv = (r < nr) ? vt[(size_t)r * DH + d] : vnew[d];
#pragma unroll
                for (int i = 0; i < GRP; i++) acc[i] = fmaf(sp[i * spitch + r], vv, acc[i]);
            }
            __syncwarp();
            if (ARR != 1 && ring_tile && lane == 0) mbar_arrive(&S.empty[vslot]);
            consumer_sync();
            if (ARR == 1 && ring_tile && tid == 0) mbar_arrive(&S.empty[vslot]);
        }
        STAMP(5);
        // fold the position subsets, write this split's partial
#pragma unroll
        for (int i = 0; i < GRP; i++) accx[(sub * 8 + i) * DH + d] = acc[i];
        consumer_sync();
        if (sub == 0) {
#pragma unroll
            for (int i = 0; i < GRP; i++) {
                float v = 0.0f;
                for (int u = 0; u < nsub; u++) v += accx[(u * 8 + i) * DH + d];
                const size_t hs = (size_t)(ap.kv * GRP + i) * ph.nsplit + ap.split;
                P.part_acc[hs * DH + d] = v;
                if (d == 0) { P.part_m[hs] = S.att_m[i]; P.part_l[hs] = S.att_l[i]; }
            }
        }
    } else if (ap.active) {
        // empty split: neutral partial
        for (int i = tid; i < GRP; i += NCT) {
            const size_t hs = (size_t)(ap.kv * GRP + i) * ph.nsplit + ap.split;
            P.part_m[hs] = -100000000.0f; P.part_l[hs] = 0.0f;
        }
        for (int i = tid; i < GRP * DH; i += NCT) {
            const size_t hs = (size_t)(ap.kv * GRP + i / DH) * ph.nsplit + ap.split;
            P.part_acc[hs * DH + i % DH] = 0.0f;
        }
    }
    if (ap.active) {
        STAMP(6);
        __threadfence();
        consumer_sync();
        if (tid == 0) S.ticket = atomicAdd(P.attn_cnt + ap.kv, 1u);
        consumer_sync();
        STAMP(7);
        if (S.ticket == (unsigned)ph.nsplit - 1) {
            __threadfence();
            // merge of the splits: weights w_s = exp(m_s - M) / sum_s l_s exp(m_s - M), then one pass
            // of independent loads over the partial outputs
            float* wgt = sp;                                   // [GRP][nsplit]
            const size_t hbase = (size_t)(ap.kv * GRP) * ph.nsplit;
            #pragma unroll 1
            for (int i = warp; i < GRP; i += NCW) {
                float mv[2], lv[2];
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int sidx = lane + 32 * j;
                    mv[j] = sidx < ph.nsplit ? __ldcg(P.part_m + hbase + (size_t)i * ph.nsplit + sidx) : -INFINITY;
                    lv[j] = sidx < ph.nsplit ? __ldcg(P.part_l + hbase + (size_t)i * ph.nsplit + sidx) : 0.0f;
                }
                const float M = hx_warp_max(fmaxf(mv[0], mv[1]));
                const float w0 = __expf(mv[0] - M), w1 = __expf(mv[1] - M);
                const float Lsum = hx_warp_sum(lv[0] * w0 + lv[1] * w1);
                if (lane < ph.nsplit) wgt[i * ph.nsplit + lane] = w0 / Lsum;
                if (lane + 32 < ph.nsplit) wgt[i * ph.nsplit + lane + 32] = w1 / Lsum;
            }
            consumer_sync();
            #pragma unroll 1
            for (int o = tid; o < GRP * DH; o += NCT) {
                const int i = o / DH, dd = o % DH;
                const float* pa = P.part_acc + (hbase + (size_t)i * ph.nsplit) * DH + dd;
                float ov = 0.0f;
#pragma unroll 6
                for (int sidx = 0; sidx < ph.nsplit; sidx++) ov = fmaf(__ldcg(pa + (size_t)sidx * DH), wgt[i * ph.nsplit + sidx], ov);
                ph.ctx[(size_t)(ap.kv * GRP + i) * DH + dd] = ov;
            }
            if (tid == 0) P.attn_cnt[ap.kv] = 0u;
        }
    }
    return true;
}

// One release-acquire ticket: the caller's CTA has met at a barrier after writing its partial results; the
// returned value tells how many arrived before.  The last arrival may read every other CTA's partials.
__device__ __forceinline__ unsigned ticket_acq_rel(unsigned* cnt) {
    unsigned old;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(cnt) : "memory");
    return old;
}

// ------------------------------------------------------------------------------------------------
// Attention phase when q arrives already normed and rotated and the current position's k and v are
// already in the cache (the qkv phase's epilogue did both).  One CTA per (kv head, split of the cached
// positions).  Per ring tile of positions: scores with one thread per (head, position) -- lanes walk the
// head dimension rotated by their position so that shared-memory accesses do not collide --, soft-max
// statistics by one warp per head, then P*V with one thread per (head, dimension).
// ------------------------------------------------------------------------------------------------
// Tiles of attention_phase2: up to ATT2_TR ring slots of K rows, then as many of V rows.
#define ATT2_TR 4
struct AttPlan2 { int tr, tile_rows, ntiles; };
__device__ __forceinline__ AttPlan2 att_plan2(const AttPlan& ap, int nring) {
    AttPlan2 q;
    q.tr = min(min(ATT2_TR, nring / 2), 159 / ap.rows_per_slot);
    if (q.tr < 1) q.tr = 1;
    q.tile_rows = q.tr * ap.rows_per_slot;
    q.ntiles = (ap.n_old + q.tile_rows - 1) / q.tile_rows;
    return q;
}

template <int GRP, class SM>
__device__ __noinline__ bool attention_phase2(const HxPersist& P, const HxPhase& ph, SM& S, uint8_t* ring, uint8_t* digb,
                                              uint32_t& ctr, int pi, int pos) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, cta = blockIdx.x;
    const AttPlan ap = att_plan(ph, cta, pos);
    const AttPlan2 ap2 = att_plan2(ap, (int)RING_SLOTS);
    const int DH = ph.DH, rps = ap.rows_per_slot;
    float* sq = reinterpret_cast<float*>(digb);                 // [GRP][DH] queries
    float* knew = sq + 8 * 256;                                  // [DH] current k
    float* vnew = knew + 256;                                    // [DH] current v
    float* sp = vnew + 256;                                      // [GRP][160] scores / probabilities
    float* accx = sp + 8 * 160;                                  // [nsub][GRP*DH] partial outputs (small heads only)
    constexpr int spitch = 160;
    const int HD = GRP * DH;
    constexpr int NACC = (GRP * 256 + NCT - 1) / NCT;           // (head, dim) pairs per thread when GRP*DH > NCT
    const int nsub = HD < NCT ? NCT / HD : 1;                    // position subsets when threads outnumber the pairs
    const int sub = HD < NCT ? tid / HD : 0;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; i++) acc[i] = 0.0f;
    if (ap.active && ap.t1 > ap.t0) {
        for (int i = tid; i < HD; i += NCT) sq[i] = __ldcg(ph.qkv + (size_t)ap.kv * HD + i);
        if (ap.has_new) {
            const size_t o = ((size_t)ap.kv * ph.cap + pos) * DH;
            for (int e = tid; e < DH; e += NCT) { knew[e] = __ldcg(ph.kc + o + e); vnew[e] = __ldcg(ph.vc + o + e); }
        }
        if (tid < 8) { S.att_m[tid] = -100000000.0f; S.att_l[tid] = 0.0f; S.att_ax[tid] = 0u; }
        consumer_sync();
        STAMP(4);
        const int ntile = ap2.ntiles + ((ap.has_new && ap.n_old % ap2.tile_rows == 0) ? 1 : 0);
        #pragma unroll 1
        for (int s = 0; s < ntile; s++) {
            const bool ring_tile = s < ap2.ntiles;
            const int nr = ring_tile ? min(ap2.tile_rows, ap.n_old - s * ap2.tile_rows) : 0;
            const int nsl = (nr + rps - 1) / rps;                       // ring slots of this tile (K, then as many of V)
            const bool add_new = ap.has_new && (s == ntile - 1);       // the current position rides on the last tile
            const float* kp[ATT2_TR]; uint32_t ks[ATT2_TR];
#pragma unroll
            for (int j = 0; j < ATT2_TR; j++) {
                kp[j] = knew; ks[j] = 0;
                if (j < nsl) {
                    ks[j] = ctr % RING_SLOTS; const uint32_t round = ctr / RING_SLOTS; ctr++;
                    if (!mbar_wait(&S.full[ks[j]], round & 1, &S.abort_flag)) return false;
                    kp[j] = reinterpret_cast<const float*>(ring + (size_t)ks[j] * HX_RING_SLOT);
                }
            }
            if (s == 0) STAMP(8);
            const int ntot = nr + (add_new ? 1 : 0);
            // scores: thread (head i, position r)
            #pragma unroll 1
            for (int it = tid; it < GRP * ntot; it += NCT) {
                const int i = it / ntot, r = it - i * ntot;
                const int j = (r >= rps) + (r >= 2 * rps) + (r >= 3 * rps);
                const float* kr = (r < nr) ? (j == 0 ? kp[0] : j == 1 ? kp[1] : j == 2 ? kp[2] : kp[3]) + (size_t)(r - j * rps) * DH : knew;
                const float* qi = sq + i * DH;
                float d0 = 0.0f, d1 = 0.0f;
                int e = (4 * r) % DH;
                #pragma unroll 4
                for (int jj = 0; jj < DH; jj += 4) {
                    const float4 k4 = *reinterpret_cast<const float4*>(kr + e);
                    const float4 q4 = *reinterpret_cast<const float4*>(qi + e);
                    d0 = fmaf(q4.x, k4.x, d0); d1 = fmaf(q4.y, k4.y, d1); d0 = fmaf(q4.z, k4.z, d0); d1 = fmaf(q4.w, k4.w, d1);
                    e += 4; if (e >= DH) e = 0;
                }
                sp[i * spitch + r] = (d0 + d1) * ph.scale;
            }
            consumer_sync();
            if (tid < nsl) mbar_arrive(&S.empty[tid == 0 ? ks[0] : tid == 1 ? ks[1] : tid == 2 ? ks[2] : ks[3]]);
            if (s == 0) STAMP(9);
            // online softmax state per head (fused_decode_attn_kernel.hx:74-102)
            if (warp < GRP) {
                const int i = warp;
                float tm = -INFINITY;
                for (int r = lane; r < ntot; r += 32) tm = fmaxf(tm, sp[i * spitch + r]);
                tm = hx_warp_max(tm);
                const float mo = S.att_m[i], mn = fmaxf(mo, tm);
                float ls = 0.0f;
                for (int r = lane; r < ntot; r += 32) { const float pr = __expf(sp[i * spitch + r] - mn); sp[i * spitch + r] = pr; ls += pr; }
                ls = hx_warp_sum(ls);
                if (lane == 0) { const float rr = __expf(mo - mn); S.att_r[i] = rr; S.att_l[i] = S.att_l[i] * rr + ls; S.att_m[i] = mn; }
            }
#pragma unroll
            for (int j = 0; j < ATT2_TR; j++) {
                kp[j] = vnew;
                if (j < nsl) {
                    ks[j] = ctr % RING_SLOTS; const uint32_t round = ctr / RING_SLOTS; ctr++;
                    if (!mbar_wait(&S.full[ks[j]], round & 1, &S.abort_flag)) return false;
                    kp[j] = reinterpret_cast<const float*>(ring + (size_t)ks[j] * HX_RING_SLOT);
                }
            }
            consumer_sync();
            if (s == 0) STAMP(10);
            // P*V: thread (head, dimension) [x position subset]
#pragma unroll
            for (int a = 0; a < NACC; a++) {
                const int hd = (HD < NCT ? tid % HD : tid + a * NCT);
                if (hd < HD && sub < nsub && (HD >= NCT || a == 0)) {
                    const int i = hd / DH, d = hd - i * DH;
                    float v = acc[a] * S.att_r[i];
#pragma unroll
                    for (int j = 0; j < ATT2_TR; j++) {
                        const int r1 = min(nr, (j + 1) * rps);
                        const float* vj = kp[j] + d - (size_t)(j * rps) * DH;
                        #pragma unroll 4
                        for (int r = j * rps + sub; r < r1; r += nsub) v = fmaf(sp[i * spitch + r], vj[(size_t)r * DH], v);
                    }
                    if (add_new && (nr % nsub) == sub) v = fmaf(sp[i * spitch + nr], vnew[d], v);
                    acc[a] = v;
                }
            }
            consumer_sync();
            if (tid < nsl) mbar_arrive(&S.empty[tid == 0 ? ks[0] : tid == 1 ? ks[1] : tid == 2 ? ks[2] : ks[3]]);
        }
        STAMP(5);
        // write this split's partial (position subsets folded through shared memory first)
        if (nsub > 1) {
            if (sub < nsub) accx[sub * HD + tid % HD] = acc[0];
            consumer_sync();
            if (tid < HD) {
                float v = 0.0f;
                for (int u = 0; u < nsub; u++) v += accx[u * HD + tid];
                acc[0] = v;
            }
        }
#pragma unroll
        for (int a = 0; a < NACC; a++) {
            const int hd = (HD < NCT ? tid : tid + a * NCT);
            if (hd < HD && (HD >= NCT || (tid < HD && a == 0))) {
                const int i = hd / DH, d = hd - i * DH;
                const size_t hs = (size_t)(ap.kv * GRP + i) * ph.nsplit + ap.split;
                P.part_acc[hs * DH + d] = acc[a];
                if (d == 0) { P.part_m[hs] = S.att_m[i]; P.part_l[hs] = S.att_l[i]; }
                if (ph.pieces) atomicMax(&S.att_ax[i], __float_as_uint(fabsf(acc[a])));
            }
        }
        if (ph.pieces) {          // bound of this split's contribution to the merged output: max |acc| / l
            consumer_sync();
            if (tid < GRP) {
                const size_t hs = (size_t)(ap.kv * GRP + tid) * ph.nsplit + ap.split;
                const float l = S.att_l[tid];
                P.part_amax[hs] = l > 0.0f ? __uint_as_float(S.att_ax[tid]) / l : 0.0f;
            }
        }
    } else if (ap.active) {
        // empty split: neutral partial
        for (int i = tid; i < GRP; i += NCT) {
            const size_t hs = (size_t)(ap.kv * GRP + i) * ph.nsplit + ap.split;
            P.part_m[hs] = -100000000.0f; P.part_l[hs] = 0.0f;
            if (ph.pieces) P.part_amax[hs] = 0.0f;
        }
        for (int i = tid; i < GRP * DH; i += NCT) {
            const size_t hs = (size_t)(ap.kv * GRP + i / DH) * ph.nsplit + ap.split;
            P.part_acc[hs * DH + i % DH] = 0.0f;
        }
    }
    if (ap.active && !ph.pieces) {
        STAMP(6);
        consumer_sync();
        if (tid == 0) S.ticket = ticket_acq_rel(P.attn_cnt + ap.kv);
        consumer_sync();
        STAMP(7);
        if (S.ticket == (unsigned)ph.nsplit - 1) {
            // merge of the splits: weights w_s = exp(m_s - M) / sum_s l_s exp(m_s - M).  The loads of the partial
            // outputs are issued first so that the weights are computed while they travel.
            float* wgt = sp;                                   // [GRP][nsplit]
            const size_t hbase = (size_t)(ap.kv * GRP) * ph.nsplit;
            constexpr int MCH = 24;
            float pv[MCH];
            const int o0 = tid, i0 = o0 / DH, dd0 = o0 - i0 * DH;
            const float* pa0 = P.part_acc + (hbase + (size_t)i0 * ph.nsplit) * DH + dd0;
            if (o0 < HD) {
#pragma unroll
                for (int u = 0; u < MCH; u++) pv[u] = u < ph.nsplit ? __ldcg(pa0 + (size_t)u * DH) : 0.0f;
            }
            #pragma unroll 1
            for (int i = warp; i < GRP; i += NCW) {
                float mv[2], lv[2];
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int sidx = lane + 32 * j;
                    mv[j] = sidx < ph.nsplit ? __ldcg(P.part_m + hbase + (size_t)i * ph.nsplit + sidx) : -INFINITY;
                    lv[j] = sidx < ph.nsplit ? __ldcg(P.part_l + hbase + (size_t)i * ph.nsplit + sidx) : 0.0f;
                }
                const float M = hx_warp_max(fmaxf(mv[0], mv[1]));
                const float w0 = __expf(mv[0] - M), w1 = __expf(mv[1] - M);
                const float Lsum = hx_warp_sum(lv[0] * w0 + lv[1] * w1);
                if (lane < ph.nsplit) wgt[i * ph.nsplit + lane] = w0 / Lsum;
                if (lane + 32 < ph.nsplit) wgt[i * ph.nsplit + lane + 32] = w1 / Lsum;
            }
            STAMP(11);
            consumer_sync();
            STAMP(12);
            #pragma unroll 1
            for (int o = tid; o < HD; o += NCT) {
                const int i = o / DH, dd = o - i * DH;
                const float* pa = P.part_acc + (hbase + (size_t)i * ph.nsplit) * DH + dd;
                float ov = 0.0f;
                int s0 = 0;
                if (o == o0) {
#pragma unroll
                    for (int u = 0; u < MCH; u++) if (u < ph.nsplit) ov = fmaf(pv[u], wgt[i * ph.nsplit + u], ov);
                    s0 = MCH;
                }
#pragma unroll 4
                for (int sidx = s0; sidx < ph.nsplit; sidx++) ov = fmaf(__ldcg(pa + (size_t)sidx * DH), wgt[i * ph.nsplit + sidx], ov);
                ph.ctx[(size_t)(ap.kv * GRP + i) * DH + dd] = ov;
            }
            STAMP(13);
            if (tid == 0) P.attn_cnt[ap.kv] = 0u;
        }
    }
    return true;
}
