// hx_persist.cu -- one cooperative kernel per decoded token.
//
// Replaces the launch sequence of decode_step_llama (helixc/runtime/gpt2_infer.c:1341-1613) by a single
// persistent grid, one CTA per SM, that walks the phases of the token
//     [qkv | attention | o_proj | gate+up | down] x layers, lm_head + arg-max
// with a grid-wide barrier between phases.  Inside a CTA one producer thread streams this CTA's share
// of the weights (and of the KV cache) from HBM into a ring of shared-memory slots with cp.async.bulk
// (TMA, mbarrier completion) and runs AHEAD of the phase barriers: weights do not depend on
// activations, so HBM keeps streaming while the consumer warps wait for the previous phase.  Eight
// consumer warps read the slots, decode the E2M1 codes in registers (cvt.rn.f16x2.e2m1x2), scale them
// by the E4M3 block scale (exact in f16) and contract them with the activations on the tensor cores
// (mma.sync m16n8k16, f32 accumulate).  The f32 activation vector is split exactly into three f16
// terms x = S*(d1 + d2*2^-11 + d3*2^-22) that occupy three of the eight B columns, so no activation
// precision is lost.  HBM-bound: 0.5625 B per weight + the f32 KV rows.
//
// Every wait (mbarrier, grid barrier) is bounded: when it runs out the kernel records an error code
// and all roles drain without touching the ring again.
#define RING_SLOTS HX_RING_SLOTS
#define NCW 16                      // consumer warps (one k-group of a slot each)
#define NCT (NCW * 32)              // consumer threads
#define PT (NCT + 32)               // + one producer warp
#define WAIT_LIMIT (1u << 24)
#include "hx_persist.cuh"
#include "hx_persist_common.cuh"

// ------------------------------------------------------------------------------------------------
// T16 repack
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_repack_t16(const int32_t* __restrict__ words, const uint8_t* __restrict__ micro,
                                                     int rows, int K, int Kpad, uint8_t* __restrict__ dst, int dstKG,
                                                     int grp, int row_mul, int row_off) {
    const int kwords = Kpad / 7, kblk = Kpad / 16, KG = (K + HX_T16_KG - 1) / HX_T16_KG;
    const size_t items = (size_t)rows * KG * 4;
    for (size_t it = (size_t)blockIdx.x * blockDim.x + threadIdx.x; it < items; it += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(it & 3);
        const int kg = (int)((it >> 2) % KG);
        const int r = (int)((it >> 2) / KG);
        const int dr = (r / grp) * grp * row_mul + row_off * grp + r % grp;
        const int32_t* wr = words + (size_t)r * kwords;
        auto code = [&](int e) -> uint32_t {
            if (e >= K) return 0u;
            const int wd = e / 7, s = e - wd * 7;
            return ((uint32_t)wr[wd] >> (4 * s)) & 15u;
        };
        uint32_t out[4];
#pragma unroll
        for (int m = 0; m < 8; m++) {
            const int p = m >> 1, h = m & 1;
            const int eA = kg * 128 + (2 * p) * 16 + t + 8 * h, eB = eA + 16;
            const uint32_t b0 = code(eA) | (code(eB) << 4), b1 = code(eA + 4) | (code(eB + 4) << 4);
            const uint32_t piece = b0 | (b1 << 8);
            if (m & 1) out[m >> 1] |= piece << 16; else out[m >> 1] = piece;
        }
        uint8_t* cell = dst + ((size_t)(dr / 16) * dstKG + kg) * HX_T16_CELL;
        *reinterpret_cast<uint4*>(cell + (dr % 16) * 64 + t * 16) = make_uint4(out[0], out[1], out[2], out[3]);
        if (t == 0) {
            uint32_t s0 = 0, s1 = 0;
#pragma unroll
            for (int b = 0; b < 8; b++) {
                const int blk = kg * 8 + b;
                const uint32_t v = (blk * 16 < K && blk < kblk) ? micro[(size_t)r * kblk + blk] : 0u;
                if (b < 4) s0 |= v << (8 * b); else s1 |= v << (8 * (b - 4));
            }
            *reinterpret_cast<uint2*>(cell + 1024 + (dr % 16) * 8) = make_uint2(s0, s1);
        }
    }
}

void hx_repack_t16(const int32_t* words, const uint8_t* micro, int rows, int K, int Kpad, uint8_t* dst,
                   int dstKG, int grp, int row_mul, int row_off, cudaStream_t st) {
    const size_t items = (size_t)rows * hx_t16_kgroups(K) * 4;
    int g = (int)((items + 255) / 256); if (g > 148 * 16) g = 148 * 16; if (g < 1) g = 1;
    k_repack_t16<<<g, 256, 0, st>>>(words, micro, rows, K, Kpad, dst, dstKG, grp, row_mul, row_off);
    HX_COUNT_LAUNCH(1);
}

__device__ __forceinline__ void cvt_e2m1x8(uint32_t w, uint32_t& h0, uint32_t& h1, uint32_t& h2, uint32_t& h3) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3) : "r"(w));
}
__device__ __forceinline__ uint32_t cvt_e4m3x2(uint32_t s16) {
    uint32_t h;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"((unsigned short)s16));
    return h;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ------------------------------------------------------------------------------------------------
// Work assignment, shared by the producer and the consumers so both walk the same slot sequence.
// Linear phase: units (1 or 2 m-tiles) are dealt round-robin, unit u = cta + i*grid; a tile is cut
// into nst stages of at most 8 k-groups.  Attention phase: CTA -> (kv head, split); its cached rows
// below the current position are cut into slots of rows_per_slot rows, K slot then V slot.
// ------------------------------------------------------------------------------------------------
struct LinPlan { int nunits, nst, kg_per; };
__device__ __forceinline__ LinPlan lin_plan(const HxPhase& ph, int cta, int grid) {
    LinPlan p;
    const int units = ph.ntiles / ph.unit;
    p.nunits = cta < units ? (units - cta + grid - 1) / grid : 0;
    p.nst = (ph.KG + HX_SLOT_CELLS - 1) / HX_SLOT_CELLS;
    p.kg_per = (ph.KG + p.nst - 1) / p.nst;
    return p;
}
struct Smem {
    uint64_t full[HX_RING_SLOTS];
    uint64_t empty[HX_RING_SLOTS];
    float partial[2][NCW][16];
    float gate[16];
    float red[NCW * 2];
    float att_m[8], att_l[8], att_r[8];
    float bv[NCW]; int bi[NCW];
    unsigned ticket;
    volatile int abort_flag;
};


__global__ void __launch_bounds__(PT, 1) k_decode_persist(const __grid_constant__ HxPersist P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem& S = *reinterpret_cast<Smem*>(smem_raw);
    uint8_t* ring = smem_raw + ((sizeof(Smem) + 127) & ~(size_t)127);
    uint8_t* digb = ring + (size_t)HX_RING_SLOTS * HX_RING_SLOT;       // f16 split of x / attention scratch
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, grid = gridDim.x;
    const int pos = *P.pos;

    if (tid == 0) {
        for (int i = 0; i < HX_RING_SLOTS; i++) { mbar_init(&S.full[i], 1); mbar_init(&S.empty[i], NCW); }
        S.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == NCW) {
        // =========================== producer: one thread streams the slots ===========================
        if (lane != 0) return;
        uint32_t ctr = 0;
        auto push = [&](const void* src, uint32_t bytes) -> bool {
            const uint32_t slot = ctr % HX_RING_SLOTS, round = ctr / HX_RING_SLOTS;
            if (round > 0 && !mbar_wait(&S.empty[slot], (round - 1) & 1, &S.abort_flag)) return false;
            mbar_expect_tx(&S.full[slot], bytes);
            bulk_g2s(ring + (size_t)slot * HX_RING_SLOT, src, bytes, &S.full[slot]);
            ctr++;
            return true;
        };
        #pragma unroll 1
        for (int pi = 0; pi < P.nphases; pi++) {
            const HxPhase& ph = P.phases[pi];
            if (ph.type == HX_PH_LINEAR) {
                const LinPlan lp = lin_plan(ph, cta, grid);
                for (int i = 0; i < lp.nunits; i++)
                    #pragma unroll 1
                    for (int tu = 0; tu < ph.unit; tu++) {
                        const int mt = (cta + i * grid) * ph.unit + tu;
                        const uint8_t* tb = ph.w + (size_t)mt * ph.KG * HX_T16_CELL;
                        #pragma unroll 1
                        for (int s = 0; s < lp.nst; s++) {
                            const int kg0 = s * lp.kg_per, nkg = min(lp.kg_per, ph.KG - kg0);
                            if (!push(tb + (size_t)kg0 * HX_T16_CELL, (uint32_t)nkg * HX_T16_CELL)) return;
                        }
                    }
            } else {
                const AttPlan ap = att_plan(ph, cta, pos);
                const size_t rowb = (size_t)ph.DH * 4;
                #pragma unroll 1
                for (int s = 0; s < ap.nslots; s++) {
                    const int r0 = ap.t0 + s * ap.rows_per_slot, nr = min(ap.rows_per_slot, ap.t0 + ap.n_old - r0);
                    const size_t off = ((size_t)ap.kv * ph.cap + r0) * ph.DH;
                    if (!push(ph.kc + off, (uint32_t)(nr * rowb))) return;
                    if (!push(ph.vc + off, (uint32_t)(nr * rowb))) return;
                }
            }
        }
        return;
    }

    // =============================== consumers ===============================
    uint32_t ctr = 0;                 // same slot sequence as the producer
    unsigned long long bar_target = P.bar_base;
    const int g = lane >> 2, t = lane & 3;
    float best_v = -INFINITY; int best_i = INT_MAX;

    #pragma unroll 1
    for (int pi = 0; pi < P.nphases; pi++) {
        const HxPhase& ph = P.phases[pi];
        STAMP(0);
        if (ph.type == HX_PH_LINEAR) {
            // ---------- prologue: x -> (norm) -> three f16 terms in mma-B order ----------
            // All loads of a thread are issued before any use (one L2 round trip), values stay in registers.
            const int K = ph.K, Kt = ph.KG * HX_T16_KG;
            const float* xin = ph.x;
            if (ph.tok) xin = ph.x + (size_t)(ph.tok[P.tok_by_pos ? pos : 0]) * K;
            __half* dig = reinterpret_cast<__half*>(digb);
            float inv = 1.0f, Sx = 1.0f;
            constexpr int XQ = 6;                                  // float4 per thread per chunk: 512*4*6 = 12288 elements
            #pragma unroll 1
            for (int c0 = 0; c0 < Kt; c0 += NCT * 4 * XQ) {
                const bool single = (Kt <= NCT * 4 * XQ);
                float4 xr[XQ];
                float ss = 0.0f, mx = 0.0f;
                // pass 1 over the whole vector when it does not fit one chunk (large K: two reads)
                if (!single && c0 == 0) {
                    for (int k = tid * 4; k < K; k += NCT * 4) {
                        const float4 v = __ldcg(reinterpret_cast<const float4*>(xin + k));
                        if (ph.norm == HX_NORM_RMS) {
                            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                            const float4 gg = *reinterpret_cast<const float4*>(ph.g + k);
                            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x * gg.x), fabsf(v.y * gg.y)), fmaxf(fabsf(v.z * gg.z), fabsf(v.w * gg.w))));
                        } else mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                    }
                }
#pragma unroll
                for (int i = 0; i < XQ; i++) {
                    const int k = c0 + (tid + i * NCT) * 4;
                    xr[i] = (k < K) ? __ldcg(reinterpret_cast<const float4*>(xin + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                if (ph.tok && ph.x_out) {
#pragma unroll
                    for (int i = 0; i < XQ; i++) {
                        const int k = c0 + (tid + i * NCT) * 4;
                        if (k < K && ((k >> 2) % grid) == cta) *reinterpret_cast<float4*>(ph.x_out + k) = xr[i];   // residual stream
                    }
                }
                if (ph.norm == HX_NORM_RMS) {
#pragma unroll
                    for (int i = 0; i < XQ; i++) {
                        const int k = c0 + (tid + i * NCT) * 4;
                        if (k < K) {
                            const float4 gg = *reinterpret_cast<const float4*>(ph.g + k);
                            if (single) ss += xr[i].x * xr[i].x + xr[i].y * xr[i].y + xr[i].z * xr[i].z + xr[i].w * xr[i].w;
                            xr[i].x *= gg.x; xr[i].y *= gg.y; xr[i].z *= gg.z; xr[i].w *= gg.w;
                        }
                    }
                }
                if (single) {
#pragma unroll
                    for (int i = 0; i < XQ; i++)
                        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(xr[i].x), fabsf(xr[i].y)), fmaxf(fabsf(xr[i].z), fabsf(xr[i].w))));
                }
                if (c0 == 0) {
                    ss = hx_warp_sum(ss); mx = hx_warp_max(mx);
                    if (lane == 0) { S.red[warp] = ss; S.red[NCW + warp] = mx; }
                    consumer_sync();
                    float tss = 0.0f, tmx = 0.0f;
#pragma unroll
                    for (int i = 0; i < NCW; i++) { tss += S.red[i]; tmx = fmaxf(tmx, S.red[NCW + i]); }
                    if (ph.norm == HX_NORM_RMS) inv = rsqrtf(tss / (float)K + ph.eps);
                    // power of two above max|x_normed|: exact scaling, first term magnitude <= 1
                    const float vmax = tmx * inv;
                    if (vmax > 0.0f && vmax < INFINITY) Sx = __uint_as_float(((__float_as_uint(vmax) >> 23) + 1u) << 23);
                }
                const float mul = inv / Sx;                    // Sx is a power of two: exact
#pragma unroll
                for (int i = 0; i < XQ; i++) {
                    const int k = c0 + (tid + i * NCT) * 4;
                    if (k < Kt) {
                        const float vv[4] = {xr[i].x * mul, xr[i].y * mul, xr[i].z * mul, xr[i].w * mul};
                        // k..k+3 share (k-group, block, half): positions differ only in the quad lane tt
                        const int kg = k >> 7, e = k & 127, blk = e >> 4, j = e & 15;
                        const int p = blk >> 1, ab = blk & 1, h = j >> 3, jj = j & 7;
                        const int slot = ((jj >> 2) << 1) | ab, m = (p << 1) | h;
                        const int base = ((kg * 8 + m) * 3) * 16 + slot;
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const float v = vv[q];
                            const __half d1 = __float2half_rn(v);
                            const float r1 = (v - __half2float(d1)) * 2048.0f;
                            const __half d2 = __float2half_rn(r1);
                            const float r2 = (r1 - __half2float(d2)) * 2048.0f;
                            const __half d3 = __float2half_rn(r2);
                            dig[base + q * 4] = d1; dig[base + q * 4 + 16] = d2; dig[base + q * 4 + 32] = d3;
                        }
                    }
                }
            }
            consumer_sync();
            STAMP(1);

            // ---------- tiles ----------
            const LinPlan lp = lin_plan(ph, cta, grid);
            long long wait_cycles = 0;
            const float total_scale = Sx;
            int pbuf = 0;
            #pragma unroll 1
            for (int i = 0; i < lp.nunits; i++) {
                #pragma unroll 1
                for (int tu = 0; tu < ph.unit; tu++) {
                    const int mt = (cta + i * grid) * ph.unit + tu;
                    float c[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};   // two chains: mma latency overlaps
                    #pragma unroll 1
                    for (int s = 0; s < lp.nst; s++) {
                        const int kg0 = s * lp.kg_per, nkg = min(lp.kg_per, ph.KG - kg0);
                        const uint32_t slot = ctr % HX_RING_SLOTS, round = ctr / HX_RING_SLOTS;
                        ctr++;
                        { const long long _w0 = clock64();
                          if (!mbar_wait(&S.full[slot], round & 1, &S.abort_flag)) goto aborted;
                          wait_cycles += clock64() - _w0; }
                        if (warp < nkg) {
                            const uint8_t* cell = ring + (size_t)slot * HX_RING_SLOT + (size_t)warp * HX_T16_CELL;
                            const uint4 qa = *reinterpret_cast<const uint4*>(cell + lane * 16);
                            const uint4 qb = *reinterpret_cast<const uint4*>(cell + 512 + lane * 16);
                            const uint2 sa = *reinterpret_cast<const uint2*>(cell + 1024 + g * 8);
                            const uint2 sb = *reinterpret_cast<const uint2*>(cell + 1024 + (g + 8) * 8);
                            const __half* dk = reinterpret_cast<const __half*>(digb) + (size_t)(kg0 + warp) * 8 * 48;
                            const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w}, wb[4] = {qb.x, qb.y, qb.z, qb.w};
                            const uint32_t sca[4] = {sa.x & 0xFFFFu, sa.x >> 16, sa.y & 0xFFFFu, sa.y >> 16};
                            const uint32_t scb[4] = {sb.x & 0xFFFFu, sb.x >> 16, sb.y & 0xFFFFu, sb.y >> 16};
#pragma unroll
                            for (int p = 0; p < 4; p++) {
                                uint32_t ha0, ha1, ha2, ha3, hb0, hb1, hb2, hb3;
                                cvt_e2m1x8(wa[p], ha0, ha1, ha2, ha3);
                                cvt_e2m1x8(wb[p], hb0, hb1, hb2, hb3);
                                const uint32_t sA = cvt_e4m3x2(sca[p]), sB = cvt_e4m3x2(scb[p]);
                                uint2 b0 = make_uint2(0u, 0u), b1 = make_uint2(0u, 0u);
                                if (g < 3) {
                                    b0 = *reinterpret_cast<const uint2*>(dk + ((2 * p) * 3 + g) * 16 + t * 4);
                                    b1 = *reinterpret_cast<const uint2*>(dk + ((2 * p + 1) * 3 + g) * 16 + t * 4);
                                }
                                mma16816(c, hmul2_u32(ha0, sA), hmul2_u32(hb0, sB), hmul2_u32(ha1, sA), hmul2_u32(hb1, sB), b0.x, b0.y);
                                mma16816(c2, hmul2_u32(ha2, sA), hmul2_u32(hb2, sB), hmul2_u32(ha3, sA), hmul2_u32(hb3, sB), b1.x, b1.y);
                            }
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&S.empty[slot]);
                    }
                    // ---------- fold the three terms, reduce across warps, epilogue ----------
                    {
#pragma unroll
                        for (int q = 0; q < 4; q++) c[q] += c2[q];
                        // columns 0,1 live in lanes t == 0 (c0,c1 / c2,c3), column 2 in lanes t == 1 (c0 / c2)
                        const float n0 = __shfl_down_sync(0xffffffffu, c[0], 1), n2 = __shfl_down_sync(0xffffffffu, c[2], 1);
                        if (t == 0) {
                            const float k1 = 1.0f / 2048.0f, k2 = 1.0f / (2048.0f * 2048.0f);
                            S.partial[pbuf][warp][g] = c[0] + c[1] * k1 + n0 * k2;
                            S.partial[pbuf][warp][g + 8] = c[2] + c[3] * k1 + n2 * k2;
                        }
                    }
                    consumer_sync();
                    if (tid < 16) {
                        float v = 0.0f;
#pragma unroll
                        for (int w = 0; w < NCW; w++) v += S.partial[pbuf][w][tid];
                        v *= total_scale;
                        const int row = mt * 16 + tid;
                        if (ph.epi == HX_EPI_SWIGLU) {
                            if (tu == 0) S.gate[tid] = v * ph.ts[0];
                            else {
                                const int hi = (mt >> 1) * 16 + tid;
                                if (hi < ph.N) ph.y[hi] = pz_silu_mul(S.gate[tid], v * ph.ts[1]);
                            }
                        } else if (row < ph.N) {
                            v *= (row < ph.bound0) ? ph.ts[0] : (row < ph.bound1 ? ph.ts[1] : ph.ts[2]);
                            if (ph.epi == HX_EPI_RESID) v = __ldcg(ph.y + row) + v;
                            ph.y[row] = v;
                            if (ph.epi == HX_EPI_ARGMAX && pz_better(v, row, best_v, best_i)) { best_v = v; best_i = row; }
                        }
                    }
                    pbuf ^= 1;
                }
            }
            if (P.dbg && cta == P.dbg_cta && tid == 0) P.dbg[pi * 16 + 4] = (unsigned long long)wait_cycles;
            if (ph.epi == HX_EPI_ARGMAX) {
                // per-CTA best, then the last CTA to arrive folds all of them (no waiting)
                if (warp == 0) {
#pragma unroll
                    for (int d = 16; d >= 1; d >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, best_v, d);
                        const int oi = __shfl_xor_sync(0xffffffffu, best_i, d);
                        if (pz_better(ov, oi, best_v, best_i)) { best_v = ov; best_i = oi; }
                    }
                    if (lane == 0) {
                        P.am_val[cta] = best_v; P.am_idx[cta] = best_i;
                        __threadfence();
                        S.ticket = atomicAdd(P.am_cnt, 1u);
                    }
                }
                consumer_sync();
                if (S.ticket == (unsigned)grid - 1 && warp == 0) {
                    __threadfence();
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
                    if (lane == 0) {
                        const int nt = (bi == INT_MAX) ? 0 : bi;
                        *P.next_tok = nt;
                        const int np = pos + 1;
                        *P.pos_inc = np;
                        if (P.hist) P.hist[np] = nt;
                        *P.am_cnt = 0u;
                    }
                }
            }
        } else {
            // ------------------------------- attention -------------------------------
            bool ok;
            switch (ph.NH / ph.NKV) {
                case 1: ok = attention_phase<1, NCW>(P, ph, S, ring, digb, ctr, pi, pos); break;
                case 2: ok = attention_phase<2, NCW>(P, ph, S, ring, digb, ctr, pi, pos); break;
                case 3: ok = attention_phase<3, NCW>(P, ph, S, ring, digb, ctr, pi, pos); break;
                case 4: ok = attention_phase<4, NCW>(P, ph, S, ring, digb, ctr, pi, pos); break;
                case 5: ok = attention_phase<5, NCW>(P, ph, S, ring, digb, ctr, pi, pos); break;
                case 6: ok = attention_phase<6, NCW>(P, ph, S, ring, digb, ctr, pi, pos); break;
                case 7: ok = attention_phase<7, NCW>(P, ph, S, ring, digb, ctr, pi, pos); break;
                default: ok = attention_phase<8, NCW>(P, ph, S, ring, digb, ctr, pi, pos); break;
            }
            if (!ok) goto aborted;
        }
        STAMP(2);
        // ---------- grid barrier: every CTA's writes of this phase are visible before the next ----------
        if (pi + 1 < P.nphases) {
            __threadfence();
            consumer_sync();
            bar_target += (unsigned long long)grid;
            if (tid == 0) {
                atomicAdd(P.bar, 1ull);
                bool ok = false;
                for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
                    unsigned long long v;
                    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(P.bar) : "memory");
                    if (v >= bar_target) { ok = true; break; }
                    if ((i & 255) == 255 && S.abort_flag) break;
                }
                if (!ok) S.abort_flag = 1;
            }
            consumer_sync();
            if (S.abort_flag) goto aborted;
        }
        STAMP(3);
    }
    if (P.advance_pos && cta == 0 && tid == 0) *P.pos_inc = pos + 1;
    return;

aborted:
    if (tid == 0) { *P.err = 1; atomicAdd(P.bar, (unsigned long long)grid * 4096ull); }   // release everyone still waiting
}

size_t hx_persist_smem(int dig_bytes) {
    const size_t att = (size_t)(8 * 256 + 256 + 256 + 8 * 160 + 8 * NCT) * 4;   // attention scratch shares the x region
    size_t d = (size_t)dig_bytes > att ? (size_t)dig_bytes : att;
    return ((sizeof(Smem) + 127) & ~(size_t)127) + (size_t)HX_RING_SLOTS * HX_RING_SLOT + d;
}

int hx_persist_launch(const HxPersist& p, int grid, cudaStream_t st) {
    const size_t smem = hx_persist_smem(p.dig_bytes);
    if (smem > 227 * 1024) return hx_fail(HX_ERR_ARG, "persistent decode needs %zu bytes of shared memory", smem);
    static std::atomic<unsigned long long> attr_seen{0};
    if (hx_first_on_device(attr_seen))
        HX_CUDA(cudaFuncSetAttribute(k_decode_persist, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    void* args[] = {(void*)&p};
    HX_CUDA(cudaLaunchCooperativeKernel((void*)k_decode_persist, dim3(grid), dim3(PT), args, smem, st));
    HX_COUNT_LAUNCH(1);
    return HX_OK;
}
