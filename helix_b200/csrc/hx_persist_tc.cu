// hx_persist_tc.cu -- the persistent decode-step kernel with the linear phases on the tensor cores.
//
// Same structure as hx_persist.cu (one cooperative CTA per SM, phases separated by a grid barrier, a
// producer thread streaming weights and KV rows through a shared-memory ring with cp.async.bulk that
// runs ahead of the barriers), but the weights are never touched by a CUDA core: the ring holds
// "T128" cells (128 rows x 64 columns of E2M1 codes + their UE4M3 scales, hx_gemm_tc.cu) and a
// dedicated warp feeds them to tcgen05.mma kind::mxf4nvf4 with the accumulator in TMEM.
//
// The f32 activation vector is made exact for the FP4 tensor path by digit slicing: after the
// (optional) RMSNorm, x = Sg * sum_j (d_j/2) 4^-j with sixteen base-4 digits d_j in {0..3} carrying the
// element's sign; each digit row is an E2M1 column (d_j/2 is one of 0, .5, 1, 1.5) with unit block
// scales, so one M=128 x N=16 x K=64 MMA contracts 128 weight rows with all sixteen digits and the
// epilogue recombines y = Sg*ts * sum_j 4^-j D_j.  32 bits below the vector's largest magnitude are
// kept, the products and the f32 accumulation in TMEM are exact for these operands.
//
// Work units are (128-row tile, K piece) so that every SM streams a similar number of bytes; the
// partial sums of a tile are merged in piece order by the last unit to finish (ticket, no waiting), so
// results do not depend on timing.
#define RING_SLOTS 6
#define NCW 16
#define NCT (NCW * 32)
#define PT (NCT + 64)               // + producer warp (16) + MMA warp (17)
#define WAIT_LIMIT (1u << 24)
#include "hx_persist.cuh"
#include "hx_persist_common.cuh"
#include "hx_gemm_tc.cuh"

#define SLOT_CELLS 2                // cells per ring slot (2 * 9216 = 18432 = HX_RING_SLOT): 8 steps of 64 columns
#define TC_NDIG 16
#define TM_COLS 256
#define TM_D0 0                     // two accumulators of TC_NDIG columns
#define TM_SFB 32                   // constant unit scales for the digit columns
#define TM_SFA 64                   // + slot * 16 + (cell * 2 + step pair) * 4

// ------------------------------------------------------------------------------------------------
// committed layout -> T64 cells
// ------------------------------------------------------------------------------------------------
// "T64" cells: per (64-row tile, group of 256 columns = four K steps) 9216 bytes: 64 rows x 128 bytes of
// codes in the K-major 128-byte-swizzle operand layout (row r at r*128, its 16-byte chunk j at position
// j ^ (r & 7)), then two 512-byte scale chunks, one per pair of K steps: inside a chunk the even step uses
// the slots of rows 0..63 and the odd step those of rows 64..127 (byte (rho%32)*16 + (rho/32)*4 + blk,
// rho = row + 64*(step&1)).  Same density as the committed information: 0.5625 B per weight.
__global__ void __launch_bounds__(256) k_repack_t128(const int32_t* __restrict__ words, const uint8_t* __restrict__ micro,
                                                      int rows, int K, int Kpad, uint8_t* __restrict__ dst, int dst_kgroups,
                                                      int grp, int row_mul, int row_off) {
    const int kwords = Kpad / 7, kblk = Kpad / 16, ksteps = (K + 63) / 64;
    const size_t items = (size_t)rows * ksteps * 2;
    for (size_t it = (size_t)blockIdx.x * blockDim.x + threadIdx.x; it < items; it += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(it & 1);
        const int ks = (int)((it >> 1) % ksteps);
        const int r = (int)((it >> 1) / ksteps);
        const int dr = (r / grp) * grp * row_mul + row_off * grp + r % grp;
        const int32_t* wr = words + (size_t)r * kwords;
        uint32_t out[4] = {0u, 0u, 0u, 0u};
#pragma unroll 4
        for (int j = 0; j < 32; j++) {
            const int e = ks * 64 + c * 32 + j;
            uint32_t code = 0u;
            if (e < K) { const int wd = e / 7, s = e - wd * 7; code = ((uint32_t)wr[wd] >> (4 * s)) & 15u; }
            out[j >> 3] |= code << (4 * (j & 7));
        }
        uint8_t* cell = dst + ((size_t)(dr / 64) * dst_kgroups + (ks >> 2)) * HX_T64_CELL;
        const int rl = dr % 64, chunk = (ks & 3) * 2 + c;
        *reinterpret_cast<uint4*>(cell + rl * 128 + ((chunk ^ (rl & 7)) * 16)) = make_uint4(out[0], out[1], out[2], out[3]);
        if (c == 0) {
            uint32_t sv = 0u;
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const int blk = ks * 4 + b;
                const uint32_t v = (blk * 16 < K && blk < kblk) ? micro[(size_t)r * kblk + blk] : 0u;
                sv |= v << (8 * b);
            }
            const int rho = rl + 64 * (ks & 1);
            *reinterpret_cast<uint32_t*>(cell + 8192 + ((ks >> 1) & 1) * 512 + (rho % 32) * 16 + (rho / 32) * 4) = sv;
        }
    }
}

void hx_repack_t128(const int32_t* words, const uint8_t* micro, int rows, int K, int Kpad, uint8_t* dst,
                    int dst_kgroups, int grp, int row_mul, int row_off, cudaStream_t st) {
    const size_t items = (size_t)rows * ((K + 63) / 64) * 2;
    int g = (int)((items + 255) / 256); if (g > 148 * 16) g = 148 * 16; if (g < 1) g = 1;
    k_repack_t128<<<g, 256, 0, st>>>(words, micro, rows, K, Kpad, dst, dst_kgroups, grp, row_mul, row_off);
    HX_COUNT_LAUNCH(1);
}

// ------------------------------------------------------------------------------------------------
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
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 2, 64;" ::: "memory"); }

// Units of a tensor-core linear phase: 64-row tiles over the whole K, dealt round-robin to the CTAs.
// A unit streams kpairs pair-cells, SLOT_CELLS per ring slot.
struct TcPlan { int nunits, kpairs, nslots; };   // kpairs counts 256-column cells
__device__ __forceinline__ TcPlan tc_plan(const HxPhase& ph, int cta, int grid) {
    TcPlan p;
    p.nunits = cta < ph.ntiles ? (ph.ntiles - cta + grid - 1) / grid : 0;
    p.kpairs = ph.ksteps >> 2;
    p.nslots = (p.kpairs + SLOT_CELLS - 1) / SLOT_CELLS;
    return p;
}

struct SmemTc {
    uint64_t full[RING_SLOTS];
    uint64_t empty[RING_SLOTS];
    uint64_t acc_full[2], acc_empty[2], b_ready;
    float red[NCW * 2];
    float att_m[8], att_l[8], att_r[8];
    float bv[NCW]; int bi[NCW];
    float swi[128];
    unsigned ticket, eticket;
    uint32_t tmem_base;
    volatile int abort_flag;
};

__global__ void __launch_bounds__(PT, 1) k_decode_tc(const __grid_constant__ HxPersist P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    SmemTc& S = *reinterpret_cast<SmemTc*>(smem_raw);
    // swizzled operands need 1024-byte aligned cells (the swizzle is a function of the shared-memory address)
    uint8_t* ring = smem_raw + (((smem_u32(smem_raw) + (uint32_t)sizeof(SmemTc) + 16u + 512u + 1023u) & ~1023u) - smem_u32(smem_raw));
    uint8_t* digb = ring + (size_t)RING_SLOTS * HX_RING_SLOT;            // digit columns / attention scratch (1024-aligned)
    uint8_t* sfb1 = smem_raw + ((sizeof(SmemTc) + 15) & ~(size_t)15);    // 512 bytes of 0x38 (scale 1.0), ahead of the ring
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, grid = gridDim.x;
    const int pos = *P.pos;

    if (tid == 0) {
        for (int i = 0; i < RING_SLOTS; i++) { mbar_init(&S.full[i], 1); mbar_init(&S.empty[i], 1); }
        mbar_init(&S.acc_full[0], 1); mbar_init(&S.acc_full[1], 1);
        mbar_init(&S.acc_empty[0], 2); mbar_init(&S.acc_empty[1], 2);
        mbar_init(&S.b_ready, 1);
        S.abort_flag = 0;
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
            uint32_t ctr = 0;
            auto push = [&](const void* src, uint32_t bytes) -> bool {
                const uint32_t slot = ctr % RING_SLOTS, round = ctr / RING_SLOTS;
                if (round > 0 && !mbar_wait(&S.empty[slot], (round - 1) & 1, &S.abort_flag)) return false;
                mbar_expect_tx(&S.full[slot], bytes);
                bulk_g2s(ring + (size_t)slot * HX_RING_SLOT, src, bytes, &S.full[slot]);
                ctr++;
                return true;
            };
            bool ok = true;
#pragma unroll 1
            for (int pi = 0; pi < P.nphases && ok; pi++) {
                const HxPhase& ph = P.phases[pi];
                if (ph.type == HX_PH_LINEAR_TC) {
                    const TcPlan tp = tc_plan(ph, cta, grid);
#pragma unroll 1
                    for (int i = 0; i < tp.nunits && ok; i++) {
                        const uint8_t* base = ph.w + (size_t)(cta + i * grid) * tp.kpairs * HX_T64_CELL;
#pragma unroll 1
                        for (int q = 0; q < tp.kpairs && ok; q += SLOT_CELLS)
                            ok = push(base + (size_t)q * HX_T64_CELL, (uint32_t)min(SLOT_CELLS, tp.kpairs - q) * HX_T64_CELL);
                    }
                } else if (ph.type == HX_PH_ATTN) {
                    const AttPlan ap = att_plan(ph, cta, pos);
                    const size_t rowb = (size_t)ph.DH * 4;
#pragma unroll 1
                    for (int s = 0; s < ap.nslots && ok; s++) {
                        const int r0 = ap.t0 + s * ap.rows_per_slot, nr = min(ap.rows_per_slot, ap.t0 + ap.n_old - r0);
                        const size_t off = ((size_t)ap.kv * ph.cap + r0) * ph.DH;
                        ok = push(ph.kc + off, (uint32_t)(nr * rowb));
                        if (ok) ok = push(ph.vc + off, (uint32_t)(nr * rowb));
                    }
                }
            }
        }
    } else if (warp == NCW + 1) {
        // =========================== MMA issuer ===========================
        if (lane == 0) {
            tc_cp_sf(tmem + TM_SFB, tc_desc(smem_u32(sfb1), 16, 128));
            const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(TC_NDIG >> 3) << 17) | (8u << 24);
            const uint64_t a_ring = tc_desc(smem_u32(ring), 16, 1024, TC_SW128);    // 8-row groups 1024 B apart, 128-byte swizzle
            const uint64_t sf_ring = tc_desc(smem_u32(ring) + 8192, 16, 128);
            const uint64_t b_base = tc_desc(smem_u32(digb), 16, 1024, TC_SW128);
            uint32_t ctr = 0, uc = 0, tcph = 0;
            bool ok = true;
#pragma unroll 1
            for (int pi = 0; pi < P.nphases && ok; pi++) {
                const HxPhase& ph = P.phases[pi];
                if (ph.type == HX_PH_LINEAR_TC) {
                    ok = mbar_wait(&S.b_ready, tcph & 1, &S.abort_flag);        // digit columns of this phase are in place
                    tcph++;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const TcPlan tp = tc_plan(ph, cta, grid);
#pragma unroll 1
                    for (int i = 0; i < tp.nunits && ok; i++) {
                        const uint32_t buf = uc & 1u;
                        if (uc >= 2) ok = mbar_wait(&S.acc_empty[buf], ((uc >> 1) - 1) & 1, &S.abort_flag);
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t dcol = tmem + TM_D0 + buf * TC_NDIG;
                        uint64_t b_run = b_base;                       // digit columns, step 0
#pragma unroll 1
                        for (int q0 = 0; q0 < tp.kpairs && ok; q0 += SLOT_CELLS) {
                            const uint32_t slot = ctr % RING_SLOTS, round = ctr / RING_SLOTS;
                            ctr++;
                            ok = mbar_wait(&S.full[slot], round & 1, &S.abort_flag);
                            if (!ok) break;
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                            // descriptors advance by constants (16-byte units): a cell is 9216 B = 576 units, a K step inside
                            // it 32 B = 2 units, its scale chunks at +8192 B and +8704 B; the digit columns are 2048 B per cell
                            const uint64_t a_slot = a_ring + (uint64_t)(slot * (HX_RING_SLOT >> 4));
                            const uint64_t sf_slot = sf_ring + (uint64_t)(slot * (HX_RING_SLOT >> 4));
                            const uint32_t tsf_slot = tmem + TM_SFA + slot * 16;
                            const int np = min(SLOT_CELLS, tp.kpairs - q0);
#pragma unroll
                            for (int c = 0; c < SLOT_CELLS; c++) {
                                if (c < np) {
                                    tc_cp_sf(tsf_slot + c * 8, sf_slot + (uint64_t)(c * 576));
                                    tc_cp_sf(tsf_slot + c * 8 + 4, sf_slot + (uint64_t)(c * 576 + 32));
                                }
                            }
#pragma unroll
                            for (int c = 0; c < SLOT_CELLS; c++) {
                                if (c < np) {
#pragma unroll
                                    for (int e = 0; e < 4; e++)
                                        tc_mma(dcol, a_slot + (uint64_t)(c * 576 + e * 2), b_run + (uint64_t)(e * 2), idesc,
                                               tsf_slot + c * 8 + (e >> 1) * 4 + (e & 1) * 2, tmem + TM_SFB, (q0 + c + e) > 0 ? 1u : 0u);
                                    b_run += 128;
                                }
                            }
                            tc_commit(&S.empty[slot]);
                        }
                        tc_commit(&S.acc_full[buf]);
                        uc++;
                    }
                } else if (ph.type == HX_PH_ATTN) {
                    const AttPlan ap = att_plan(ph, cta, pos);
                    ctr += 2u * (uint32_t)ap.nslots;             // ring slots the consumers use for K and V rows
                }
            }
        }
    } else {
        // =============================== consumers ===============================
        uint32_t ctr = 0, uc = 0;
        unsigned long long bar_target = P.bar_base;
        float best_v = -INFINITY; int best_i = INT_MAX;

#pragma unroll 1
        for (int pi = 0; pi < P.nphases; pi++) {
            const HxPhase& ph = P.phases[pi];
            STAMP(0);
            if (ph.type == HX_PH_LINEAR_TC) {
                // ---------- prologue: x -> (norm) -> sixteen base-4 digit columns in operand layout ----------
                // A thread owns items of 8 consecutive elements; up to XI items stay in registers between the
                // statistics pass and the digit pass (one L2 round trip); longer vectors are read twice.
                const int K = ph.K, Kt = ph.ksteps * 64;
                const float* xin = ph.x;
                if (ph.tok) xin = ph.x + (size_t)(ph.tok[P.tok_by_pos ? pos : 0]) * K;
                constexpr int XI = 3;
                const bool inreg = Kt <= NCT * 8 * XI;
                float xv[XI][8];
                float inv = 1.0f, Sg = 1.0f;
                {
                    float ss = 0.0f, mx = 0.0f;
                    if (inreg) {
#pragma unroll
                        for (int i = 0; i < XI; i++) {
                            const int k = (tid + i * NCT) * 8;
                            float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
                            if (k < K) { a = __ldcg(reinterpret_cast<const float4*>(xin + k)); b = __ldcg(reinterpret_cast<const float4*>(xin + k + 4)); }
                            xv[i][0] = a.x; xv[i][1] = a.y; xv[i][2] = a.z; xv[i][3] = a.w; xv[i][4] = b.x; xv[i][5] = b.y; xv[i][6] = b.z; xv[i][7] = b.w;
                        }
#pragma unroll
                        for (int i = 0; i < XI; i++) {
                            const int k = (tid + i * NCT) * 8;
                            if (k < K) {
                                if (ph.tok && ph.x_out && ((k >> 3) % grid) == cta) {
                                    *reinterpret_cast<float4*>(ph.x_out + k) = make_float4(xv[i][0], xv[i][1], xv[i][2], xv[i][3]);
                                    *reinterpret_cast<float4*>(ph.x_out + k + 4) = make_float4(xv[i][4], xv[i][5], xv[i][6], xv[i][7]);
                                }
                                if (ph.norm == HX_NORM_RMS) {
                                    const float4 ga = *reinterpret_cast<const float4*>(ph.g + k), gb = *reinterpret_cast<const float4*>(ph.g + k + 4);
                                    const float gg[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
                                    for (int e = 0; e < 8; e++) { ss = fmaf(xv[i][e], xv[i][e], ss); xv[i][e] *= gg[e]; }
                                }
#pragma unroll
                                for (int e = 0; e < 8; e++) mx = fmaxf(mx, fabsf(xv[i][e]));
                            }
                        }
                    } else {
#pragma unroll 1
                        for (int k = tid * 4; k < K; k += NCT * 4) {
                            const float4 v = __ldcg(reinterpret_cast<const float4*>(xin + k));
                            if (ph.tok && ph.x_out && ((k >> 2) % grid) == cta) *reinterpret_cast<float4*>(ph.x_out + k) = v;
                            if (ph.norm == HX_NORM_RMS) {
                                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                                const float4 gg = *reinterpret_cast<const float4*>(ph.g + k);
                                mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x * gg.x), fabsf(v.y * gg.y)), fmaxf(fabsf(v.z * gg.z), fabsf(v.w * gg.w))));
                            } else mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                        }
                    }
                    ss = hx_warp_sum(ss); mx = hx_warp_max(mx);
                    if (lane == 0) { S.red[warp] = ss; S.red[NCW + warp] = mx; }
                    consumer_sync();
                    float tss = 0.0f, tmx = 0.0f;
#pragma unroll
                    for (int i = 0; i < NCW; i++) { tss += S.red[i]; tmx = fmaxf(tmx, S.red[NCW + i]); }
                    if (ph.norm == HX_NORM_RMS) inv = rsqrtf(tss / (float)K + ph.eps);
                    const float vmax = tmx * inv * 1.0000005f;            // margin for the rounding of x*g*inv
                    if (vmax > 0.0f && vmax < INFINITY) Sg = __uint_as_float(__float_as_uint(vmax) & 0x7F800000u);   // vmax/Sg in [1,2)
                }
                const float mul = (inv / Sg) * 2147483648.0f;             // |x_n| / Sg * 2^31 < 2^32
                auto emit = [&](int k, const float (&v)[8]) {
                    uint32_t M[8]; uint32_t sg = 0u;
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        M[e] = __float2uint_rn(fabsf(v[e]) * mul);
                        sg |= (v[e] < 0.0f ? 8u : 0u) << (4 * e);
                    }
                    const int kg = k >> 8, j = (k >> 5) & 7, w = (k >> 3) & 3;     // 256-column cell, 16-byte chunk, word
                    uint8_t* dst = digb + (size_t)kg * 2048 + w * 4;
#pragma unroll
                    for (int n = 0; n < TC_NDIG; n++) {
                        uint32_t word = 0u;
#pragma unroll
                        for (int e = 0; e < 8; e++) {
                            const int sh = 30 - 2 * n - 4 * e;           // digit n of element e lands on nibble e
                            word |= (sh >= 0 ? (M[e] >> sh) : (M[e] << (-sh))) & (3u << (4 * e));
                        }
                        const uint32_t nz = (word | (word >> 1)) & 0x11111111u;   // a zero digit carries no sign
                        word |= sg & (nz << 3);
                        *reinterpret_cast<uint32_t*>(dst + n * 128 + ((j ^ (n & 7)) << 4)) = word;
                    }
                };
                if (inreg) {
#pragma unroll
                    for (int i = 0; i < XI; i++) {
                        const int k = (tid + i * NCT) * 8;
                        if (k < Kt) emit(k, xv[i]);                        // elements at or beyond K are zero
                    }
                } else {
#pragma unroll 1
                    for (int k = tid * 8; k < Kt; k += NCT * 8) {
                        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                        if (k < K) {
                            float4 a = __ldcg(reinterpret_cast<const float4*>(xin + k)), b = __ldcg(reinterpret_cast<const float4*>(xin + k + 4));
                            if (ph.norm == HX_NORM_RMS) {
                                const float4 ga = *reinterpret_cast<const float4*>(ph.g + k), gb = *reinterpret_cast<const float4*>(ph.g + k + 4);
                                a.x *= ga.x; a.y *= ga.y; a.z *= ga.z; a.w *= ga.w; b.x *= gb.x; b.y *= gb.y; b.z *= gb.z; b.w *= gb.w;
                            }
                            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
                        }
                        emit(k, v);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                consumer_sync();
                if (tid == 0) mbar_arrive(&S.b_ready);
                STAMP(1);

                // ---------- units: accumulator -> digits recombined -> epilogue ----------
                const TcPlan tp = tc_plan(ph, cta, grid);
                ctr += (uint32_t)(tp.nunits * tp.nslots);
                if (warp < 2) {
                    const float out_scale = Sg;       // x_n = Sg * sum_j 4^-j * (digit_j / 2), and digit/2 is the E2M1 value
#pragma unroll 1
                    for (int i = 0; i < tp.nunits; i++) {
                        const int tile = cta + i * grid;
                        const uint32_t buf = uc & 1u;
                        if (!mbar_wait(&S.acc_full[buf], (uc >> 1) & 1, &S.abort_flag)) goto aborted;
                        uc++;
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
                        const int rl = warp * 32 + lane;
                        if (ph.epi == HX_EPI_SWIGLU) {
                            // rows 0..31 of a tile are gate rows, 32..63 the matching up rows
                            S.swi[rl] = v * (rl < 32 ? ph.ts[0] : ph.ts[1]);
                            epi_sync();
                            const int hi = tile * 32 + rl;
                            if (rl < 32 && hi < ph.N) ph.y[hi] = pz_silu_mul(S.swi[rl], S.swi[rl + 32]);
                            epi_sync();
                        } else {
                            const int row = tile * 64 + rl;
                            if (row < ph.N) {
                                v *= (row < ph.bound0) ? ph.ts[0] : (row < ph.bound1 ? ph.ts[1] : ph.ts[2]);
                                if (ph.epi == HX_EPI_RESID) v = __ldcg(ph.y + row) + v;
                                ph.y[row] = v;
                                if (ph.epi == HX_EPI_ARGMAX && pz_better(v, row, best_v, best_i)) { best_v = v; best_i = row; }
                            }
                        }
                    }
                } else uc += (uint32_t)tp.nunits;
                if (ph.epi == HX_EPI_ARGMAX) {
                    // per-CTA best (held by warps 0-1), then the last CTA to arrive folds all of them
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
                        for (int i = 1; i < 2; i++) if (pz_better(S.bv[i], S.bi[i], bv, bi)) { bv = S.bv[i]; bi = S.bi[i]; }
                        P.am_val[cta] = bv; P.am_idx[cta] = bi;
                        __threadfence();
                        S.ticket = atomicAdd(P.am_cnt, 1u);
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
                            *P.pos_inc = pos + 1;
                            if (P.hist) P.hist[pos + 1] = nt;
                            *P.am_cnt = 0u;
                        }
                    }
                }
            } else if (ph.type == HX_PH_ATTN) {
                bool ok;
                switch (ph.NH / ph.NKV) {
                    case 1: ok = attention_phase<1, 1>(P, ph, S, ring, digb, ctr, pi, pos); break;
                    case 2: ok = attention_phase<2, 1>(P, ph, S, ring, digb, ctr, pi, pos); break;
                    case 3: ok = attention_phase<3, 1>(P, ph, S, ring, digb, ctr, pi, pos); break;
                    case 4: ok = attention_phase<4, 1>(P, ph, S, ring, digb, ctr, pi, pos); break;
                    case 5: ok = attention_phase<5, 1>(P, ph, S, ring, digb, ctr, pi, pos); break;
                    case 6: ok = attention_phase<6, 1>(P, ph, S, ring, digb, ctr, pi, pos); break;
                    case 7: ok = attention_phase<7, 1>(P, ph, S, ring, digb, ctr, pi, pos); break;
                    default: ok = attention_phase<8, 1>(P, ph, S, ring, digb, ctr, pi, pos); break;
                }
                if (!ok) goto aborted;
            }
            STAMP(2);
            // ---------- grid barrier ----------
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
        goto done;
aborted:
        if (tid == 0) { S.abort_flag = 1; *P.err = 1; atomicAdd(P.bar, (unsigned long long)grid * 4096ull); }
done:   ;
    }
    // every role meets here; the MMA warp then releases the tensor memory
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == NCW + 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "n"(TM_COLS) : "memory");
}

}  // namespace

size_t hx_persist_tc_smem(int bdig_bytes) {
    const size_t att = (size_t)(8 * 256 + 256 + 256 + 8 * 160 + 8 * NCT) * 4;
    const size_t d = (size_t)bdig_bytes > att ? (size_t)bdig_bytes : att;
    return ((sizeof(SmemTc) + 15) & ~(size_t)15) + 512 + 1024 + (size_t)RING_SLOTS * HX_RING_SLOT + d;
}

int hx_persist_tc_launch(const HxPersist& p, int grid, cudaStream_t st) {
    const size_t smem = hx_persist_tc_smem(p.bdig_bytes);
    if (smem > 227 * 1024) return hx_fail(HX_ERR_ARG, "tensor-core decode needs %zu bytes of shared memory", smem);
    static bool attr = false;
    if (!attr) {
        HX_CUDA(cudaFuncSetAttribute(k_decode_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr = true;
    }
    void* args[] = {(void*)&p};
    HX_CUDA(cudaLaunchCooperativeKernel((void*)k_decode_tc, dim3(grid), dim3(PT), args, smem, st));
    HX_COUNT_LAUNCH(1);
    return HX_OK;
}
