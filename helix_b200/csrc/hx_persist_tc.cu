// hx_persist_tc.cu -- the persistent decode-step kernel with the linear phases on the tensor cores.
//
// Same structure as hx_persist.cu (one cooperative CTA per SM, phases separated by a grid barrier, a
// producer thread streaming weights and KV rows through a shared-memory ring with cp.async.bulk that
// runs ahead of the barriers), but the weights are never touched by a CUDA core: the ring holds
// "T128" cells (128 rows x 256 columns of E2M1 codes + their UE4M3 scales, hx_gemm_tc.cuh) and a
// dedicated thread feeds them to tcgen05.mma kind::mxf4nvf4 with the accumulator in TMEM.
//
// The f32 activation vector is made exact for the FP4 tensor path by digit slicing: after the
// (optional) RMSNorm, x = Sg * sum_j (d_j/2) 4^-j with sixteen base-4 digits d_j in {0..3} carrying the
// element's sign; each digit row is an E2M1 column (d_j/2 is one of 0, .5, 1, 1.5) with unit block
// scales, so one M=128 x N=16 x K=64 MMA contracts 128 weight rows with all sixteen digits and the
// epilogue recombines y = Sg*ts * sum_j 4^-j D_j.  32 bits below the vector's largest magnitude are
// kept, the products and the f32 accumulation in TMEM are exact for these operands.
//
// Work split of a linear phase: the cells of the weight, in storage order (tile-major, K-minor), are cut
// into gridDim equal contiguous runs, so every SM streams the same number of bytes as one linear read.
// A run covers the tail of one tile, whole tiles, and the head of another; each piece of a tile yields a
// partial sum of 128 rows, and the last piece of a tile to finish (ticket, nobody waits) adds the pieces
// in K order and applies the epilogue, so results do not depend on timing.
#define HX_TC_MAX_RING 10
#define RING_SLOTS ((uint32_t)P.tc_ring)
#define NCW 16
#define NCT (NCW * 32)
#define PT (NCT + 64)               // + producer warp (16) + MMA warp (17)
#define WAIT_LIMIT (1u << 24)
#include "hx_persist.cuh"
#include "hx_persist_common.cuh"
#include "hx_gemm_tc.cuh"

#define TC_NDIG 16
#define TM_COLS 256
#define TM_D0 0                     // two accumulators of TC_NDIG columns
#define TM_SFB 32                   // constant unit scales for the digit columns
#define TM_SFA 64                   // + slot * 16 + K step * 4
#define EPI_WARPS 4                 // warps 0..3 own TMEM lanes 0..127 = the rows of a tile

// ------------------------------------------------------------------------------------------------
// committed layout -> T128 cells
// ------------------------------------------------------------------------------------------------
// One cell per (128-row tile, group of 256 columns = four K steps of the MMA), HX_T128_CELL = 18432 bytes:
// 128 rows x 128 bytes of codes in the K-major 128-byte-swizzle operand layout (row r at r*128, its
// 16-byte chunk j at position j ^ (r & 7)), then four 512-byte scale chunks, one per K step, in the
// 32x128b layout tcgen05.cp expects (byte (r%32)*16 + (r/32)*4 + blk).  0.5625 B per weight, the density
// of the committed data.  Cells of a tile are contiguous in K, tiles follow one another.
__global__ void __launch_bounds__(256) k_repack_t128(const int32_t* __restrict__ words, const uint8_t* __restrict__ micro,
                                                      int rows, int K, int Kpad, uint8_t* __restrict__ dst, int kcells,
                                                      int grp, int row_mul, int row_off, int k0) {
    // K = columns taken from the source rows starting at column k0 (a multiple of 16): a K shard of the tensor
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
            if (e < K) { const int es = e + k0, wd = es / 7, s = es - wd * 7; code = ((uint32_t)wr[wd] >> (4 * s)) & 15u; }
            out[j >> 3] |= code << (4 * (j & 7));
        }
        uint8_t* cell = dst + ((size_t)(dr / 128) * kcells + (ks >> 2)) * HX_T128_CELL;
        const int rl = dr % 128, chunk = (ks & 3) * 2 + c;
        *reinterpret_cast<uint4*>(cell + rl * 128 + ((chunk ^ (rl & 7)) * 16)) = make_uint4(out[0], out[1], out[2], out[3]);
        if (c == 0) {
            uint32_t sv = 0u;
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const int blk = ks * 4 + b;
                const uint32_t v = (blk * 16 < K && blk + k0 / 16 < kblk) ? micro[(size_t)r * kblk + blk + k0 / 16] : 0u;
                sv |= v << (8 * b);
            }
            *reinterpret_cast<uint32_t*>(cell + 16384 + (ks & 3) * 512 + (rl % 32) * 16 + (rl / 32) * 4) = sv;
        }
    }
}

void hx_repack_t128(const int32_t* words, const uint8_t* micro, int rows, int K, int Kpad, uint8_t* dst,
                    int kcells, int grp, int row_mul, int row_off, cudaStream_t st, int k0) {
    const size_t items = (size_t)rows * ((K + 63) / 64) * 2;
    int g = (int)((items + 255) / 256); if (g > 148 * 16) g = 148 * 16; if (g < 1) g = 1;
    k_repack_t128<<<g, 256, 0, st>>>(words, micro, rows, K, Kpad, dst, kcells, grp, row_mul, row_off, k0);
    HX_COUNT_LAUNCH(1);
}

// How a phase of ntiles x C cells is cut over `grid` CTAs.
//  * few tiles (2 * ntiles <= grid): every tile is cut into P = min(grid / ntiles, C) pieces of nearly equal
//    length and CTA tile * P + q takes piece q, so each CTA produces exactly one partial sum;
//  * many tiles: the cells in storage order are cut into `grid` equal contiguous runs (a run may cover the
//    tail of one tile, whole tiles and the head of another).
// Returns the most pieces of one tile and the most K cells one CTA touches.
void hx_tc_split(int ntiles, int C, int grid, int* max_pieces, int* max_run) {
    const long long total = (long long)ntiles * C;
    if (2 * ntiles <= grid) {
        int P = grid / ntiles; if (P > C) P = C;
        *max_pieces = P; *max_run = (C + P - 1) / P;
        return;
    }
    if (total < grid) grid = (int)total;          // fewer cells than CTAs: the first `total` CTAs take one cell each
    int mp = 1, mr = 1;
    for (int c = 0; c < grid; c++) {
        const long long b0 = c * total / grid, b1 = (c + 1) * total / grid;
        if (b1 - b0 > mr) mr = (int)(b1 - b0);
    }
    for (int t = 0; t < ntiles; t++) {
        const long long x0 = (long long)t * C, x1 = x0 + C - 1;
        const int c0 = (int)(((x0 + 1) * grid + total - 1) / total) - 1, c1 = (int)(((x1 + 1) * grid + total - 1) / total) - 1;
        if (c1 - c0 + 1 > mp) mp = c1 - c0 + 1;
    }
    *max_pieces = mp; *max_run = mr < C ? mr : C;
}

// The same split, per CTA, for the dataflow engine (hx_decode_df.cu), which reads it from a table.
void hx_df_plan(int ntiles, int C, int grid, HxCtaPlan* out, int* max_pieces, int* max_run) {
    const long long total = (long long)ntiles * C;
    int P = 0, geff = grid;
    if (2 * ntiles <= grid) { P = grid / ntiles; if (P > C) P = C; }
    else if (total < grid) geff = (int)total;
    auto bounds = [&](int cta, long long& b0, long long& b1) {
        b0 = b1 = 0;
        if (P) { if (cta < ntiles * P) { const int tile = cta / P, q = cta - tile * P; b0 = (long long)tile * C + (q * C) / P; b1 = (long long)tile * C + ((q + 1) * C) / P; } }
        else if (cta < geff) { b0 = (long long)cta * total / geff; b1 = (long long)(cta + 1) * total / geff; }
    };
    int mp = 1, mr = 1;
    for (int cta = 0; cta < grid; cta++) {
        HxCtaPlan p = {};
        long long b0, b1; bounds(cta, b0, b1);
        p.b0 = (int)b0; p.b1 = (int)b1; p.C = C;
        p.k0 = (int)(b0 % C);
        const long long n = b1 - b0;
        p.run = n < C ? (int)n : C;
        p.t_first = (int)(b0 / C); p.t_last = n > 0 ? (int)((b1 - 1) / C) : p.t_first - 1;
        p.first_merger = (b0 % C) == 0 ? 1 : 0;
        if (n > 0 && !p.first_merger) {            // piece index = CTAs between the tile's first cell and this one
            int c = cta - 1; long long a0, a1;
            for (;; c--) { bounds(c, a0, a1); if (a0 <= (long long)p.t_first * C) break; }
            p.first_piece = cta - c - 1;
        }
        if (n > 0) {                               // pieces of the last tile in the CTAs that follow
            const long long tile_end = (long long)(p.t_last + 1) * C;
            int others = 0; long long a0, a1 = b1;
            for (int c = cta + 1; a1 < tile_end && c < grid; c++) { bounds(c, a0, a1); if (a1 > a0) others++; }
            p.last_others = others;
            if (others + 1 > mp) mp = others + 1;
            if (!p.first_merger && p.first_piece + 1 > mp) mp = p.first_piece + 1;
        }
        if (p.run > mr) mr = p.run;
        out[cta] = p;
    }
    if (max_pieces) *max_pieces = mp;
    if (max_run) *max_run = mr;
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
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 2, %0;" :: "n"(EPI_WARPS * 32) : "memory"); }

// This CTA's run of cells [b0, b1) of the phase; k0 = K cell of the first one; run = distinct K cells it touches.
// P > 0: every tile is cut into P pieces, CTA tile * P + q takes piece q.  P = 0: equal contiguous runs over geff
// CTAs (with fewer cells than CTAs the first `total` CTAs take one cell each).
struct TcPlan { long long b0, b1, total; int C, k0, run, geff, P; };
__device__ __forceinline__ TcPlan tc_plan(const HxPhase& ph, int cta, int grid) {
    TcPlan p;
    p.C = ph.ksteps >> 2;
    p.total = (long long)ph.ntiles * p.C;
    p.P = 0; p.geff = grid;
    if (2 * ph.ntiles <= grid) {
        p.P = min(grid / ph.ntiles, p.C);
        if (cta < ph.ntiles * p.P) {
            const int tile = cta / p.P, q = cta - tile * p.P;
            p.b0 = (long long)tile * p.C + (q * p.C) / p.P; p.b1 = (long long)tile * p.C + ((q + 1) * p.C) / p.P;
        } else { p.b0 = p.b1 = 0; }
    } else {
        p.geff = p.total < grid ? (int)p.total : grid;
        if (cta >= p.geff) { p.b0 = p.b1 = 0; }
        else if (p.total * (p.geff + 1) < 0x7FFFFFFFLL) {       // 32-bit divisions (the usual case) are several times cheaper
            const unsigned t32 = (unsigned)p.total, g32 = (unsigned)p.geff;
            p.b0 = (unsigned)cta * t32 / g32; p.b1 = (unsigned)(cta + 1) * t32 / g32;
        } else { p.b0 = (long long)cta * p.total / p.geff; p.b1 = (long long)(cta + 1) * p.total / p.geff; }
    }
    p.k0 = p.b0 < 0x7FFFFFFFLL ? (int)((unsigned)p.b0 % (unsigned)p.C) : (int)(p.b0 % p.C);
    const long long n = p.b1 - p.b0;
    p.run = n < p.C ? (int)n : p.C;
    return p;
}
// CTA whose run holds cell x (contiguous runs)
__device__ __forceinline__ int tc_owner(long long x, long long total, int grid) {
    if ((x + 2) * grid + total < 0x7FFFFFFFLL) return (int)((((unsigned)x + 1u) * (unsigned)grid + (unsigned)total - 1u) / (unsigned)total) - 1;
    return (int)(((x + 1) * grid + total - 1) / total) - 1;
}

// ---- tensor-parallel exchange buffer (floats / 32-bit words) ----
__device__ __forceinline__ size_t tp_off_part(const HxPersist& P, int slot, int w) { return ((size_t)slot * P.tp_world + w) * P.tp_dm; }
__device__ __forceinline__ size_t tp_off_am(const HxPersist& P) { return (size_t)2 * P.tp_world * P.tp_dm; }
__device__ __forceinline__ size_t tp_off_flags(const HxPersist& P) { return tp_off_am(P) + 2 * P.tp_world; }
__device__ __forceinline__ size_t tp_off_amflags(const HxPersist& P) { return tp_off_flags(P) + P.tp_world; }
__device__ __forceinline__ size_t tp_off_go(const HxPersist& P) { return tp_off_amflags(P) + P.tp_world; }
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) { asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) { unsigned v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
// Every rank writes `ep` into slot `rank` of each peer's flag array, then waits (bounded) until all peers have written
// theirs here.  Epochs only grow, so a late reader still sees a value >= ep.  One thread per GPU calls this.
__device__ __forceinline__ void tp_signal(const HxPersist& P, size_t flags_off, unsigned ep) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    for (int w = 0; w < P.tp_world; w++)
        if (w != P.tp_rank) st_release_sys(reinterpret_cast<unsigned*>(P.tp_peer[w] + flags_off) + P.tp_rank, ep);
}
__device__ __forceinline__ bool tp_wait(const HxPersist& P, size_t flags_off, unsigned ep, volatile int* abort_flag) {
    const unsigned* mine = reinterpret_cast<const unsigned*>(P.tp_peer[P.tp_rank] + flags_off);
    for (int w = 0; w < P.tp_world; w++) {
        if (w == P.tp_rank) continue;
        bool ok = false;
        for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
            if ((int)(ld_acquire_sys(mine + w) - ep) >= 0) { ok = true; break; }
            if ((i & 255) == 255 && *abort_flag) break;
        }
        if (!ok) return false;
    }
    return true;
}
__device__ __forceinline__ bool tp_handshake(const HxPersist& P, size_t flags_off, unsigned ep, volatile int* abort_flag) {
    tp_signal(P, flags_off, ep);
    return tp_wait(P, flags_off, ep, abort_flag);
}

struct SmemTc {
    uint64_t full[HX_TC_MAX_RING];
    uint64_t empty[HX_TC_MAX_RING];
    uint64_t acc_full[2], acc_empty[2], b_ready;
    float red[NCW * 2];
    float att_m[8], att_l[8], att_r[8]; unsigned att_ax[8];
    float wgt[2304];                // merge weights of the attention splits, [head][split] (o_proj prologue)
    float bv[NCW]; int bi[NCW];
    float swi[128];
    HxPhase ph[2];                  // descriptor of the running phase (pi & 1), the next one is fetched during the grid barrier
    unsigned ticket, eticket;
    uint32_t tmem_base;
    volatile int abort_flag;
};

// TP: compiled with the tensor-parallel exchange (partial sums, cross-GPU barrier, arg-max exchange); the single-GPU
// instantiation carries none of it.
template <bool TP>
__global__ void __launch_bounds__(PT, 1) k_decode_tc(const __grid_constant__ HxPersist P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    SmemTc& S = *reinterpret_cast<SmemTc*>(smem_raw);
    // swizzled operands need 1024-byte aligned cells (the swizzle is a function of the shared-memory address)
    uint8_t* sfb1 = smem_raw + ((sizeof(SmemTc) + 15) & ~(size_t)15);    // 512 bytes of 0x38 (scale 1.0)
    uint8_t* ring = smem_raw + (((smem_u32(smem_raw) + (uint32_t)sizeof(SmemTc) + 16u + 512u + 1023u) & ~1023u) - smem_u32(smem_raw));
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
            uint32_t slot = 0, par = 0;          // parity the empty barrier of `slot` completes when its previous use is over
            bool first_round = true;
            auto push = [&](const void* src, uint32_t bytes) -> bool {
                if (!first_round && !mbar_wait(&S.empty[slot], par, &S.abort_flag)) return false;
                mbar_expect_tx(&S.full[slot], bytes);
                bulk_g2s(ring + (size_t)slot * HX_RING_SLOT, src, bytes, &S.full[slot]);
                if (++slot == nring) { slot = 0; if (first_round) first_round = false; else par ^= 1u; }
                return true;
            };
            bool ok = true;
            // the descriptor of the next phase is loaded one phase early so that streaming never waits for it
            HxPhase nxt = P.phases[0];
#pragma unroll 1
            for (int pi = 0; pi < P.nphases && ok; pi++) {
                const HxPhase ph = nxt;
                if (pi + 1 < P.nphases) {
                    nxt = P.phases[pi + 1];
                    // one CTA per phase pulls the small vectors of the next phase into L2 (they were evicted by a
                    // token's worth of weights since their last use)
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
                    const TcPlan tp = tc_plan(ph, cta, grid);
                    const uint8_t* src = ph.w + (size_t)tp.b0 * HX_T128_CELL;
#pragma unroll 1
                    for (long long g = tp.b0; g < tp.b1 && ok; g++, src += HX_T128_CELL) ok = push(src, HX_T128_CELL);
                } else if (ph.type == HX_PH_ATTN) {
                    const AttPlan ap = att_plan(ph, cta, pos);
                    const size_t rowb = (size_t)ph.DH * 4;
                    if (ph.epi == HX_EPI_QKV) {
                        // tiles of up to tr slots of K rows followed by as many of V rows (attention_phase2)
                        const AttPlan2 ap2 = att_plan2(ap, (int)nring);
#pragma unroll 1
                        for (int t = 0; t < ap2.ntiles && ok; t++) {
                            const int r0 = ap.t0 + t * ap2.tile_rows, nrt = min(ap2.tile_rows, ap.t0 + ap.n_old - r0);
#pragma unroll 1
                            for (int kv2 = 0; kv2 < 2 && ok; kv2++) {
#pragma unroll 1
                                for (int r = 0; r < nrt && ok; r += ap.rows_per_slot) {
                                    const size_t off = ((size_t)ap.kv * ph.cap + r0 + r) * ph.DH;
                                    ok = push((kv2 ? ph.vc : ph.kc) + off, (uint32_t)(min(ap.rows_per_slot, nrt - r) * rowb));
                                }
                            }
                        }
                    } else
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
            const uint64_t sf_ring = tc_desc(smem_u32(ring) + 16384, 16, 128);
            const uint64_t b_base = tc_desc(smem_u32(digb), 16, 1024, TC_SW128);
            uint32_t ctr = 0, slot = 0, par = 0, uc = 0, tcph = 0;
            bool ok = true;
#pragma unroll 1
            for (int pi = 0; pi < P.nphases && ok; pi++) {
                const HxPhase& ph = P.phases[pi];
                if (ph.type == HX_PH_LINEAR_TC) {
                    const TcPlan tp = tc_plan(ph, cta, grid);                    // worked out while the consumers build the digits
                    ok = mbar_wait(&S.b_ready, tcph & 1, &S.abort_flag);        // digit columns of this phase are in place
                    tcph++;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    int kc = tp.k0, dp = 0;              // K cell of the tile, its position among the digit cells
                    bool fresh = true;
                    uint32_t dcol = 0;
#pragma unroll 1
                    for (long long g = tp.b0; g < tp.b1 && ok; g++) {
                        if (fresh) {
                            const uint32_t buf = uc & 1u;
                            if (uc >= 2) ok = mbar_wait(&S.acc_empty[buf], ((uc >> 1) - 1) & 1, &S.abort_flag);
                            if (!ok) break;
                            dcol = tmem + TM_D0 + buf * TC_NDIG;
                        }
                        ok = mbar_wait(&S.full[slot], par, &S.abort_flag);
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
                        ctr++;
                        if (++dp == tp.C) dp = 0;
                        if (++kc == tp.C || g + 1 == tp.b1) {          // last cell of this tile's piece
                            tc_commit(&S.acc_full[uc & 1u]);
                            uc++; kc = 0; fresh = true;
                        }
                    }
                } else if (ph.type == HX_PH_ATTN) {
                    const AttPlan ap = att_plan(ph, cta, pos);
                    const uint32_t adv = 2u * (uint32_t)ap.nslots;             // ring slots the consumers use for K and V rows
                    ctr += adv;
                    const uint32_t s2 = slot + adv;
                    slot = s2 % nring; if ((s2 / nring) & 1u) par ^= 1u;
                }
            }
        }
    } else {
        // =============================== consumers ===============================
        uint32_t ctr = 0, uc = 0;
        unsigned long long bar_target = P.bar_base;
        float best_v = -INFINITY; int best_i = INT_MAX;

        constexpr int PH_CHUNKS = (int)(sizeof(HxPhase) / 16);
        if (tid < PH_CHUNKS) reinterpret_cast<uint4*>(&S.ph[0])[tid] = __ldg(reinterpret_cast<const uint4*>(P.phases) + tid);
        consumer_sync();
#pragma unroll 1
        for (int pi = 0; pi < P.nphases; pi++) {
            const HxPhase& ph = S.ph[pi & 1];
            STAMP(0);
            if (ph.type == HX_PH_LINEAR_TC) {
                // ---------- prologue: x -> (norm) -> sixteen base-4 digit columns in operand layout ----------
                // Pass 1 (all of x): sum of squares and largest magnitude of x*g.  Pass 2: every thread turns items
                // of 8 consecutive elements of the K cells this CTA streams into digit words; the first item is
                // fetched before pass 1 so that its latency hides behind it.  Loops are kept rolled: this code runs
                // once per phase and is bound by instruction fetch, not by arithmetic.
                const int K = ph.K;
                const TcPlan tp = tc_plan(ph, cta, grid);
                const float* xin = ph.x;
                if (ph.tok) xin = ph.x + (size_t)(ph.tok[P.tok_by_pos ? pos : 0]) * K;
                const bool rms = ph.norm == HX_NORM_RMS;
                // tensor parallel: the vector is x + the partial sums every rank left in its slot of the exchange buffer
                const float* tpp = (TP && ph.tp_sum) ? P.tp_peer[P.tp_rank] + tp_off_part(P, ph.tp_sum - 1, 0) : nullptr;
                auto ldx4 = [&](int k) -> float4 {
                    float4 r = __ldcg(reinterpret_cast<const float4*>(xin + k));
                    if (TP && tpp) {
                        for (int w = 0; w < P.tp_world; w++) {
                            const float4 q = __ldcg(reinterpret_cast<const float4*>(tpp + (size_t)w * P.tp_dm + k));
                            r.x += q.x; r.y += q.y; r.z += q.z; r.w += q.w;
                        }
                    }
                    return r;
                };
                const int nitems = tp.run * 32;
                auto item_k = [&](int it) { int kc = tp.k0 + (it >> 5); if (kc >= tp.C) kc -= tp.C; return kc * 256 + (it & 31) * 8; };
                float4 ia = make_float4(0.f, 0.f, 0.f, 0.f), ib = ia, ja = make_float4(1.f, 1.f, 1.f, 1.f), jb = ja;
                if (tid < nitems && ph.norm != HX_NORM_ATTN) {
                    const int k = item_k(tid);
                    if (k < K) {
                        ia = ldx4(k);
                        if (k + 4 < K) ib = ldx4(k + 4);
                        if (rms) { ja = *reinterpret_cast<const float4*>(ph.g + k); if (k + 4 < K) jb = *reinterpret_cast<const float4*>(ph.g + k + 4); }
                    }
                }
                float inv = 1.0f, Sg = 1.0f;
                const bool merge_in = ph.norm == HX_NORM_ATTN;
                if (merge_in) {
                    // x is the merge of the attention splits: x[h*DH + d] = sum_s w[h][s] * acc[h][s][d] with
                    // w[h][s] = exp(m_s - M_h) / sum_s l_s exp(m_s - M_h).  Weights of all heads go to shared memory;
                    // the magnitude bound comes from the per-split bounds (the merge is a convex combination).
                    const int NS = ph.nsplit;
                    float mx = 0.0f;
                    for (int i = tid; i < ph.NH * NS; i += NCT) mx = fmaxf(mx, __ldcg(P.part_amax + i));
                    // two heads per pass so that their statistics travel together (one L2 round trip instead of two)
                    #pragma unroll 1
                    for (int h0 = warp; h0 < ph.NH; h0 += 2 * NCW) {
                        float mv[2][2], lv[2][2];
#pragma unroll
                        for (int u = 0; u < 2; u++) {
                            const int h = h0 + u * NCW;
#pragma unroll
                            for (int j = 0; j < 2; j++) {
                                const int sidx = lane + 32 * j;
                                const bool ok = h < ph.NH && sidx < NS;
                                mv[u][j] = ok ? __ldcg(P.part_m + (size_t)h * NS + sidx) : -INFINITY;
                                lv[u][j] = ok ? __ldcg(P.part_l + (size_t)h * NS + sidx) : 0.0f;
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 2; u++) {
                            const int h = h0 + u * NCW;
                            if (h >= ph.NH) break;
                            const float M = hx_warp_max(fmaxf(mv[u][0], mv[u][1]));
                            const float w0 = __expf(mv[u][0] - M), w1 = __expf(mv[u][1] - M);
                            const float Lsum = hx_warp_sum(lv[u][0] * w0 + lv[u][1] * w1);
                            if (lane < NS) S.wgt[h * NS + lane] = w0 / Lsum;
                            if (lane + 32 < NS) S.wgt[h * NS + lane + 32] = w1 / Lsum;
                        }
                    }
                    mx = hx_warp_max(mx);
                    if (lane == 0) S.red[NCW + warp] = mx;
                    consumer_sync();
                    float tmx = 0.0f;
#pragma unroll
                    for (int i = 0; i < NCW; i++) tmx = fmaxf(tmx, S.red[NCW + i]);
                    const float vmax = tmx * 1.0001f;                      // margin for the rounding of the merge
                    if (vmax > 0.0f && vmax < INFINITY) Sg = __uint_as_float(__float_as_uint(vmax) & 0x7F800000u);
                } else {
                    float ss = 0.0f, mx = 0.0f;
#pragma unroll 1
                    for (int k0 = tid * 4; k0 < K; k0 += NCT * 4 * 3) {
                        float4 v[3], gq[3];
#pragma unroll
                        for (int u = 0; u < 3; u++) {
                            const int k = k0 + u * NCT * 4;
                            v[u] = make_float4(0.f, 0.f, 0.f, 0.f); gq[u] = v[u];
                            if (k < K) {
                                v[u] = ldx4(k);
                                if (rms) gq[u] = *reinterpret_cast<const float4*>(ph.g + k);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 3; u++) {
                            const int k = k0 + u * NCT * 4;
                            if (k < K) {
                                if ((ph.tok || tpp) && ph.x_out && ((k >> 2) % grid) == cta) *reinterpret_cast<float4*>(ph.x_out + k) = v[u];
                                if (rms) {
                                    ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
                                    mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v[u].x * gq[u].x), fabsf(v[u].y * gq[u].y)), fmaxf(fabsf(v[u].z * gq[u].z), fabsf(v[u].w * gq[u].w))));
                                } else mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w))));
                            }
                        }
                    }
                    ss = hx_warp_sum(ss); mx = hx_warp_max(mx);
                    if (lane == 0) { S.red[warp] = ss; S.red[NCW + warp] = mx; }
                    consumer_sync();
                    float tss = 0.0f, tmx = 0.0f;
#pragma unroll
                    for (int i = 0; i < NCW; i++) { tss += S.red[i]; tmx = fmaxf(tmx, S.red[NCW + i]); }
                    if (rms) inv = rsqrtf(tss / (float)K + ph.eps);
                    const float vmax = tmx * inv * 1.0000005f;            // margin for the rounding of x*g*inv
                    if (vmax > 0.0f && vmax < INFINITY) Sg = __uint_as_float(__float_as_uint(vmax) & 0x7F800000u);   // vmax/Sg in [1,2)
                }
                STAMP(14);
                const float mul = (inv / Sg) * 2147483648.0f;             // |x_n| / Sg * 2^31 < 2^32
                if (merge_in) {
                    // TPI threads share an item: each sums every TPI-th split, a butterfly adds them up (all lanes
                    // end with the same bits), then each lane writes its share of the sixteen digit rows.
                    const int NS = ph.nsplit, DH = ph.DH;
                    int tpi = 1; while (tpi < 8 && nitems * tpi * 2 <= NCT) tpi *= 2;
                    const int sub = tid & (tpi - 1);
#pragma unroll 1
                    for (int it = tid / tpi; it < nitems; it += NCT / tpi) {
                        const int k = item_k(it);
                        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                        if (k < K) {
                            const int h = k / DH, d = k - h * DH;
                            const float* pa = P.part_acc + ((size_t)h * NS) * DH + d;
#pragma unroll 3
                            for (int sp2 = sub; sp2 < NS; sp2 += tpi) {
                                const float4 a = __ldcg(reinterpret_cast<const float4*>(pa + (size_t)sp2 * DH));
                                const float4 b = __ldcg(reinterpret_cast<const float4*>(pa + (size_t)sp2 * DH + 4));
                                const float w = S.wgt[h * NS + sp2];
                                v[0] = fmaf(a.x, w, v[0]); v[1] = fmaf(a.y, w, v[1]); v[2] = fmaf(a.z, w, v[2]); v[3] = fmaf(a.w, w, v[3]);
                                v[4] = fmaf(b.x, w, v[4]); v[5] = fmaf(b.y, w, v[5]); v[6] = fmaf(b.z, w, v[6]); v[7] = fmaf(b.w, w, v[7]);
                            }
                        }
                        for (int dlt = 1; dlt < tpi; dlt <<= 1) {
#pragma unroll
                            for (int e = 0; e < 8; e++) v[e] += __shfl_xor_sync(0xffffffffu, v[e], dlt);
                        }
                        uint32_t M[8]; uint32_t sg = 0u;
#pragma unroll
                        for (int e = 0; e < 8; e++) {
                            M[e] = __float2uint_rn(fabsf(v[e]) * mul);
                            sg |= (v[e] < 0.0f ? 8u : 0u) << (4 * e);
                        }
                        const int j = (it >> 2) & 7, w = it & 3;
                        uint8_t* dst = digb + (size_t)(it >> 5) * 2048 + w * 4;
#pragma unroll 2
                        for (int n = sub; n < TC_NDIG; n += tpi) {
                            uint32_t word = 0u;
#pragma unroll
                            for (int e = 0; e < 8; e++) word |= ((M[e] >> (30 - 2 * n)) & 3u) << (4 * e);
                            const uint32_t nz = (word | (word >> 1)) & 0x11111111u;
                            word |= sg & (nz << 3);
                            *reinterpret_cast<uint32_t*>(dst + n * 128 + ((j ^ (n & 7)) << 4)) = word;
                        }
                    }
                } else
#pragma unroll 1
                for (int it = tid; it < nitems; it += NCT) {
                    const int k = item_k(it);
                    if (it != tid) {                                       // later items of a long run: fetched here
                        ia = make_float4(0.f, 0.f, 0.f, 0.f); ib = ia; ja = make_float4(1.f, 1.f, 1.f, 1.f); jb = ja;
                        if (k < K) {
                            ia = ldx4(k);
                            if (k + 4 < K) ib = ldx4(k + 4);
                            if (rms) { ja = *reinterpret_cast<const float4*>(ph.g + k); if (k + 4 < K) jb = *reinterpret_cast<const float4*>(ph.g + k + 4); }
                        }
                    }
                    const float v[8] = {ia.x * ja.x, ia.y * ja.y, ia.z * ja.z, ia.w * ja.w, ib.x * jb.x, ib.y * jb.y, ib.z * jb.z, ib.w * jb.w};
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
                STAMP(15);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                consumer_sync();
                if (tid == 0) mbar_arrive(&S.b_ready);
                STAMP(1);

                // ---------- pieces of tiles: accumulator -> digits recombined -> (merge) -> epilogue ----------
                ctr += (uint32_t)(tp.b1 - tp.b0);
                // number of pieces this CTA produces: one per tile its run touches
                const int t_first = (int)((unsigned)tp.b0 / (unsigned)tp.C), t_last = tp.b1 > tp.b0 ? (int)((unsigned)(tp.b1 - 1) / (unsigned)tp.C) : t_first - 1;
                if (warp < EPI_WARPS) {
                    const float out_scale = Sg;       // x_n = Sg * sum_j 4^-j * (digit_j / 2), and digit/2 is the E2M1 value
                    const int rl = warp * 32 + lane;
#pragma unroll 1
                    for (int tile = t_first; tile <= t_last; tile++) {
                        const uint32_t buf = uc & 1u;
                        // the residual row is final since the last barrier: fetch it while the MMAs of this piece run
                        float yres = 0.0f;
                        if (ph.epi == HX_EPI_RESID && !(TP && ph.tp_partial) && tile * 128 + rl < ph.N) yres = __ldcg(ph.y + tile * 128 + rl);
                        // likewise the norm gain and the RoPE factors of this row (qkv epilogue)
                        float pre_g = 1.0f, pre_cs = 1.0f, pre_sn = 0.0f;
                        if (ph.epi == HX_EPI_QKV) {
                            const int row = tile * 128 + rl, e = row % ph.DH, half = ph.DH >> 1;
                            const int sec = row < ph.NH * ph.DH ? 0 : (row < (ph.NH + ph.NKV) * ph.DH ? 1 : 2);
                            const float* gg = sec == 0 ? ph.qn_g : (sec == 1 ? ph.kn_g : nullptr);
                            if (gg) pre_g = gg[e];
                            if (ph.cosT) { pre_cs = ph.cosT[(size_t)pos * half + (e < half ? e : e - half)]; pre_sn = ph.sinT[(size_t)pos * half + (e < half ? e : e - half)]; }
                        }
                        if (!mbar_wait(&S.acc_full[buf], (uc >> 1) & 1, &S.abort_flag)) break;   // flag is latched; leave with the others at the barrier
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
                        // which CTAs share this tile
                        const long long x0 = (long long)tile * tp.C;
                        const int c0 = tp.P ? tile * tp.P : tc_owner(x0, tp.total, tp.geff);
                        const int c1 = tp.P ? c0 + tp.P - 1 : tc_owner(x0 + tp.C - 1, tp.total, tp.geff);
                        if (c1 != c0) {
                            float* pp = P.tc_partial + ((size_t)tile * ph.pieces) * 128;
                            pp[(size_t)(cta - c0) * 128 + rl] = v;
                            epi_sync();
                            if (tid == 0) S.eticket = ticket_acq_rel(P.tc_cnt + tile);
                            epi_sync();
                            if (S.eticket != (unsigned)(c1 - c0)) continue;          // a later piece finishes the tile
                            v = 0.0f;
                            for (int q = 0; q <= c1 - c0; q++) v += __ldcg(pp + (size_t)q * 128 + rl);
                            if (tid == 0) P.tc_cnt[tile] = 0u;
                        }
                        if (ph.epi == HX_EPI_QKV) {
                            // A tile holds 128 / DH whole heads (DH is 32, 64 or 128).  Per-head RMSNorm and rotate_half
                            // RoPE on q and k; q goes to the qkv buffer, k and v to the cache row of this position.
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
                                const float cs = pre_cs, sn = pre_sn;
                                if (sec < 2) v = e < half ? v * cs - other * sn : v * cs + other * sn;
                                epi_sync();
                            }
                            if (valid) {
                                if (sec == 0) ph.y[row] = v;
                                else {
                                    const int hrow = row - QD - (sec == 2 ? KVD : 0);
                                    float* dst = sec == 1 ? ph.kc : ph.vc;
                                    dst[((size_t)(hrow / DH) * ph.cap + pos) * DH + e] = v;
                                }
                            }
                        } else if (ph.epi == HX_EPI_SWIGLU) {
                            // rows 0..63 of a tile are gate rows, 64..127 the matching up rows
                            S.swi[rl] = v * (rl < 64 ? ph.ts[0] : ph.ts[1]);
                            epi_sync();
                            const int hi = tile * 64 + rl;
                            if (rl < 64 && hi < ph.N) ph.y[hi] = pz_silu_mul(S.swi[rl], S.swi[rl + 64]);
                            epi_sync();
                        } else {
                            const int row = tile * 128 + rl;
                            if (row < ph.N) {
                                v *= (row < ph.bound0) ? ph.ts[0] : (row < ph.bound1 ? ph.ts[1] : ph.ts[2]);
                                if (TP && ph.tp_partial) {
                                    // row-split linear: this rank's partial sum of the row goes to every rank's buffer;
                                    // the consumer's prologue adds them to the residual stream in rank order
                                    const size_t o = tp_off_part(P, ph.tp_partial - 1, P.tp_rank) + row;
                                    for (int w = 0; w < P.tp_world; w++) P.tp_peer[w][o] = v;
                                } else {
                                    if (ph.epi == HX_EPI_RESID) v = yres + v;
                                    ph.y[row] = v;
                                }
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
                        if (TP && lane == 0 && P.tp_world > 1) {
                            // vocabulary split over the ranks: exchange (value, global index) and take the best of all
                            const size_t ao = tp_off_am(P) + 2 * P.tp_rank;
                            const int gi = bi == INT_MAX ? INT_MAX : bi + P.tp_vocab_off;
                            for (int w = 0; w < P.tp_world; w++) { P.tp_peer[w][ao] = bv; reinterpret_cast<int*>(P.tp_peer[w])[ao + 1] = gi; }
                            if (!tp_handshake(P, tp_off_amflags(P), P.tp_epoch_base + 4095u, &S.abort_flag)) { S.abort_flag = 1; *P.err = 1; }
                            bv = -INFINITY; bi = INT_MAX;
                            const float* am = P.tp_peer[P.tp_rank] + tp_off_am(P);
                            for (int w = 0; w < P.tp_world; w++) {
                                const float ov = __ldcg(am + 2 * w); const int oi = __ldcg(reinterpret_cast<const int*>(am) + 2 * w + 1);
                                if (pz_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
                            }
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
                if (ph.epi == HX_EPI_QKV) switch (ph.NH / ph.NKV) {
                    case 1: ok = attention_phase2<1>(P, ph, S, ring, digb, ctr, pi, pos); break;
                    case 2: ok = attention_phase2<2>(P, ph, S, ring, digb, ctr, pi, pos); break;
                    case 3: ok = attention_phase2<3>(P, ph, S, ring, digb, ctr, pi, pos); break;
                    case 4: ok = attention_phase2<4>(P, ph, S, ring, digb, ctr, pi, pos); break;
                    case 5: ok = attention_phase2<5>(P, ph, S, ring, digb, ctr, pi, pos); break;
                    case 6: ok = attention_phase2<6>(P, ph, S, ring, digb, ctr, pi, pos); break;
                    case 7: ok = attention_phase2<7>(P, ph, S, ring, digb, ctr, pi, pos); break;
                    default: ok = attention_phase2<8>(P, ph, S, ring, digb, ctr, pi, pos); break;
                }
                else switch (ph.NH / ph.NKV) {
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
            STAMP_ALL();
            // ---------- grid barrier ----------
            if (pi + 1 < P.nphases) {
                // the next descriptor travels to shared memory while the barrier is pending
                if (tid < PH_CHUNKS)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_u32(reinterpret_cast<uint4*>(&S.ph[(pi + 1) & 1]) + tid)),
                                 "l"(reinterpret_cast<const uint4*>(P.phases + pi + 1) + tid) : "memory");
                consumer_sync();                 // every thread's results are ordered before thread 0's release below
                bar_target += (unsigned long long)grid;
                if (tid == 0) {
                    if (TP && ph.tp_barrier) asm volatile("red.release.sys.global.add.u64 [%0], 1;" :: "l"(P.bar) : "memory");   // covers the stores to the peers
                    else asm volatile("red.release.gpu.global.add.u64 [%0], 1;" :: "l"(P.bar) : "memory");
                    bool ok = false;
                    for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
                        unsigned long long v;
                        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(P.bar) : "memory");
                        if (v >= bar_target) { ok = true; break; }
                        if ((i & 255) == 255 && S.abort_flag) break;
                    }
                    if (!ok) S.abort_flag = 1;
                    if (TP && ok && ph.tp_barrier) {
                        // all CTAs of this GPU have arrived: CTA 0 tells the other GPUs, and every CTA waits until each peer
                        // has said the same (the peers' flags land in local memory, so the wait costs one NVLink crossing)
                        const unsigned ep = P.tp_epoch_base + (unsigned)ph.tp_epoch;
                        if (cta == 0) tp_signal(P, tp_off_flags(P), ep);
                        if (!tp_wait(P, tp_off_flags(P), ep, &S.abort_flag)) S.abort_flag = 1;
                    }
                }
                asm volatile("cp.async.wait_all;" ::: "memory");
                consumer_sync();
                if (S.abort_flag) goto aborted;
            }
            STAMP(3);
        }
        if (S.abort_flag) goto aborted;
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
    return ((sizeof(SmemTc) + 15) & ~(size_t)15) + 512 + 1024 + d;      // + ring slots
}

// Ring depth that fits beside the digit columns (0 = does not fit).
int hx_persist_tc_ring(int bdig_bytes) {
    const size_t fixed = hx_persist_tc_smem(bdig_bytes);
    if (fixed + 3 * (size_t)HX_RING_SLOT > 227 * 1024) return 0;
    size_t n = (227 * 1024 - fixed) / HX_RING_SLOT;
    return (int)(n > HX_TC_MAX_RING ? HX_TC_MAX_RING : n);
}

int hx_persist_tc_launch(const HxPersist& p, int grid, cudaStream_t st) {
    if (p.tc_ring < 3 || p.tc_ring > HX_TC_MAX_RING) return hx_fail(HX_ERR_ARG, "tensor-core decode: ring depth %d", p.tc_ring);
    const size_t smem = hx_persist_tc_smem(p.bdig_bytes) + (size_t)p.tc_ring * HX_RING_SLOT;
    if (smem > 227 * 1024) return hx_fail(HX_ERR_ARG, "tensor-core decode needs %zu bytes of shared memory", smem);
    static std::atomic<unsigned long long> attr_seen{0};
    if (hx_first_on_device(attr_seen)) {
        HX_CUDA(cudaFuncSetAttribute(k_decode_tc<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        HX_CUDA(cudaFuncSetAttribute(k_decode_tc<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    }
    void* args[] = {(void*)&p};
    void* fn = p.tp_world > 1 ? (void*)k_decode_tc<true> : (void*)k_decode_tc<false>;
    HX_CUDA(cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(PT), args, smem, st));
    HX_COUNT_LAUNCH(1);
    return HX_OK;
}
