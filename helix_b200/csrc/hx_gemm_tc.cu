// hx_gemm_tc.cu -- block-scaled NVFP4 GEMM on the 5th-generation tensor cores (tcgen05, TMEM).
//
//   D[row, n] = sum_k  A[row,k] * SFA[row,k/16]  *  B[n,k] * SFB[n,k/16]         (f32 accumulate in TMEM)
//
// A = weights, E2M1 codes with one UE4M3 scale per 16 elements along K: exactly the information of
// the committed NVFP4 layout (helixc/runtime/gpt2_pack.c:350-373), so the weights feed the tensor
// cores without any per-weight instruction.  B = activations as E2M1 columns: in digit mode (the chunk
// paths: batched prefill, batched decode, the verify forward; replaces tiled_matmul_abt of
// forward_layer_llama, helixc/runtime/gpt2_infer.c:1231-1287) ten balanced base-9 digit columns per token
// with unit block scales, folded in the epilogue; in raw mode (hx_gemm_nvfp4_tc) any E2M1 columns with
// their own UE4M3 block scales, the accumulators stored as they are.
//
// Work units of one 128-row tile of A (times a piece of K and a group of 16 tokens), a CTA per SM walking
// through its units.  Warp 0 streams A (and, in raw mode, B) cells into a shared-memory ring with
// cp.async.bulk; warp 1 copies the scale factors to TMEM (tcgen05.cp) and issues
// tcgen05.mma.kind::mxf4nvf4.block_scale (M=128, N=ncols of the group, K=64 per instruction); warps 2-9 read
// the accumulator with tcgen05.ld and store it while the next unit's MMAs run; warp 10 counts the finished K
// pieces of a tile.  In digit mode the B cells of a CTA's (K piece, token group) stay in shared memory, so
// only the weights stream: once per launch from DRAM.
//
// "T128" layout of A: per (128-row tile, group of 256 columns = four MMA K steps) one 18432-byte cell:
// 128 rows x 128 bytes of codes in the canonical K-major 128-byte-swizzle operand layout (row r at
// r*128, its 16-byte chunk j stored at position j ^ (r & 7)), then four 512-byte scale chunks, one per
// K step (byte (row%32)*16 + (row/32)*4 + block).  B cells: N rows x 128 swizzled bytes + four scale
// chunks indexed by n.  The cells are the shared-memory image, so plain bulk copies load them; the
// 128-byte swizzle lets the tensor core fetch operands at full shared-memory width (the unswizzled
// layout measured 8x slower per instruction).  Every wait is bounded.
#include "hx_common.cuh"
#include "hx_gemm_tc.cuh"
#include <stdlib.h>

#define TC_WAIT_LIMIT (1u << 22)

// Timing probes of a debug build (-DTC_STAMPS): CTA 0 leaves globaltimer values in tc_stamps[role][unit][event].
#ifdef TC_STAMPS
__device__ unsigned long long tc_stamps[3][32][8];
__device__ long long tc_clocks[3][32][8];
#define TC_MARK(role, unit, ev) do { if (blockIdx.x == 0 && (unit) < 32) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); tc_stamps[role][unit][ev] = t_; tc_clocks[role][unit][ev] = clock64(); } } while (0)
#else
#define TC_MARK(role, unit, ev) do { } while (0)
#endif

namespace {

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mb_init(uint64_t* b, uint32_t n) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(s_u32(b)), "r"(n) : "memory"); }
__device__ __forceinline__ void mb_expect(uint64_t* b, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(s_u32(b)), "r"(bytes) : "memory"); }
__device__ __forceinline__ void mb_arrive(uint64_t* b) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(s_u32(b)) : "memory"); }
__device__ __forceinline__ bool mb_try(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(s_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mb_wait(uint64_t* b, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < TC_WAIT_LIMIT; i++) {
        if (mb_try(b, parity)) return true;
        if ((i & 255) == 255 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(s_u32(dst)), "l"(src), "r"(bytes), "r"(s_u32(bar)) : "memory");
}
// K-major, no swizzle: 8 rows x 16 bytes core matrices; lbo = byte distance between the two 16-byte
// K halves, sbo = byte distance between 8-row groups.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout = 0) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) |
           (1ull << 46) | ((uint64_t)layout << 61);
}
#define SW128 2u
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" :: "r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                 :: "r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(s_u32(bar)) : "memory");
}

struct TcSmem {
    uint64_t full[HX_TC_STAGES], empty[HX_TC_STAGES], accum[2], acc_free[2], part_done, tk_ready, bfull[HX_TC_RES_CELLS];
    uint32_t tmem_base;
    unsigned ticket[2];
    volatile int abort_flag;
};
#define TC_EPI_Q 3              // epilogue warps per quarter of the TMEM lanes: each takes eight tokens (or every third group of eight columns)
#define TC_THREADS ((3 + 4 * TC_EPI_Q) * 32)      // warp 0 loads, warp 1 issues the MMAs, warps 2-13 read the accumulators, warp 14 draws the tickets
#define TC_HDR 1536u            // header + the chunk of unit scales
#define TC_SWI (HX_TC_MAX_TOK * 128 * 4)      // SwiGLU exchange: [token][row of the tile]
#define TC_DIGIT_CELL (HX_TC_GROUP_COLS * 128)      // digit cell of one token group: 240 rows of 128 bytes

__device__ __forceinline__ void tc_ld8(uint32_t (&r)[8], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr));
}

// The roles run through the CTA's work units on their own and meet only at mbarriers: `full`/`empty` per ring slot
// between the loader and the MMA issuer, `accum` (accumulator complete) and `acc_free` (accumulator read out) between
// the issuer and the twelve epilogue warps.
//
// Digit mode (the chunk paths).  Work units: (128-row tile, K piece, group of 24 tokens).  An activation enters as ten
// balanced base-9 digits (-4 .. 4: E2M1 values) of the 30-bit integer |x| / scale * 2^29, digit d of token t in column
// 24 d + t of the group: 240 columns per MMA, whose cost does not depend on the column count.  Two accumulators of 240
// columns fill TMEM together with one set of scale-factor columns, so the MMAs of a unit run while the accumulator of
// the unit before is read out: per token and row the ten digit accumulators are folded by Horner's rule
// (v = 9 v + D_d, most significant digit first) -- f32-accurate, not exact: the digits' own resolution is 2^-29 of
// the largest element.  K is cut into pieces of whole 256-column cells; each piece leaves its values in `partial`, and
// the last piece of a (tile, group) to finish (a ticket) adds the pieces in K order and applies the epilogue, so the
// result does not depend on the order the CTAs finish in.  The ticket of a unit is drawn by a warp of its own after the
// unit's partial sums are stored and looked at one unit later, so neither its round trip nor the wait for the stores
// holds up an epilogue warp.  The grid is a multiple of pieces x groups: a CTA keeps one (piece, group), loads its
// digit cells once, and the CTAs of the groups walk through the same tiles together, so a weight cell comes from
// DRAM once.
//
// Raw mode (hx_gemm_nvfp4_tc): one accumulator, the ring holds the A and the B cells of a stage, the accumulators
// are stored as they are.
__global__ void __launch_bounds__(TC_THREADS, 1) k_gemm_tc(const __grid_constant__ HxGemmTC g) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    TcSmem& S = *reinterpret_cast<TcSmem*>(smem_raw);
    // swizzled operands need 1024-byte aligned cells (the swizzle is a function of the shared-memory address)
    static_assert(sizeof(TcSmem) <= 1024, "header overlaps the unit-scale chunk");
    float* swi = reinterpret_cast<float*>(smem_raw + TC_HDR);
    uint8_t* ring = smem_raw + (((s_u32(smem_raw) + TC_HDR + TC_SWI + 1023u) & ~1023u) - s_u32(smem_raw));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int Sk = g.stage_ksteps;
    const int P = g.ksplit > 1 ? g.ksplit : 1, kcells = g.ksteps / 4;
    const bool DG = g.digit_mode != 0;      // digit mode: resident digit cells, two accumulators
    const int G = DG ? (g.ntok + HX_TC_MAX_TOK - 1) / HX_TC_MAX_TOK : 1, PG = P * G;
    const int nunits = g.ntiles * PG;
    const int grp = ((int)blockIdx.x % PG) % G;
    const int NB = DG ? HX_TC_GROUP_COLS : g.ncols;                                         // columns of this CTA's MMAs
    const uint32_t b_src_cell = DG ? (uint32_t)G * TC_DIGIT_CELL : (uint32_t)g.ncols * 128u + 2048u;      // one 256-column cell of B in memory
    const uint32_t b_cell_bytes = DG ? (uint32_t)TC_DIGIT_CELL : b_src_cell;                // ... and in shared memory
    const uint32_t a_cell = HX_T128_CELL / 4, b_cell = b_cell_bytes / 4;                     // bytes per K step
    const uint32_t stage_bytes = (uint32_t)Sk * (a_cell + (DG ? 0u : b_cell));
    uint8_t* bres = ring + (size_t)HX_TC_STAGES * stage_bytes;      // digit mode: [cells of a piece][240 * 128]

    if (tid < 128) reinterpret_cast<uint32_t*>(smem_raw + 1024)[tid] = 0x38383838u;      // a chunk of unit scales (digit mode)
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (tid == 0) {
        for (int i = 0; i < HX_TC_STAGES; i++) { mb_init(&S.full[i], 1); mb_init(&S.empty[i], 1); }
        for (int i = 0; i < HX_TC_RES_CELLS; i++) mb_init(&S.bfull[i], 1);
        for (int i = 0; i < 2; i++) { mb_init(&S.accum[i], 1); mb_init(&S.acc_free[i], 4 * TC_EPI_Q); }
        mb_init(&S.part_done, 4 * TC_EPI_Q); mb_init(&S.tk_ready, 1);
        S.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {    // one warp owns the TMEM allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" :: "r"(s_u32(&S.tmem_base)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = S.tmem_base;
    // TMEM columns.  Raw mode: [0, 256) accumulator, then per ring slot Sk*4 columns of SFA and of SFB.  Digit mode:
    // two accumulators of 240 columns, sixteen columns for the scale factors of the stage at hand (the tensor pipe works
    // through copies and MMAs in the order they were issued, so the copy of the next stage follows the MMAs of this one),
    // sixteen for the unit scales of the digit columns.
    const uint32_t col_sfa = DG ? 2u * HX_TC_GROUP_COLS : 256u;
    const uint32_t col_sfb = DG ? 2u * HX_TC_GROUP_COLS + 16u : 256u + HX_TC_STAGES * HX_TC_MAX_SK * 4;
    static_assert(2 * HX_TC_GROUP_COLS + 32 <= 512, "two accumulators and the scale factors fill TMEM");
    // unit u of this CTA: tile u / PG and, with `combo` = u % PG, piece combo / G (and group combo % G = grp)
#define TC_UNIT(u) const int mt = (u) / PG, piece = ((u) - mt * PG) / G; \
                   const int ks_lo = (piece * kcells / P) * 4, ks_hi = ((piece + 1) * kcells / P) * 4

    if (warp == 0) {
        // ------------------------------ loader ------------------------------
        if (lane == 0) {
            uint32_t git = 0;
            bool ok = true;
            if (DG) {
                const int piece0 = ((int)blockIdx.x % PG) / G;
                const int c_lo = piece0 * kcells / P, c_hi = (piece0 + 1) * kcells / P;
                for (int c = c_lo; c < c_hi; c++) {
                    mb_expect(&S.bfull[c - c_lo], b_cell_bytes);
                    bulk_load(bres + (size_t)(c - c_lo) * b_cell_bytes, g.b + (size_t)c * b_src_cell + (size_t)grp * TC_DIGIT_CELL, b_cell_bytes, &S.bfull[c - c_lo]);
                }
            }
            int lu = 0;
            for (int u = blockIdx.x; u < nunits && ok; u += gridDim.x, lu++) {
                TC_UNIT(u);
                TC_MARK(0, lu, 0);
                for (int ks0 = ks_lo; ks0 < ks_hi; ks0 += Sk, git++) {
                    const uint32_t slot = git % HX_TC_STAGES, round = git / HX_TC_STAGES;
                    if (round > 0 && !mb_wait(&S.empty[slot], (round - 1) & 1, &S.abort_flag)) { ok = false; break; }
                    const int nk = min(Sk, ks_hi - ks0);
                    uint8_t* sa = ring + (size_t)slot * stage_bytes;
                    uint8_t* sb = sa + (size_t)Sk * a_cell;
                    mb_expect(&S.full[slot], (uint32_t)nk * (a_cell + (DG ? 0u : b_cell)));
                    bulk_load(sa, g.a + ((size_t)mt * g.ksteps + ks0) * a_cell, (uint32_t)nk * a_cell, &S.full[slot]);
                    if (!DG) bulk_load(sb, g.b + (size_t)ks0 * b_cell, (uint32_t)nk * b_cell, &S.full[slot]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            // instruction descriptor: E2M1 x E2M1, UE4M3 scales, K-major both, N = NB, M = 128, K = 64
            const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) | (8u << 24);
            uint32_t git = 0;
            bool ok = true;
            int unit_iter = 0;
            if (DG) {
                // One (piece, group) for the whole CTA: its stages form one sequence, a cell of A against a resident cell of
                // B each.  The four descriptors of a cell differ by constants (the address field counts 16-byte units).
                const uint64_t dA0 = smem_desc(s_u32(ring), 16, 1024, SW128), dS0 = smem_desc(s_u32(ring) + 16384, 16, 128);
                const uint64_t dB0 = smem_desc(s_u32(bres), 16, 1024, SW128);
                // unit scales (E4M3 1.0) for every digit column: sixteen TMEM columns cover any N up to 256
                for (int c = 0; c < 4; c++) tc_cp_sf(tmem + col_sfb + c * 4, smem_desc(s_u32(smem_raw + 1024), 16, 128));
                const int piece0 = ((int)blockIdx.x % PG) / G;
                const int ncell = (piece0 + 1) * kcells / P - piece0 * kcells / P;
                const int nu = ((int)blockIdx.x < nunits) ? (nunits - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
                const uint32_t total = (uint32_t)(nu * ncell);
                int ci = 0;
                for (git = 0; git < total && ok; git++) {
                    const uint32_t acc = tmem + (uint32_t)(unit_iter & 1) * HX_TC_GROUP_COLS;
                    if (ci == 0) {
                        TC_MARK(1, unit_iter, 0);
                        if (unit_iter >= 2) {      // the epilogue has read this accumulator's previous unit out
                            if (!mb_wait(&S.acc_free[unit_iter & 1], (uint32_t)((unit_iter >> 1) - 1) & 1u, &S.abort_flag)) break;
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        }
                        TC_MARK(1, unit_iter, 1);
                    }
                    const uint32_t slot = git % HX_TC_STAGES, round = git / HX_TC_STAGES;
                    if (git < (uint32_t)ncell && !mb_wait(&S.bfull[git], 0, &S.abort_flag)) { ok = false; break; }
                    if (!mb_wait(&S.full[slot], round & 1, &S.abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (ci == 0) TC_MARK(1, unit_iter, 2);
                    const uint64_t dA = dA0 + (uint64_t)((slot * stage_bytes) >> 4), dS = dS0 + (uint64_t)((slot * stage_bytes) >> 4);
                    const uint64_t dB = dB0 + (uint64_t)(((uint32_t)ci * b_cell_bytes) >> 4);
#pragma unroll
                    for (int k = 0; k < 4; k++) tc_cp_sf(tmem + col_sfa + k * 4, dS + (uint64_t)(k * 32));
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        tc_mma(acc, dA + (uint64_t)(k * 2), dB + (uint64_t)(k * 2), idesc, tmem + col_sfa + k * 4, tmem + col_sfb, (k > 0 || ci > 0) ? 1u : 0u);
                    tc_commit(&S.empty[slot]);          // the slot is free once these MMAs have read it
                    if (++ci == ncell) {
                        tc_commit(&S.accum[unit_iter & 1]);            // accumulator complete
                        TC_MARK(1, unit_iter, 3);
                        ci = 0; unit_iter++;
                    }
                }
            } else
            for (int u = blockIdx.x; u < nunits && ok; u += gridDim.x, unit_iter++) {
                TC_UNIT(u);
                (void)mt;
                if (unit_iter > 0) {      // the epilogue has read the previous unit's accumulator out
                    if (!mb_wait(&S.acc_free[0], (uint32_t)(unit_iter - 1) & 1u, &S.abort_flag)) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                }
                for (int ks0 = ks_lo; ks0 < ks_hi; ks0 += Sk, git++) {
                    const uint32_t slot = git % HX_TC_STAGES, round = git / HX_TC_STAGES;
                    if (!mb_wait(&S.full[slot], round & 1, &S.abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const int nk = min(Sk, ks_hi - ks0);
                    const uint32_t sa = s_u32(ring + (size_t)slot * stage_bytes);
                    const uint32_t sb = sa + (uint32_t)Sk * a_cell;
                    for (int k = 0; k < nk; k++) {
                        const uint32_t ta = tmem + col_sfa + (slot * HX_TC_MAX_SK + k) * 4;
                        const uint32_t tb = tmem + col_sfb + (slot * HX_TC_MAX_SK + k) * 4;
                        const uint32_t acell = sa + (uint32_t)(k >> 2) * HX_T128_CELL, bcell = sb + (uint32_t)(k >> 2) * b_cell_bytes;
                        const uint32_t e = (uint32_t)(k & 3);
                        tc_cp_sf(ta, smem_desc(acell + 16384 + e * 512, 16, 128));
                        tc_cp_sf(tb, smem_desc(bcell + (uint32_t)NB * 128u + e * 512, 16, 128));
                        tc_mma(tmem, smem_desc(acell + e * 32, 16, 1024, SW128), smem_desc(bcell + e * 32, 16, 1024, SW128), idesc,
                               ta, tb, (ks0 > ks_lo || k > 0) ? 1u : 0u);
                    }
                    tc_commit(&S.empty[slot]);          // the slot is free once these MMAs have read it
                }
                if (ok) tc_commit(&S.accum[0]);         // accumulator complete
            }
        }
    } else if (warp < 2 + 4 * TC_EPI_Q) {
        // ------------------------------ epilogue: TMEM -> registers -> global ------------------------------
        const int ew = warp - 2, sub = warp & 3, third = ew >> 2;      // TMEM lanes 32*sub .. 32*sub+31; tokens 8*third .. 8*third+7 of the group
        const int rl = sub * 32 + lane, etid = tid - 64;
        const uint32_t bar_third = 1u + (uint32_t)third;             // named barriers 1 .. 3: the four warps that share a set of tokens
        constexpr int TH = HX_TC_MAX_TOK / TC_EPI_Q;
        static_assert(TH == 8, "a warp reads its tokens' digit accumulators as eight columns per digit");
        const int ntok = DG ? min(HX_TC_MAX_TOK, g.ntok - grp * HX_TC_MAX_TOK) : 0;      // tokens of this CTA's group
        const int tok0 = grp * HX_TC_MAX_TOK + third * TH;             // this thread's tokens: tok0 .. tok0+TH-1 of the launch
        const int tleft = ntok - third * TH;                           // ... of which tleft exist
        constexpr int ptok = HX_TC_NTOK;                               // token slots of a piece in `partial` (a constant: the loads of a merge differ by immediates)
        float cs[TH];
#pragma unroll
        for (int t = 0; t < TH; t++) cs[t] = (DG && t < tleft) ? __ldg(g.col_scale + tok0 + t) : 0.0f;
        bool dead = false;      // a wait ran out: keep to the barrier protocol, touch nothing
        // final values of tile mtf: tensor scale, then store / residual add / SwiGLU across the gate (rows 0..63 of the
        // tile) and up (rows 64..127) halves
        auto finalize = [&](int mtf, const float (&val)[TH], const float (&prev)[TH]) {
            const int row = mtf * 128 + rl;
            const float tsr = g.pair64 ? ((rl < 64) ? g.ts[0] : g.ts[1])
                                       : (row < g.bound0 ? g.ts[0] : (row < g.bound1 ? g.ts[1] : g.ts[2]));
            if (g.swiglu) {
#pragma unroll
                for (int t = 0; t < TH; t++) swi[(third * TH + t) * 128 + rl] = val[t] * tsr;
                asm volatile("bar.sync %0, 128;" :: "r"(bar_third) : "memory");
                if (rl < 64 && mtf * 64 + rl < g.rows && !dead) {
#pragma unroll
                    for (int t = 0; t < TH; t++) {
                        if (t >= tleft) break;
                        const float gt = swi[(third * TH + t) * 128 + rl], up = swi[(third * TH + t) * 128 + rl + 64];
                        const float sgn = gt < 0.0f ? -1.0f : 1.0f;
                        const float ex = __expf(-(sgn * gt));
                        const float th = sgn * ((1.0f - ex) / (1.0f + ex));
                        g.out[(size_t)(tok0 + t) * g.ld_out + mtf * 64 + rl] = gt * (0.5f * (1.0f + th)) * up;
                    }
                }
                asm volatile("bar.sync %0, 128;" :: "r"(bar_third) : "memory");
            } else if (row < g.rows && !dead) {
#pragma unroll
                for (int t = 0; t < TH; t++) {
                    if (t >= tleft) break;
                    const float v = val[t] * tsr;
                    g.out[(size_t)(tok0 + t) * g.ld_out + row] = g.resid ? prev[t] + v : v;
                }
            }
        };
        auto load_prev = [&](int mtf, float (&prev)[TH]) {      // residual linears: the old values of this row
            const int row = mtf * 128 + rl;
#pragma unroll
            for (int t = 0; t < TH; t++)
                prev[t] = (g.resid && !g.swiglu && t < tleft && row < g.rows) ? __ldcg(g.out + (size_t)(tok0 + t) * g.ld_out + row) : 0.0f;
        };
        // the ticket drawn for tile mtf said that its other pieces are done: add all pieces in K order and finish the tile.
        // Eight values per thread, the loads of four pieces in flight together.  SwiGLU tiles: thread (row r of 64, half of
        // the lanes' quarter pair) takes four tokens and fetches the gate row r and the up row r + 64 of each, so no
        // exchange between warps is needed.
        auto merge = [&](int mtf) {
            if (etid == 0 && !dead) g.tickets[mtf * G + grp] = 0u;
            const bool sw = g.swiglu != 0;
            const int r0 = sw ? (rl & 63) : rl, tb = sw ? (rl >> 6) * (TH / 2) : 0;
            const float* part = g.partial + ((size_t)mtf * P * ptok + tok0 + tb) * 128 + r0;      // [piece][token][row in tile]
            float val[TH], prev[TH];
            if (!sw) load_prev(mtf, prev);
#pragma unroll
            for (int i = 0; i < TH; i++) val[i] = 0.0f;
            for (int q0 = 0; q0 < P; q0 += 4) {
                float pv[4][TH];
#pragma unroll
                for (int qq = 0; qq < 4; qq++)
#pragma unroll
                    for (int i = 0; i < TH; i++) {
                        const int tt = sw ? tb + (i % (TH / 2)) : i;                            // token of value i
                        const int off = sw ? (i % (TH / 2)) * 128 + (i / (TH / 2)) * 64 : i * 128;   // its place from `part`
                        pv[qq][i] = (q0 + qq < P && tt < tleft) ? __ldcg(part + (size_t)(q0 + qq) * ptok * 128 + off) : 0.0f;
                    }
#pragma unroll
                for (int qq = 0; qq < 4; qq++)
                    if (q0 + qq < P) {
#pragma unroll
                        for (int i = 0; i < TH; i++) val[i] += pv[qq][i];
                    }
            }
            if (!sw) { finalize(mtf, val, prev); return; }
            if (mtf * 64 + r0 >= g.rows || dead) return;
#pragma unroll
            for (int i = 0; i < TH / 2; i++) {
                if (tb + i >= tleft) break;
                const float gt = val[i] * g.ts[0], up = val[i + TH / 2] * g.ts[1];
                const float sgn = gt < 0.0f ? -1.0f : 1.0f;
                const float ex = __expf(-(sgn * gt));
                const float th = sgn * ((1.0f - ex) / (1.0f + ex));
                g.out[(size_t)(tok0 + tb + i) * g.ld_out + mtf * 64 + r0] = gt * (0.5f * (1.0f + th)) * up;
            }
        };
        int unit_iter = 0, pend_mt = -1;
        for (int u = blockIdx.x; u < nunits; u += gridDim.x, unit_iter++) {
            TC_UNIT(u);
            (void)ks_lo; (void)ks_hi;
            const int row = mt * 128 + rl;
            const int ab = DG ? (unit_iter & 1) : 0;                                   // accumulator of this unit
            const uint32_t aph = DG ? (uint32_t)(unit_iter >> 1) & 1u : (uint32_t)unit_iter & 1u;
            float prev[TH];
            if (DG && P == 1) load_prev(mt, prev);      // fetched before the accumulator is ready
            if (etid == 0) TC_MARK(2, unit_iter, 0);
            if (dead || !mb_wait(&S.accum[ab], aph, &S.abort_flag)) dead = true;
            if (etid == 0) TC_MARK(2, unit_iter, 1);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tlane = tmem + ((uint32_t)(sub * 32) << 16);
            if (!DG) {
                for (int c0 = third * 8; c0 < NB && !dead; c0 += 8 * TC_EPI_Q) {
                    uint32_t r[8];
                    tc_ld8(r, tlane + (uint32_t)c0);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (row < g.rows) {
#pragma unroll
                        for (int j = 0; j < 8; j++) g.y[(size_t)row * NB + c0 + j] = __uint_as_float(r[j]);
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mb_arrive(&S.acc_free[0]);
                continue;
            }
            // ---- digit mode: this thread's row and eight tokens: ten digit accumulators each, most significant first,
            // folded by v = 9 v + D (two digits' loads in flight per wait)
            float val[TH];
            {
                const uint32_t tcol = tlane + (uint32_t)(ab * HX_TC_GROUP_COLS + third * TH);
                const bool any = !dead && tleft > 0;
#pragma unroll
                for (int t = 0; t < TH; t++) val[t] = 0.0f;
                uint32_t ra[8], rb[8];
#pragma unroll
                for (int d = 0; d < HX_TC_DIGITS; d += 2) {
                    if (any) {
                        tc_ld8(ra, tcol + (uint32_t)(d * HX_TC_MAX_TOK));
                        tc_ld8(rb, tcol + (uint32_t)((d + 1) * HX_TC_MAX_TOK));
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int t = 0; t < TH; t++) {
                            val[t] = fmaf(val[t], 9.0f, __uint_as_float(ra[t]));
                            val[t] = fmaf(val[t], 9.0f, __uint_as_float(rb[t]));
                        }
                    }
                }
#pragma unroll
                for (int t = 0; t < TH; t++) val[t] = (any && t < tleft) ? val[t] * cs[t] : 0.0f;
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mb_arrive(&S.acc_free[ab]);       // the issuer may overwrite this accumulator
            if (etid == 0) TC_MARK(2, unit_iter, 2);
            if (P == 1) { finalize(mt, val, prev); continue; }
            // K pieces: leave this piece's values, look at the ticket of the previous unit
            float* part = g.partial + (((size_t)mt * P + piece) * ptok + tok0) * 128 + rl;
#pragma unroll
            for (int t = 0; t < TH; t++)
                if (t < tleft && !dead) part[(size_t)t * 128] = val[t];
            // The previous unit's ticket has long arrived.  It is looked at BEFORE this warp reports its partial sums: the
            // ticket of this unit cannot be drawn without that report, so the ticket barrier is never two phases ahead of a
            // warp that still has to wait on it, and no warp reports twice before another has reported once.
            bool fin = false;
            if (pend_mt >= 0) {
                if (dead || !mb_wait(&S.tk_ready, (uint32_t)(unit_iter - 1) & 1u, &S.abort_flag)) dead = true;
                fin = !dead && S.ticket[(unit_iter - 1) & 1] == (unsigned)(P - 1);
            }
            __syncwarp();
            if (lane == 0) mb_arrive(&S.part_done);      // this warp's partial sums are written: the ticket may be drawn
            if (etid == 0) TC_MARK(2, unit_iter, 3);
            if (fin) merge(pend_mt);
            if (etid == 0) TC_MARK(2, unit_iter, 4 + (fin ? 1 : 0));
            pend_mt = mt;
        }
        if (pend_mt >= 0) {      // the last unit's ticket
            if (dead || !mb_wait(&S.tk_ready, (uint32_t)(unit_iter - 1) & 1u, &S.abort_flag)) dead = true;
            if (!dead && S.ticket[(unit_iter - 1) & 1] == (unsigned)(P - 1)) merge(pend_mt);
        }
    } else if (lane == 0 && P > 1) {
        // ------------------------------ tickets ------------------------------
        // One atomic per unit, after the epilogue warps have stored the unit's partial sums: the count of the (tile, group)'s
        // pieces that are done.  The release of the atomic waits for those stores, which is why no epilogue warp issues it.
        int unit_iter = 0;
        for (int u = blockIdx.x; u < nunits; u += gridDim.x, unit_iter++) {
            TC_UNIT(u);
            (void)piece; (void)ks_lo; (void)ks_hi;
            if (!mb_wait(&S.part_done, (uint32_t)unit_iter & 1u, &S.abort_flag)) break;
            unsigned old;
            asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(g.tickets + mt * G + grp) : "memory");
            S.ticket[unit_iter & 1] = old;
            mb_arrive(&S.tk_ready);
        }
    }
#undef TC_UNIT
    __syncthreads();
    if (S.abort_flag && tid == 0 && g.err) *g.err = 1;
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" :: "r"(tmem) : "memory");
    }
}

}  // namespace

// header, SwiGLU exchange and the slack of the 1024-byte alignment of the ring
#define TC_FRONT (((TC_HDR + TC_SWI + 1023u) & ~1023u) + 1024u)
size_t hx_gemm_tc_smem(int ncols, int stage_ksteps) {
    return TC_FRONT + (size_t)HX_TC_STAGES * (stage_ksteps / 4) * (HX_T128_CELL + (size_t)ncols * 128 + 2048);
}
// digit mode: ring of A cells + the digit cells of one (K piece, token group)
static size_t gemm_tc_smem_digits(int stage_ksteps, int cells_per_piece) {
    return TC_FRONT + (size_t)HX_TC_STAGES * (stage_ksteps / 4) * HX_T128_CELL + (size_t)cells_per_piece * TC_DIGIT_CELL;
}

// One-time function attribute (call outside any stream capture).
int hx_gemm_tc_prepare() {
    static std::atomic<unsigned long long> attr_seen{0};
    if (hx_first_on_device(attr_seen)) HX_CUDA(cudaFuncSetAttribute(k_gemm_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    return HX_OK;
}

int hx_gemm_tc_launch(const HxGemmTC& g, cudaStream_t st) {
    HX_CHECK_ARG(g.a && g.b && g.ntiles > 0 && g.ksteps > 0);
    HX_CHECK_ARG(g.stage_ksteps >= 4 && g.stage_ksteps <= HX_TC_MAX_SK && g.stage_ksteps % 4 == 0 && g.ksteps % 4 == 0);
    const int P = g.ksplit > 1 ? g.ksplit : 1, kc = g.ksteps / 4;
    size_t smem;
    int G = 1;
    if (g.digit_mode) {
        HX_CHECK_ARG(g.out && g.col_scale && g.b_resident && g.stage_ksteps == 4 && g.ntok >= 1 && g.ntok <= HX_TC_NTOK);
        HX_CHECK_ARG((kc + P - 1) / P <= HX_TC_RES_CELLS && P <= kc);
        if (P > 1) HX_CHECK_ARG(g.partial && g.tickets);
        G = (g.ntok + HX_TC_MAX_TOK - 1) / HX_TC_MAX_TOK;
        HX_CHECK_ARG(P * G <= 148);
        smem = gemm_tc_smem_digits(g.stage_ksteps, (kc + P - 1) / P);
    } else {
        HX_CHECK_ARG(g.y != nullptr && P == 1 && !g.b_resident);
        HX_CHECK_ARG(g.ncols >= 8 && g.ncols <= 256 && g.ncols % 8 == 0);
        smem = hx_gemm_tc_smem(g.ncols, g.stage_ksteps);
    }
    if (smem > 227 * 1024) return hx_fail(HX_ERR_ARG, "tensor-core GEMM stage too large (%zu bytes of shared memory)", smem);
    { const int prc = hx_gemm_tc_prepare(); if (prc) return prc; }
    int grid = g.ntiles * P * G; if (grid > 148) grid = g.digit_mode ? (148 / (P * G)) * (P * G) : 148;      // digit mode: a CTA keeps one (K piece, token group)
    k_gemm_tc<<<grid, TC_THREADS, smem, st>>>(g);
    HX_COUNT_LAUNCH(1);
    HX_CUDA(cudaGetLastError());
    return HX_OK;
}

// C-ABI entry for tests and tools: all pointers are device pointers.
HX_API int hx_gemm_nvfp4_tc(const uint8_t* a_t128, int rows, int K, const uint8_t* b_cells, int ncols, float* y,
                            int stage_ksteps, void* stream) {
    HX_CHECK_ARG(rows > 0 && K > 0 && K % 256 == 0);
    HxGemmTC g = {};
    g.a = a_t128; g.b = b_cells; g.y = y; g.rows = rows; g.ntiles = (rows + 127) / 128; g.ksteps = K / 64;
    g.ncols = ncols; g.stage_ksteps = stage_ksteps > 0 ? stage_ksteps : 4;
    int* derr = nullptr;
    HX_CUDA(cudaMalloc(&derr, 4));
    HX_CUDA(cudaMemsetAsync(derr, 0, 4, (cudaStream_t)stream));
    g.err = derr;
    int rc = hx_gemm_tc_launch(g, (cudaStream_t)stream);
    int e = 0;
    if (!rc) {
        cudaError_t ce = cudaStreamSynchronize((cudaStream_t)stream);
        if (ce != cudaSuccess) rc = hx_fail(HX_ERR_CUDA, "tensor-core GEMM: %s", cudaGetErrorString(ce));
        else { cudaMemcpy(&e, derr, 4, cudaMemcpyDeviceToHost); if (e) rc = hx_fail(HX_ERR_TIMEOUT, "tensor-core GEMM: a bounded wait ran out"); }
    }
    cudaFree(derr);
    return rc;
}

// Timing helper: `reps` back-to-back launches between two CUDA events (device pointers as above).
HX_API int hx_gemm_nvfp4_tc_bench(const uint8_t* a_t128, int rows, int K, const uint8_t* b_cells, int ncols, float* y,
                                  int stage_ksteps, int reps, float* ms_per_launch) {
    HX_CHECK_ARG(rows > 0 && K > 0 && K % 256 == 0 && reps > 0 && ms_per_launch);
    HxGemmTC g = {};
    g.a = a_t128; g.b = b_cells; g.y = y; g.rows = rows; g.ntiles = (rows + 127) / 128; g.ksteps = K / 64;
    g.ncols = ncols; g.stage_ksteps = stage_ksteps > 0 ? stage_ksteps : 4;
    int* derr = nullptr;
    HX_CUDA(cudaMalloc(&derr, 4));
    HX_CUDA(cudaMemset(derr, 0, 4));
    g.err = derr;
    cudaEvent_t e0, e1;
    HX_CUDA(cudaEventCreate(&e0)); HX_CUDA(cudaEventCreate(&e1));
    int rc = hx_gemm_tc_launch(g, nullptr);
    if (!rc) {
        cudaEventRecord(e0, nullptr);
        for (int i = 0; i < reps && !rc; i++) rc = hx_gemm_tc_launch(g, nullptr);
        cudaEventRecord(e1, nullptr);
        cudaError_t ce = cudaEventSynchronize(e1);
        if (ce != cudaSuccess) rc = hx_fail(HX_ERR_CUDA, "tensor-core GEMM: %s", cudaGetErrorString(ce));
        else { float t = 0; cudaEventElapsedTime(&t, e0, e1); *ms_per_launch = t / reps; }
    }
    int e = 0; cudaMemcpy(&e, derr, 4, cudaMemcpyDeviceToHost);
    if (!rc && e) rc = hx_fail(HX_ERR_TIMEOUT, "tensor-core GEMM: a bounded wait ran out");
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaFree(derr);
    return rc;
}
