// hx_gemm_tc.cu -- block-scaled NVFP4 GEMM on the 5th-generation tensor cores (tcgen05, TMEM).
//
//   D[row, n] = sum_k  A[row,k] * SFA[row,k/16]  *  B[n,k] * SFB[n,k/16]         (f32 accumulate in TMEM)
//
// A = weights, E2M1 codes with one UE4M3 scale per 16 elements along K: exactly the information of
// the committed NVFP4 layout (helixc/runtime/gpt2_pack.c:350-373), so the weights feed the tensor
// cores without any per-weight instruction.  B = activations as E2M1 columns with UE4M3 block scales:
// either the activation quantized once to NVFP4 (batched prefill, replaces tiled_matmul_abt of
// forward_layer_llama, helixc/runtime/gpt2_infer.c:1231-1287) or several exact base-8 digit columns
// of one f32 vector (decode, replaces fused_gemv :2281-2297).
//
// One CTA per 128-row tile of A.  Warp 0 streams A and B cells into a shared-memory ring with
// cp.async.bulk; warp 1 copies the scale factors to TMEM (tcgen05.cp) and issues
// tcgen05.mma.kind::mxf4nvf4.block_scale (M=128, N=ncols, K=64 per instruction); warps 2-5 read the
// accumulator with tcgen05.ld and store it.  Tensor-bound for large N, HBM-bound for small N.
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
    uint64_t full[HX_TC_STAGES], empty[HX_TC_STAGES], accum, bfull;
    uint32_t tmem_base;
    unsigned ticket;
    float swi[128];
    volatile int abort_flag;
};

__global__ void __launch_bounds__(192, 1) k_gemm_tc(const __grid_constant__ HxGemmTC g) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    TcSmem& S = *reinterpret_cast<TcSmem*>(smem_raw);
    // swizzled operands need 1024-byte aligned cells (the swizzle is a function of the shared-memory address)
    static_assert(sizeof(TcSmem) <= 1024, "header overlaps the unit-scale chunk");
    uint8_t* ring = smem_raw + (((s_u32(smem_raw) + 1536u + 1023u) & ~1023u) - s_u32(smem_raw));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NB = g.ncols, Sk = g.stage_ksteps;
    // a stage holds Sk K steps = Sk/4 cells of 256 columns
    const uint32_t b_cell_bytes = (uint32_t)NB * 128u + (g.digit_mode ? 0u : 2048u);       // one 256-column cell of B
    const uint32_t a_cell = HX_T128_CELL / 4, b_cell = b_cell_bytes / 4;                     // bytes per K step
    // b_resident: the B cells of this CTA's K piece stay in shared memory across its units (the ring holds A only)
    const int BR = g.b_resident;
    const uint32_t stage_bytes = (uint32_t)Sk * (a_cell + (BR ? 0u : b_cell));
    uint8_t* bres = ring + (size_t)HX_TC_STAGES * stage_bytes;      // [cells of a piece][NB * 128]

    if (tid < 128) reinterpret_cast<uint32_t*>(smem_raw + 1024)[tid] = 0x38383838u;      // a chunk of unit scales (digit mode)
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (tid == 0) {
        for (int i = 0; i < HX_TC_STAGES; i++) { mb_init(&S.full[i], 1); mb_init(&S.empty[i], 1); }
        mb_init(&S.accum, 1); mb_init(&S.bfull, 1);
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
    // TMEM columns: [0, 256) accumulator (ncols used), then per ring slot Sk*4 columns of SFA and of SFB
    const uint32_t col_sfa = 256, col_sfb = 256 + HX_TC_STAGES * HX_TC_MAX_SK * 4;

    // Work units: (128-row tile, K piece).  ksplit > 1 (digit mode only) cuts K into pieces of whole 256-column
    // cells; each piece recombines its own digits and the last piece of a tile to finish (ticket) adds the
    // pieces in K order and applies the epilogue.
    const int P = g.ksplit > 1 ? g.ksplit : 1, kcells = g.ksteps / 4;
    const int nunits = g.ntiles * P;
    uint32_t base_it = 0;                          // stage iterations of the units this CTA has finished
    uint32_t b_loads = 0; int cur_piece = -1;      // resident-B bookkeeping (same in every role)
    int unit_iter = 0;
    for (int u = blockIdx.x; u < nunits; u += gridDim.x, unit_iter++) {
        const int mt = u / P, piece = u - mt * P;
        const int ks_lo = (piece * kcells / P) * 4, ks_hi = ((piece + 1) * kcells / P) * 4;
        const int n_it = (ks_hi - ks_lo + Sk - 1) / Sk;
        int n_it_run = n_it;
        const bool new_b = BR && (unit_iter == 0 || piece != cur_piece);
        if (warp == 0 && lane == 0) {
            // ------------------------------ producer ------------------------------
            if (new_b) {        // every MMA of the previous unit has completed (its epilogue ran before the CTA barrier)
                const uint32_t bytes = (uint32_t)((ks_hi - ks_lo) / 4) * b_cell_bytes;
                mb_expect(&S.bfull, bytes);
                bulk_load(bres, g.b + (size_t)(ks_lo / 4) * b_cell_bytes, bytes, &S.bfull);
            }
            for (int it = 0; it < n_it; it++) {
                const uint32_t git = base_it + it, slot = git % HX_TC_STAGES, round = git / HX_TC_STAGES;
                if (round > 0 && !mb_wait(&S.empty[slot], (round - 1) & 1, &S.abort_flag)) break;
                const int ks0 = ks_lo + it * Sk, nk = min(Sk, ks_hi - ks0);
                uint8_t* sa = ring + (size_t)slot * stage_bytes;
                uint8_t* sb = sa + (size_t)Sk * a_cell;
                mb_expect(&S.full[slot], (uint32_t)nk * (a_cell + (BR ? 0u : b_cell)));
                bulk_load(sa, g.a + ((size_t)mt * g.ksteps + ks0) * a_cell, (uint32_t)nk * a_cell, &S.full[slot]);
                if (!BR) bulk_load(sb, g.b + (size_t)ks0 * b_cell, (uint32_t)nk * b_cell, &S.full[slot]);
            }
        } else if (warp == 1 && lane == 0) {
            // ------------------------------ MMA issuer ------------------------------
            // instruction descriptor: E2M1 x E2M1, UE4M3 scales, K-major both, N = NB, M = 128, K = 64
            const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) | (8u << 24);
            if (g.digit_mode && unit_iter == 0) {
                // unit scales (E4M3 1.0) for every digit column: sixteen TMEM columns cover any N up to 256
                for (int c = 0; c < 4; c++) tc_cp_sf(tmem + col_sfb + c * 4, smem_desc(s_u32(smem_raw + 1024), 16, 128));
            }
            if (new_b) { if (!mb_wait(&S.bfull, b_loads & 1u, &S.abort_flag)) n_it_run = 0; }
            for (int it = 0; it < n_it_run; it++) {
                const uint32_t git = base_it + it, slot = git % HX_TC_STAGES, round = git / HX_TC_STAGES;
                if (!mb_wait(&S.full[slot], round & 1, &S.abort_flag)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int ks0 = ks_lo + it * Sk, nk = min(Sk, ks_hi - ks0);
                const uint32_t sa = s_u32(ring + (size_t)slot * stage_bytes);
                const uint32_t sb = BR ? s_u32(bres) + (uint32_t)(it * (Sk / 4)) * b_cell_bytes : sa + (uint32_t)Sk * a_cell;
                for (int rep = 0; rep < ((g.dbg & 8) ? 4 : 1); rep++)
                for (int k = 0; k < nk; k++) {
                    const uint32_t ta = tmem + col_sfa + (slot * HX_TC_MAX_SK + k) * 4;
                    const uint32_t tb = tmem + col_sfb + (slot * HX_TC_MAX_SK + k) * 4;
                    const uint32_t acell = sa + (uint32_t)(k >> 2) * HX_T128_CELL, bcell = sb + (uint32_t)(k >> 2) * b_cell_bytes;
                    const uint32_t e = (uint32_t)(k & 3);
                    if (!(g.dbg & 1) || (it == 0 && k == 0)) {
                        tc_cp_sf(ta, smem_desc(acell + 16384 + e * 512, 16, 128));
                        if (!g.digit_mode) tc_cp_sf(tb, smem_desc(bcell + (uint32_t)NB * 128u + e * 512, 16, 128));
                    }
                    tc_mma(tmem + ((g.dbg & 4) ? (uint32_t)(k & 3) * 64u : 0u), smem_desc(acell + e * 32, 16, 1024, SW128), smem_desc(bcell + e * 32, 16, 1024, SW128), idesc,
                           (g.dbg & 2) ? tmem + col_sfa : ta, ((g.dbg & 2) || g.digit_mode) ? tmem + col_sfb : tb, (it > 0 || k > 0) ? 1u : 0u);
                }
                tc_commit(&S.empty[slot]);          // the slot is free once these MMAs have read it
            }
            tc_commit(&S.accum);                    // accumulator complete
        } else if (warp >= 2) {
            // ------------------------------ epilogue: TMEM -> registers -> global ------------------------------
            if (mb_wait(&S.accum, (uint32_t)unit_iter & 1u, &S.abort_flag)) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int sub = warp & 3;                          // TMEM lanes 32*sub .. 32*sub+31
                const int rl = sub * 32 + lane, row = mt * 128 + rl;
                if (g.digit_mode) {
                    const int ntok = NB / 16;
                    const float tsr = g.pair64 ? (((row & 127) < 64) ? g.ts[0] : g.ts[1])
                                               : (row < g.bound0 ? g.ts[0] : (row < g.bound1 ? g.ts[1] : g.ts[2]));
                    // final value of (token t, this row): tensor scale, then store / residual add / SwiGLU across the
                    // gate (rows 0..63 of the tile) and up (rows 64..127) halves
                    // residual linears: the old values of this row for every token are fetched up front, all loads in
                    // flight together (one dependent round trip per token was most of a short GEMM's time)
                    float prev[HX_TC_MAX_TOK];
#pragma unroll
                    for (int t = 0; t < HX_TC_MAX_TOK; t++)
                        prev[t] = (g.resid && !g.swiglu && t < ntok && row < g.rows) ? __ldcg(g.out + (size_t)t * g.ld_out + row) : 0.0f;
                    auto finalize = [&](int t, float v, float old) {
                        v *= tsr;
                        if (g.swiglu) {
                            S.swi[rl] = v;
                            asm volatile("bar.sync 1, 128;" ::: "memory");
                            if (rl < 64 && mt * 64 + rl < g.rows) {
                                const float gt = S.swi[rl], up = S.swi[rl + 64];
                                const float sgn = gt < 0.0f ? -1.0f : 1.0f;
                                const float ex = __expf(-(sgn * gt));
                                const float th = sgn * ((1.0f - ex) / (1.0f + ex));
                                g.out[(size_t)t * g.ld_out + mt * 64 + rl] = gt * (0.5f * (1.0f + th)) * up;
                            }
                            asm volatile("bar.sync 1, 128;" ::: "memory");
                        } else if (row < g.rows) {
                            g.out[(size_t)t * g.ld_out + row] = g.resid ? old + v : v;
                        }
                    };
                    // the tokens' digit scales, fetched once (a load per token between the stores below would be a dependent
                    // round trip each)
                    float cs[HX_TC_MAX_TOK];
#pragma unroll
                    for (int t = 0; t < HX_TC_MAX_TOK; t++) cs[t] = t < ntok ? __ldg(g.col_scale + t) : 0.0f;
                    float* part = g.partial + ((size_t)(mt * P) * HX_TC_MAX_TOK) * 128;      // [piece][token][row in tile]
#pragma unroll
                    for (int t = 0; t < HX_TC_MAX_TOK; t++) {
                        if (t >= ntok) break;
                        uint32_t r[16];
                        const uint32_t ta = tmem + ((uint32_t)(sub * 32) << 16) + (uint32_t)(t * 16);
                        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                                       "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                                     : "r"(ta));
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        float v = 0.0f;
#pragma unroll
                        for (int j = 15; j >= 0; j--) v = fmaf(v, 0.25f, __uint_as_float(r[j]));
                        v = v * cs[t];
                        if (P > 1) part[((size_t)piece * HX_TC_MAX_TOK + t) * 128 + rl] = v;
                        else finalize(t, v, prev[t]);
                    }
                    if (P > 1) {
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (tid == 64) {
                            unsigned old;
                            asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(g.tickets + mt) : "memory");
                            S.ticket = old;
                        }
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (S.ticket == (unsigned)(P - 1)) {
                            // the pieces of all tokens: sixteen loads in flight per piece, added in piece order per token
                            float sum[HX_TC_MAX_TOK];
#pragma unroll
                            for (int t = 0; t < HX_TC_MAX_TOK; t++) sum[t] = 0.0f;
                            for (int q = 0; q < P; q++) {
#pragma unroll
                                for (int t = 0; t < HX_TC_MAX_TOK; t++)
                                    if (t < ntok) sum[t] += __ldcg(part + ((size_t)q * HX_TC_MAX_TOK + t) * 128 + rl);
                            }
#pragma unroll
                            for (int t = 0; t < HX_TC_MAX_TOK; t++) if (t < ntok) finalize(t, sum[t], prev[t]);
                            if (tid == 64) g.tickets[mt] = 0u;
                        }
                    }
                } else
                for (int c0 = 0; c0 < NB; c0 += 8) {
                    uint32_t r[8];
                    const uint32_t ta = tmem + ((uint32_t)(sub * 32) << 16) + (uint32_t)c0;
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(ta));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (row < g.rows) {
#pragma unroll
                        for (int j = 0; j < 8; j++) g.y[(size_t)row * NB + c0 + j] = __uint_as_float(r[j]);
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
        }
        base_it += (uint32_t)n_it;
        if (new_b) { b_loads++; cur_piece = piece; }
        // all roles meet before the next unit (the accumulator is reused)
        __syncthreads();
    }
    if (S.abort_flag && tid == 0 && g.err) *g.err = 1;
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" :: "r"(tmem) : "memory");
}

}  // namespace

size_t hx_gemm_tc_smem(int ncols, int stage_ksteps) {
    return 4096 + (size_t)HX_TC_STAGES * (stage_ksteps / 4) * (HX_T128_CELL + (size_t)ncols * 128 + 2048);
}
// resident-B variant: ring of A cells + the B cells of one K piece
static size_t gemm_tc_smem_resident(int ncols, int stage_ksteps, int cells_per_piece) {
    return 4096 + (size_t)HX_TC_STAGES * (stage_ksteps / 4) * HX_T128_CELL + (size_t)cells_per_piece * ncols * 128;
}

// One-time function attribute (call outside any stream capture).
int hx_gemm_tc_prepare() {
    static std::atomic<unsigned long long> attr_seen{0};
    if (hx_first_on_device(attr_seen)) HX_CUDA(cudaFuncSetAttribute(k_gemm_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    return HX_OK;
}

int hx_gemm_tc_launch(const HxGemmTC& g, cudaStream_t st) {
    HX_CHECK_ARG(g.a && g.b && (g.digit_mode ? (g.out && g.col_scale && g.ncols % 16 == 0) : g.y != nullptr) && g.ntiles > 0 && g.ksteps > 0);
    HX_CHECK_ARG(g.ncols >= 8 && g.ncols <= 256 && g.ncols % 8 == 0);
    HX_CHECK_ARG(g.stage_ksteps >= 4 && g.stage_ksteps <= HX_TC_MAX_SK && g.stage_ksteps % 4 == 0 && g.ksteps % 4 == 0);
    const int Pq = g.ksplit > 1 ? g.ksplit : 1, kc = g.ksteps / 4;
    if (g.b_resident) HX_CHECK_ARG(g.digit_mode && g.stage_ksteps == 4);
    const size_t smem = g.b_resident ? gemm_tc_smem_resident(g.ncols, g.stage_ksteps, (kc + Pq - 1) / Pq) : hx_gemm_tc_smem(g.ncols, g.stage_ksteps);
    if (smem > 227 * 1024) return hx_fail(HX_ERR_ARG, "tensor-core GEMM stage too large (%zu bytes of shared memory)", smem);
    { const int prc = hx_gemm_tc_prepare(); if (prc) return prc; }
    const int P = g.ksplit > 1 ? g.ksplit : 1;
    if (P > 1) HX_CHECK_ARG(g.digit_mode && g.partial && g.tickets && P <= g.ksteps / 4 && g.ncols / 16 <= HX_TC_MAX_TOK);
    int grid = g.ntiles * P; if (grid > 148) grid = g.b_resident ? (148 / P) * P : 148;      // resident B: a CTA keeps one K piece
    k_gemm_tc<<<grid, 192, smem, st>>>(g);
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
    { const char* d = getenv("HX_TC_DBG"); g.dbg = d ? atoi(d) : 0; }
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
