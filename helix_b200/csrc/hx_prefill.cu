// hx_prefill.cu -- batched prefill around the tcgen05 GEMM.
//
// Replaces forward_layer_llama / forward_full (helixc/runtime/gpt2_infer.c:1231-1333): where the reference runs
// f32 tiled_matmul_abt over a dequantized weight copy per layer, a chunk of HX_PF_TB prompt tokens here is one
// block-scaled NVFP4 GEMM per linear with the weights read in their packed form.  The activations enter the FP4
// tensor path as digits: after the optional RMSNorm each element is x = s * sum_d digit_d 9^(9-d) with ten balanced
// base-9 digits (-4 .. 4: E2M1 values, sign included) of the integer |x| / S * 2^29 (S: the power of two at or below
// the vector's largest element, s = S * 2^-29), every digit row being an E2M1 column with unit block scale; the GEMM
// epilogue folds the ten accumulators of a token.  The digits resolve 2^-29 of the vector's largest element, beyond
// what an f32 dot product keeps.  (The decode kernel uses sixteen exact base-4 digits: there the column count is free.)
// Norm, RoPE, KV append and attention are small f32 kernels over the chunk.
#include "hx_prefill.cuh"
#include "hx_gemm_tc.cuh"
#include "hx_kernels.cuh"
#include <math.h>
#include <atomic>

namespace {

__device__ __forceinline__ float pf_silu_mul(float g, float u) {      // same formula as the decode epilogue (silu_mul_k)
    const float sgn = g < 0.0f ? -1.0f : 1.0f;
    const float e = __expf(-(sgn * g));
    const float th = sgn * ((1.0f - e) / (1.0f + e));
    return g * (0.5f * (1.0f + th)) * u;
}

__global__ void __launch_bounds__(256) k_pf_embed(const int* __restrict__ ids, HxPfWhere wh, const float* __restrict__ emb, float* __restrict__ X, int DM) {
    const float4* src = reinterpret_cast<const float4*>(emb + (size_t)ids[wh.pos_arr ? (int)blockIdx.x : *wh.posp + (int)blockIdx.x] * DM);
    float4* dst = reinterpret_cast<float4*>(X + (size_t)blockIdx.x * DM);
    for (int i = threadIdx.x; i < DM / 4; i += blockDim.x) dst[i] = src[i];
}

// grid (token, slice of K): every CTA of a token computes the token's statistics, then emits its slice of items.
// A value becomes the integer M = round(|x| / S * 2^29) < 2^30 (S: the power of two at or below the vector's largest
// element) and that integer ten balanced base-9 digits (-4 .. 4), least significant first: r = M mod 9, M = M div 9,
// and a remainder above 4 becomes r - 9 with a carry.  A negative value has all its digits negated.  Digit d (d = 0:
// weight 9^9) of token t lies in row 24 d + t % 24 of the token group t / 24 of a cell, as the E2M1 code of its value.
__global__ void __launch_bounds__(512) k_pf_digits(const float* __restrict__ src, int ld, int K, int swiglu, const float* __restrict__ g,
                                                    float eps, uint8_t* __restrict__ cells, int groups, float* __restrict__ scale) {
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = src + (size_t)t * ld;
    __shared__ float red[32];
    auto value = [&](int k) -> float {        // element k of the vector before the norm scale (gain applied)
        float v;
        if (swiglu) { const int tile = k >> 6, r = k & 63; v = pf_silu_mul(x[tile * 128 + r], x[tile * 128 + 64 + r]); }
        else v = x[k];
        return v;
    };
    // pass 1: sum of squares (of x) and largest |x * g|
    float ss = 0.0f, mx = 0.0f;
    for (int k = tid; k < K; k += 512) {
        const float v = value(k);
        ss = fmaf(v, v, ss);
        mx = fmaxf(mx, fabsf(g ? v * g[k] : v));
    }
    ss = hx_warp_sum(ss); mx = hx_warp_max(mx);
    if (lane == 0) { red[warp] = ss; red[16 + warp] = mx; }
    __syncthreads();
    float tss = 0.0f, tmx = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i++) { tss += red[i]; tmx = fmaxf(tmx, red[16 + i]); }
    const float inv = g ? rsqrtf(tss / (float)K + eps) : 1.0f;
    float Sg = 1.0f;
    const float vmax = tmx * inv * 1.0000005f;
    if (vmax > 0.0f && vmax < INFINITY) Sg = __uint_as_float(__float_as_uint(vmax) & 0x7F800000u);
    if (tid == 0 && blockIdx.y == 0) scale[t] = Sg * (1.0f / HX_TC_DIGIT_UNIT);
    const float mul = (inv / Sg) * HX_TC_DIGIT_UNIT;
    // pass 2: items of 8 consecutive elements -> one word per digit
    const int Kc = ((K + 255) / 256) * 256;
    const size_t cell_bytes = (size_t)groups * (HX_TC_GROUP_COLS * 128);
    const int tg = t / HX_TC_MAX_TOK, tl = t - tg * HX_TC_MAX_TOK;
    const int nit = Kc / 8, per = (nit + gridDim.y - 1) / gridDim.y;
    const int it_hi = min(nit, (int)(blockIdx.y + 1) * per);
    for (int it = blockIdx.y * per + tid; it < it_hi; it += 512) {
        const int k = it * 8;
        uint32_t word[HX_TC_DIGITS];
#pragma unroll
        for (int n = 0; n < HX_TC_DIGITS; n++) word[n] = 0u;
#pragma unroll
        for (int e = 0; e < 8; e++) {
            float v = 0.0f;
            if (k + e < K) { v = value(k + e); if (g) v *= g[k + e]; }
            uint32_t m = __float2uint_rn(fabsf(v) * mul);
            const uint32_t neg = v < 0.0f ? 8u : 0u;
#pragma unroll
            for (int n = HX_TC_DIGITS - 1; n >= 0; n--) {
                const uint32_t q = __umulhi(m, 0x38E38E39u) >> 1;      // m / 9
                uint32_t r = m - 9u * q;                                // 0 .. 8
                const bool up = r > 4u;                                 // balanced: 5 .. 8 are -4 .. -1 of the next power
                m = q + (up ? 1u : 0u);
                const uint32_t mag = up ? 9u - r : r;                   // 0 .. 4
                const uint32_t code = (0x65420u >> (4u * mag)) & 0xFu;  // E2M1 codes of 0, 1, 2, 3, 4
                const uint32_t sgn = (mag != 0u && (up != (neg != 0u))) ? 8u : 0u;
                word[n] |= (code | sgn) << (4 * e);
            }
        }
        const int j = (it >> 2) & 7, w = it & 3;
        uint8_t* dst = cells + (size_t)(it >> 5) * cell_bytes + (size_t)tg * (HX_TC_GROUP_COLS * 128) + w * 4;
#pragma unroll
        for (int n = 0; n < HX_TC_DIGITS; n++) {
            const int row = n * HX_TC_MAX_TOK + tl;
            *reinterpret_cast<uint32_t*>(dst + (size_t)row * 128 + ((j ^ (row & 7)) << 4)) = word[n];
        }
    }
}

// grid (NH + 2 NKV, n_tok), block DH threads (DH <= 256)
__global__ void __launch_bounds__(256) k_pf_qkpost(float* __restrict__ qkv, int ld, HxPfWhere wh, int NH, int NKV, int DH,
                                                    const float* __restrict__ qn_g, const float* __restrict__ kn_g, float eps,
                                                    const float* __restrict__ cosT, const float* __restrict__ sinT,
                                                    float* __restrict__ kc, float* __restrict__ vc, int cap) {
    const int hs = blockIdx.x, t = blockIdx.y, e = threadIdx.x, half = DH >> 1, pos = wh.pos_arr ? wh.pos_arr[t] : *wh.posp + t;
    const size_t seq_off = wh.seq_arr ? (size_t)wh.seq_arr[t] * wh.seq_stride : (wh.seqp ? (size_t)(*wh.seqp) * wh.seq_stride : 0);
    const int sec = hs < NH ? 0 : (hs < NH + NKV ? 1 : 2);
    float* row = qkv + (size_t)t * ld + (size_t)hs * DH;
    __shared__ float sm[256]; __shared__ float red[8];
    float v = e < DH ? row[e] : 0.0f;
    const float* gg = sec == 0 ? qn_g : (sec == 1 ? kn_g : nullptr);
    float ssq = hx_warp_sum(v * v);
    if ((e & 31) == 0) red[e >> 5] = ssq;
    __syncthreads();
    ssq = 0.0f;
    for (int i = 0; i < (DH + 31) / 32; i++) ssq += red[i];
    if (gg) v = gg[e] * (v * rsqrtf(ssq / (float)DH + eps));
    if (cosT && sec < 2) {
        sm[e] = v;
        __syncthreads();
        const float other = sm[e < half ? e + half : e - half];
        const float cs = cosT[(size_t)pos * half + (e < half ? e : e - half)], sn = sinT[(size_t)pos * half + (e < half ? e : e - half)];
        v = e < half ? v * cs - other * sn : v * cs + other * sn;
    }
    if (e < DH) {
        if (sec == 0) row[e] = v;
        else {
            const int kvh = hs - NH - (sec == 2 ? NKV : 0);
            (sec == 1 ? kc : vc)[seq_off + ((size_t)kvh * cap + pos) * DH + e] = v;
        }
    }
}

// ---- causal attention of a chunk over the cache ------------------------------------------------------------------
// grid (NKV, groups of TG tokens, NS), PF_AT threads: CTA (kv head, token group, s) covers the s-th run of whole key
// tiles of the group's context (NS runs at most, fewer for a short context; CTAs without a run leave at once).
// The K and V rows of a tile are contiguous in the cache, so one thread brings each tile into a ring of PF_ST
// shared-memory stages with two bulk copies (cp.async.bulk, completion on an mbarrier), PF_ST - 1 tiles ahead of the
// arithmetic: the loads of a CTA never wait for its softmax.  In a prefill chunk (one sequence, consecutive positions)
// the TG = 4 tokens of a group share every tile; in batched decode every token has a cache of its own (TG = 1).
// Per token: online softmax over the tiles (m seeded -1e8 like fused_decode_attn_kernel.hx:74-102).  Scores: a warp
// takes four keys at a time against every (token, head) query, the 4 x GRP dot products of a token are reduced across
// the lanes together (each exchange halves the values a lane carries).  Softmax step: a warp per (token, head).
// P*V: thread (dimension, run of keys inside the tile), a V value serving all tokens and heads; the runs are added
// up through shared memory at the end.  With more than one active run per (token group, kv head) each CTA leaves (sum, m, l) in
// `part`, and the last one to finish (a ticket per (token group, kv head)) merges them.  Waits are bounded: after a
// wait that ran out the CTA keeps to its barriers, writes nothing and raises *err.
#define PF_AT 512
#define PF_ST 3
#define PF_NS_MAX 16
#define PF_TILE_BYTES 32768          // K rows of a tile (and as many V rows)
#define PF_AT_WAIT (1u << 22)
__device__ __forceinline__ uint32_t pf_s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool pf_mb_wait(uint64_t* b, uint32_t parity) {
    for (uint32_t i = 0; i < PF_AT_WAIT; i++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(pf_s32(b)), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
template <int GRP, int TG>
__global__ void __launch_bounds__(PF_AT) k_pf_attn(const float* __restrict__ qkv, int ld, HxPfWhere wh, int n_tok, int NH, int DH,
                                                    const float* __restrict__ kc, const float* __restrict__ vc, int cap, float scale,
                                                    float* __restrict__ ctx, int ld_ctx, float* __restrict__ part, unsigned* __restrict__ tickets, int* err) {
    extern __shared__ __align__(128) float smf[];
    const int kvh = blockIdx.x, t0 = blockIdx.y * TG, s = blockIdx.z, NS = gridDim.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NW = PF_AT / 32;
    constexpr int GP = GRP <= 1 ? 1 : (GRP <= 2 ? 2 : (GRP <= 4 ? 4 : 8));      // GRP rounded up to a power of two
    constexpr int NP = 4 * GP;                                                   // values reduced together (4 keys x GP heads)
    constexpr int LG = NP == 4 ? 2 : (NP == 8 ? 3 : (NP == 16 ? 4 : 5));
    const int KT = min(128, PF_TILE_BYTES / (DH * 4));                           // keys per tile (32 .. 128, a multiple of 32)
    const int ntk = min(TG, n_tok - t0);                                         // tokens of this group
    const int pos0 = wh.pos_arr ? wh.pos_arr[t0] : *wh.posp + t0;                // TG > 1 only with consecutive positions
    const int Tmax = pos0 + ntk;                                                 // context of the group's last token
    const int tiles = (Tmax + KT - 1) / KT, per = ((tiles + NS - 1) / NS) * KT;  // keys per run: whole tiles
    const int n_act = (Tmax + per - 1) / per;
    if (s >= n_act) return;
    const int j_lo = s * per, j_hi = min(Tmax, j_lo + per);
    const size_t seq_off = wh.seq_arr ? (size_t)wh.seq_arr[t0] * wh.seq_stride : (wh.seqp ? (size_t)(*wh.seqp) * wh.seq_stride : 0);
    // shared memory: ring [PF_ST][K tile | V tile], then q, p and the P*V partial outputs
    float* ringf = smf;
    const int stage_f = 2 * (PF_TILE_BYTES / 4);
    float* sq = smf + PF_ST * stage_f;         // [TG][GRP][DH]
    float* sp = sq + TG * GRP * DH;            // [TG][GRP][128]
    float* sacc = sp + TG * GRP * 128;              // [nsub][GRP][DH] partial outputs of the key runs inside a tile
    __shared__ float sm_m[TG][GRP], sm_l[TG][GRP], sm_r[TG][GRP];
    __shared__ unsigned sm_ticket;
    __shared__ int sm_abort;
    __shared__ __align__(8) uint64_t full[PF_ST];
    for (int i = tid; i < ntk * GRP * DH; i += PF_AT) {
        const int tk = i / (GRP * DH), r = i - tk * GRP * DH;
        sq[i] = qkv[(size_t)(t0 + tk) * ld + (size_t)kvh * GRP * DH + r];
    }
    if (tid < TG * GRP) { sm_m[tid / GRP][tid % GRP] = -100000000.0f; sm_l[tid / GRP][tid % GRP] = 0.0f; }
    if (tid == 0) {
        sm_abort = 0;
        for (int i = 0; i < PF_ST; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(pf_s32(&full[i])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const float* kbase = kc + seq_off + (size_t)kvh * cap * DH;
    const float* vbase = vc + seq_off + (size_t)kvh * cap * DH;
    const int ntile = (j_hi - j_lo + KT - 1) / KT;
    auto issue = [&](int it) {       // thread 0: tile `it` of this run into its stage
        const int j0 = j_lo + it * KT, nj = min(KT, j_hi - j0);
        const uint32_t bytes = (uint32_t)nj * DH * 4;
        float* st = ringf + (size_t)(it % PF_ST) * stage_f;
        uint64_t* bar = &full[it % PF_ST];
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(pf_s32(bar)), "r"(2 * bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     :: "r"(pf_s32(st)), "l"(kbase + (size_t)j0 * DH), "r"(bytes), "r"(pf_s32(bar)) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     :: "r"(pf_s32(st + PF_TILE_BYTES / 4)), "l"(vbase + (size_t)j0 * DH), "r"(bytes), "r"(pf_s32(bar)) : "memory");
    };
    if (tid == 0) for (int it = 0; it < PF_ST - 1 && it < ntile; it++) issue(it);
    const int nsub = PF_AT / DH, d = tid % DH, ksub = tid / DH;      // DH divides PF_AT (32, 64, 128, 256)
    const int krun = KT / nsub;                                      // keys of a tile per P*V thread: a multiple of 4
    float acc[TG][GRP];
#pragma unroll
    for (int tk = 0; tk < TG; tk++)
#pragma unroll
        for (int i = 0; i < GRP; i++) acc[tk][i] = 0.0f;
    // Batched decode at head_dim 128 (tiles of 64 keys): a leaner arrangement of the same arithmetic.  Scores: thread (key,
    // eighth of the row) with its slice of q in registers (groups of up to four heads) -- chunk c * 8 + eighth of the row, so that the eight lanes of a
    // key read eight different bank groups -- and three exchanges per head.  P*V: a warp per four keys, a lane per
    // float4 of the row; the sixteen warps' sums are added up through the (then idle) ring at the end.
    constexpr bool kLean = TG == 1;
    constexpr bool kQreg = GRP <= 4;       // larger groups read q from shared memory (eight lanes, one 128-byte row: a broadcast)
    const bool lean = kLean && DH == 128;
    float acc4[kLean ? GRP : 1][4];
#pragma unroll
    for (int i = 0; i < (kLean ? GRP : 1); i++) acc4[i][0] = acc4[i][1] = acc4[i][2] = acc4[i][3] = 0.0f;
    if (lean) {
        const int key = tid >> 3, pt = tid & 7;
        float4 qr[(kLean && kQreg) ? GRP : 1][4];
#pragma unroll
        for (int i = 0; i < ((kLean && kQreg) ? GRP : 1); i++)
#pragma unroll
            for (int c = 0; c < 4; c++) qr[i][c] = *reinterpret_cast<const float4*>(sq + i * 128 + (c * 8 + pt) * 4);
        for (int it = 0; it < ntile; it++) {
            const int j0 = j_lo + it * 64, nj = min(64, j_hi - j0);
            if (tid == 0 && it + PF_ST - 1 < ntile) issue(it + PF_ST - 1);
            if (!pf_mb_wait(&full[it % PF_ST], (uint32_t)(it / PF_ST) & 1u)) sm_abort = 1;
            const float* kt = ringf + (size_t)(it % PF_ST) * stage_f;
            const float* vt = kt + PF_TILE_BYTES / 4;
            {
                float4 k4[4];
#pragma unroll
                for (int c = 0; c < 4; c++) k4[c] = *reinterpret_cast<const float4*>(kt + key * 128 + (c * 8 + pt) * 4);
                float dot[kLean ? GRP : 1];
#pragma unroll
                for (int i = 0; i < (kLean ? GRP : 1); i++) {
                    float a = 0.0f;
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const float4 q4 = kQreg ? qr[kQreg ? i : 0][c] : *reinterpret_cast<const float4*>(sq + i * 128 + (c * 8 + pt) * 4);
                        a = fmaf(q4.x, k4[c].x, a); a = fmaf(q4.y, k4[c].y, a); a = fmaf(q4.z, k4[c].z, a); a = fmaf(q4.w, k4[c].w, a);
                    }
                    a += __shfl_xor_sync(0xffffffffu, a, 1); a += __shfl_xor_sync(0xffffffffu, a, 2); a += __shfl_xor_sync(0xffffffffu, a, 4);
                    dot[i] = a;
                }
#pragma unroll
                for (int i = 0; i < (kLean ? GRP : 1); i++)
                    if (pt == i && key < nj) sp[i * 128 + key] = dot[i] * scale;
            }
            __syncthreads();
            for (int i = warp; i < GRP; i += NW) {
                const float s0 = lane < nj ? sp[i * 128 + lane] : -INFINITY, s1 = lane + 32 < nj ? sp[i * 128 + lane + 32] : -INFINITY;
                const float tm = hx_warp_max(fmaxf(s0, s1));
                const float mo = sm_m[0][i], mn = fmaxf(mo, tm);
                const float p0 = lane < nj ? __expf(s0 - mn) : 0.0f, p1 = lane + 32 < nj ? __expf(s1 - mn) : 0.0f;
                sp[i * 128 + lane] = p0; sp[i * 128 + lane + 32] = p1;
                const float ls = hx_warp_sum(p0 + p1);
                if (lane == 0) { const float rr = __expf(mo - mn); sm_r[0][i] = rr; sm_l[0][i] = sm_l[0][i] * rr + ls; sm_m[0][i] = mn; }
            }
            __syncthreads();
            {
                float4 p4[kLean ? GRP : 1];
#pragma unroll
                for (int i = 0; i < (kLean ? GRP : 1); i++) {
                    const float rr = sm_r[0][i];
                    acc4[i][0] *= rr; acc4[i][1] *= rr; acc4[i][2] *= rr; acc4[i][3] *= rr;
                    p4[i] = *reinterpret_cast<const float4*>(sp + i * 128 + warp * 4);
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int j = warp * 4 + u;
                    const float4 v4 = j < nj ? *reinterpret_cast<const float4*>(vt + j * 128 + lane * 4) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                    for (int i = 0; i < (kLean ? GRP : 1); i++) {
                        const float pj = u == 0 ? p4[i].x : (u == 1 ? p4[i].y : (u == 2 ? p4[i].z : p4[i].w));
                        acc4[i][0] = fmaf(pj, v4.x, acc4[i][0]); acc4[i][1] = fmaf(pj, v4.y, acc4[i][1]);
                        acc4[i][2] = fmaf(pj, v4.z, acc4[i][2]); acc4[i][3] = fmaf(pj, v4.w, acc4[i][3]);
                    }
                }
            }
            __syncthreads();
        }
    } else
    for (int it = 0; it < ntile; it++) {
        const int j0 = j_lo + it * KT, njt = min(KT, j_hi - j0);
        // every thread is past tile it - 1 (the barrier that ended it), so its stage may be refilled
        if (tid == 0 && it + PF_ST - 1 < ntile) issue(it + PF_ST - 1);
        if (!pf_mb_wait(&full[it % PF_ST], (uint32_t)(it / PF_ST) & 1u)) sm_abort = 1;
        const float* kt = ringf + (size_t)(it % PF_ST) * stage_f;
        const float* vt = kt + PF_TILE_BYTES / 4;
        const int njm = min(njt, pos0 + ntk - j0);          // keys of the tile the group's last token may see (> 0)
        // ---- scores of all tokens: a warp takes four keys at a time against every (token, head) query
        for (int jb = warp; jb < njm; jb += 4 * NW) {
            float v[TG][NP];
#pragma unroll
            for (int tk = 0; tk < TG; tk++)
#pragma unroll
                for (int i = 0; i < NP; i++) v[tk][i] = 0.0f;
            for (int e = lane * 4; e < DH; e += 128) {
                float4 k4[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int j = jb + u * NW;
                    k4[u] = j < njm ? *reinterpret_cast<const float4*>(kt + (size_t)j * DH + e) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
#pragma unroll
                for (int tk = 0; tk < TG; tk++) {
                    if (tk >= ntk) break;
#pragma unroll
                    for (int i = 0; i < GRP; i++) {
                        const float4 q4 = *reinterpret_cast<const float4*>(sq + (tk * GRP + i) * DH + e);
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            float a = v[tk][u * GP + i];
                            a = fmaf(q4.x, k4[u].x, a); a = fmaf(q4.y, k4[u].y, a); a = fmaf(q4.z, k4[u].z, a); a = fmaf(q4.w, k4[u].w, a);
                            v[tk][u * GP + i] = a;
                        }
                    }
                }
            }
#pragma unroll
            for (int tk = 0; tk < TG; tk++) {
                if (tk >= ntk) break;
                // lanes with the exchange bit set keep the upper half of the values, the others the lower half
#pragma unroll
                for (int st = 0; st < 5; st++) {
                    const int o = 16 >> st;
                    if (st < LG) {
                        const int h = NP >> (st + 1);
                        const bool up = (lane & o) != 0;
#pragma unroll
                        for (int k = 0; k < h; k++) {
                            const float send = up ? v[tk][k] : v[tk][k + h], keep = up ? v[tk][k + h] : v[tk][k];
                            v[tk][k] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                        }
                    } else v[tk][0] += __shfl_xor_sync(0xffffffffu, v[tk][0], o);
                }
                const int idx = lane >> (5 - LG), u = idx / GP, i = idx - u * GP, j = jb + u * NW;
                if ((lane & ((1 << (5 - LG)) - 1)) == 0 && i < GRP && j < njm) sp[(tk * GRP + i) * 128 + j] = v[tk][0] * scale;
            }
        }
        __syncthreads();
        // ---- softmax step of every (token, head) row: a warp per row; keys a token may not see count as absent
        for (int r = warp; r < ntk * GRP; r += NW) {
            const int tk = r / GRP, i = r - tk * GRP;
            const int nj = max(0, min(njt, pos0 + tk + 1 - j0));
            float tm = -INFINITY;
            for (int j = lane; j < nj; j += 32) tm = fmaxf(tm, sp[r * 128 + j]);
            tm = hx_warp_max(tm);
            const float mo = sm_m[tk][i], mn = fmaxf(mo, tm);
            float ls = 0.0f;
            for (int j = lane; j < KT; j += 32) {
                const float pr = j < nj ? __expf(sp[r * 128 + j] - mn) : 0.0f;
                sp[r * 128 + j] = pr; ls += pr;
            }
            ls = hx_warp_sum(ls);
            if (lane == 0) { const float rr = __expf(mo - mn); sm_r[tk][i] = rr; sm_l[tk][i] = sm_l[tk][i] * rr + ls; sm_m[tk][i] = mn; }
        }
        __syncthreads();
        // ---- P*V: a V value is fetched once for all tokens and heads
        {
#pragma unroll
            for (int tk = 0; tk < TG; tk++)
#pragma unroll
                for (int i = 0; i < GRP; i++) acc[tk][i] *= (tk < ntk ? sm_r[tk][i] : 1.0f);
            const int jlo = ksub * krun;
            for (int jj = 0; jj < krun; jj += 4) {
                const int j = jlo + jj;
                if (j >= njm) break;
                float vv[4];
#pragma unroll
                for (int u = 0; u < 4; u++) vv[u] = j + u < njm ? vt[(size_t)(j + u) * DH + d] : 0.0f;
#pragma unroll
                for (int tk = 0; tk < TG; tk++) {
                    if (tk >= ntk) break;
#pragma unroll
                    for (int i = 0; i < GRP; i++) {
                        const float4 p4 = *reinterpret_cast<const float4*>(sp + (tk * GRP + i) * 128 + j);
                        acc[tk][i] = fmaf(p4.x, vv[0], acc[tk][i]); acc[tk][i] = fmaf(p4.y, vv[1], acc[tk][i]);
                        acc[tk][i] = fmaf(p4.z, vv[2], acc[tk][i]); acc[tk][i] = fmaf(p4.w, vv[3], acc[tk][i]);
                    }
                }
            }
        }
        __syncthreads();
    }
    const bool bad = sm_abort != 0;       // (every thread passed a barrier after the last write of the flag)
    if (bad && tid == 0 && err) *err = 1;
    const int PW = GRP * (DH + 2);
    // per token: add the key runs inside the tiles up, then either the result or this run's (sum, m, l)
#pragma unroll
    for (int tk = 0; tk < TG; tk++) {
        if (tk >= ntk) break;
        const int t = t0 + tk;
        // (lean arrangement: one partial output per warp, in the ring, which no copy writes any more)
        const float* red = lean ? ringf : sacc;
        const int nred = lean ? NW : nsub;
        if (lean) {
#pragma unroll
            for (int i = 0; i < (kLean ? GRP : 1); i++)
                *reinterpret_cast<float4*>(ringf + ((size_t)warp * GRP + i) * DH + lane * 4) = make_float4(acc4[i][0], acc4[i][1], acc4[i][2], acc4[i][3]);
        } else {
#pragma unroll
            for (int i = 0; i < GRP; i++) sacc[((size_t)ksub * GRP + i) * DH + d] = acc[tk][i];
        }
        __syncthreads();
        float* mine = part + ((size_t)(t * gridDim.x + kvh) * NS + s) * PW;
        for (int o = tid; o < GRP * DH; o += PF_AT) {
            const int i = o / DH, dd = o - i * DH;
            float v = 0.0f;
            for (int u = 0; u < nred; u++) v += red[((size_t)u * GRP + i) * DH + dd];
            if (bad) continue;
            if (n_act == 1) ctx[(size_t)t * ld_ctx + (size_t)(kvh * GRP + i) * DH + dd] = v / sm_l[tk][i];
            else mine[o] = v;
        }
        if (n_act > 1 && tid < GRP && !bad) { mine[GRP * DH + tid] = sm_m[tk][tid]; mine[GRP * DH + GRP + tid] = sm_l[tk][tid]; }
        __syncthreads();
    }
    if (n_act == 1) return;
    // several runs: the last CTA of the (token group, kv head) merges the runs in order
    __threadfence();
    __syncthreads();
    if (tid == 0) sm_ticket = atomicAdd(tickets + blockIdx.y * gridDim.x + kvh, 1u);
    __syncthreads();
    if (sm_ticket != (unsigned)(n_act - 1)) return;
    __threadfence();
    for (int tk = 0; tk < ntk; tk++) {
        const int t = t0 + tk;
        const float* all = part + (size_t)(t * gridDim.x + kvh) * NS * PW;
        for (int o = tid; o < GRP * DH; o += PF_AT) {
            const int i = o / DH;
            float mx = -INFINITY;
            for (int r = 0; r < n_act; r++) mx = fmaxf(mx, __ldcg(all + (size_t)r * PW + GRP * DH + i));
            float num = 0.0f, den = 0.0f;
            for (int r = 0; r < n_act; r++) {
                const float w = __expf(__ldcg(all + (size_t)r * PW + GRP * DH + i) - mx);
                num = fmaf(w, __ldcg(all + (size_t)r * PW + o), num);
                den = fmaf(w, __ldcg(all + (size_t)r * PW + GRP * DH + GRP + i), den);
            }
            if (!bad) ctx[(size_t)t * ld_ctx + (size_t)kvh * GRP * DH + o] = num / den;
        }
    }
    if (tid == 0) tickets[blockIdx.y * gridDim.x + kvh] = 0u;
}

// Tensor-parallel chunk: the partial rows of a row-split linear (o_proj, down_proj) summed over the ranks and added to
// the residual stream.  Every rank stores its [n][DM] partial as 8-byte (value, epoch) pairs into every peer's
// exchange area (plain NVLink stores), then adds the ranks' values in rank order -- the same bits on every rank.  A
// matching epoch proves the value beside it (an aligned 8-byte store is single-copy atomic).  Waits are bounded.
struct HxPfPeers { unsigned long long* p[8]; };
__global__ void __launch_bounds__(256) k_pf_tp_reduce(const float* __restrict__ part, float* __restrict__ x, HxPfPeers peers, int rank, int world,
                                                      int count, size_t area_pairs, unsigned ep, unsigned wait_limit, int* err) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)count; i += (size_t)gridDim.x * blockDim.x) {
        const float v = part[i];
        const unsigned long long w64 = ((unsigned long long)ep << 32) | (unsigned long long)__float_as_uint(v);
        for (int w = 0; w < world; w++)
            if (w != rank) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(peers.p[w] + (size_t)rank * area_pairs + i), "l"(w64) : "memory");
        float sum = 0.0f;
        for (int w = 0; w < world; w++) {
            if (w == rank) { sum += v; continue; }
            const unsigned long long* src = peers.p[rank] + (size_t)w * area_pairs + i;
            unsigned long long got = 0; bool ok = false;
            for (unsigned t = 0; t < wait_limit; t++) {
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(got) : "l"(src) : "memory");
                if ((unsigned)(got >> 32) == ep) { ok = true; break; }
                if ((t & 1023u) == 1023u && *reinterpret_cast<volatile int*>(err) != 0) break;
            }
            if (!ok) { *err = 1; }
            sum += __uint_as_float((unsigned)got);
        }
        x[i] += sum;
    }
}

// Tensor-parallel batched decode: one CTA per sequence takes the first maximum of this rank's vocabulary slice, the ranks
// exchange (value, global index) as pairs, and every rank keeps the best of all (greater value, or equal value and smaller
// index -- the first maximum of the whole vocabulary); the sequence's position advances by one.
__global__ void __launch_bounds__(1024) k_pf_tp_argmax_rows(const float* __restrict__ logits, int n, int ld, int vocab_off, HxPfPeers peers, int rank, int world,
                                                            size_t area_pairs, unsigned ep, unsigned wait_limit, int* err, int* __restrict__ next, int* __restrict__ pos_arr) {
    const float* lg = logits + (size_t)blockIdx.x * ld;
    float bv = -INFINITY; int bi = INT_MAX;
    for (int i = threadIdx.x; i < n; i += 1024) { const float v = lg[i]; if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; } }
    __shared__ float sv[1024]; __shared__ int si[1024];
    sv[threadIdx.x] = bv; si[threadIdx.x] = bi;
    __syncthreads();
    for (int s = 512; s >= 1; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = sv[threadIdx.x + s]; const int oi = si[threadIdx.x + s];
            if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) { sv[threadIdx.x] = ov; si[threadIdx.x] = oi; }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        float fv = sv[0]; int fi = si[0] == INT_MAX ? INT_MAX : si[0] + vocab_off;
        const size_t o = 2 * (size_t)blockIdx.x;
        const unsigned long long wv = ((unsigned long long)ep << 32) | (unsigned long long)__float_as_uint(fv);
        const unsigned long long wi = ((unsigned long long)ep << 32) | (unsigned long long)(unsigned)fi;
        for (int w = 0; w < world; w++) if (w != rank) {
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(peers.p[w] + (size_t)rank * area_pairs + o), "l"(wv) : "memory");
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(peers.p[w] + (size_t)rank * area_pairs + o + 1), "l"(wi) : "memory");
        }
        for (int w = 0; w < world; w++) if (w != rank) {
            unsigned long long gv = 0, gi = 0; bool ok = false;
            const unsigned long long* src = peers.p[rank] + (size_t)w * area_pairs + o;
            for (unsigned t = 0; t < wait_limit; t++) {
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(gv) : "l"(src) : "memory");
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(gi) : "l"(src + 1) : "memory");
                if ((unsigned)(gv >> 32) == ep && (unsigned)(gi >> 32) == ep) { ok = true; break; }
                if ((t & 1023u) == 1023u && *reinterpret_cast<volatile int*>(err) != 0) break;
            }
            if (!ok) { *err = 1; continue; }
            const float ov = __uint_as_float((unsigned)gv); const int oi = (int)(unsigned)gi;
            if (ov > fv || (ov == fv && oi < fi)) { fv = ov; fi = oi; }
        }
        next[blockIdx.x] = fi == INT_MAX ? 0 : fi;
        if (pos_arr) pos_arr[blockIdx.x] += 1;
    }
}

__global__ void k_pf_advance(int* posp, int n) { if (threadIdx.x == 0) *posp += n; }
// one CTA per token row: first maximum of logits[row][0..n) -> next[row]; the row's position advances by one
__global__ void __launch_bounds__(1024) k_pf_argmax_rows(const float* __restrict__ logits, int n, int ld, int* __restrict__ next, int* __restrict__ pos_arr) {
    const float* lg = logits + (size_t)blockIdx.x * ld;
    float bv = -INFINITY; int bi = INT_MAX;
    for (int i = threadIdx.x; i < n; i += 1024) { const float v = lg[i]; if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; } }
    __shared__ float sv[1024]; __shared__ int si[1024];
    sv[threadIdx.x] = bv; si[threadIdx.x] = bi;
    __syncthreads();
    for (int s = 512; s >= 1; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = sv[threadIdx.x + s]; const int oi = si[threadIdx.x + s];
            if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) { sv[threadIdx.x] = ov; si[threadIdx.x] = oi; }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) { next[blockIdx.x] = si[0] == INT_MAX ? 0 : si[0]; if (pos_arr) pos_arr[blockIdx.x] += 1; }
}

// one CTA per token row: first maximum -> next[row], and how far the runner-up lies below it -> margin[row]
// (0 when two entries tie for the maximum).  The speculative decoder trusts a row only above a margin.
__global__ void __launch_bounds__(1024) k_pf_top2_rows(const float* __restrict__ logits, int n, int ld, int* __restrict__ next, float* __restrict__ margin) {
    const float* lg = logits + (size_t)blockIdx.x * ld;
    float bv = -INFINITY, b2 = -INFINITY; int bi = INT_MAX;
    for (int i = threadIdx.x; i < n; i += 1024) {
        const float v = lg[i];
        if (v > bv || (v == bv && i < bi)) { b2 = fmaxf(b2, bv); bv = v; bi = i; }
        else b2 = fmaxf(b2, v);
    }
    __shared__ float sv[1024], s2[1024]; __shared__ int si[1024];
    sv[threadIdx.x] = bv; s2[threadIdx.x] = b2; si[threadIdx.x] = bi;
    __syncthreads();
    for (int s = 512; s >= 1; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = sv[threadIdx.x + s], o2 = s2[threadIdx.x + s]; const int oi = si[threadIdx.x + s];
            const float mv = sv[threadIdx.x], m2 = s2[threadIdx.x];
            if (ov > mv || (ov == mv && oi < si[threadIdx.x])) { sv[threadIdx.x] = ov; si[threadIdx.x] = oi; s2[threadIdx.x] = fmaxf(fmaxf(m2, o2), mv); }
            else s2[threadIdx.x] = fmaxf(fmaxf(m2, o2), ov);
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) { next[blockIdx.x] = si[0] == INT_MAX ? 0 : si[0]; margin[blockIdx.x] = sv[0] - s2[0]; }
}

__global__ void __launch_bounds__(1024) k_pf_argmax(const float* __restrict__ logits, int n, int* tok, int* hist, int* pos_out, int pos) {   // pos: position of the logits row
    float bv = -INFINITY; int bi = INT_MAX;
    for (int i = threadIdx.x; i < n; i += 1024) { const float v = logits[i]; if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; } }
    __shared__ float sv[1024]; __shared__ int si[1024];
    sv[threadIdx.x] = bv; si[threadIdx.x] = bi;
    __syncthreads();
    for (int s = 512; s >= 1; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = sv[threadIdx.x + s]; const int oi = si[threadIdx.x + s];
            if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) { sv[threadIdx.x] = ov; si[threadIdx.x] = oi; }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const int nt = si[0] == INT_MAX ? 0 : si[0];
        *tok = nt; if (hist) hist[pos + 1] = nt; *pos_out = pos + 1;
    }
}

}  // namespace

void hx_pf_embed(const int* ids, HxPfWhere wh, const float* emb, float* X, int n_tok, int DM, cudaStream_t st) {
    k_pf_embed<<<n_tok, 256, 0, st>>>(ids, wh, emb, X, DM);
    HX_COUNT_LAUNCH(1);
}

void hx_pf_digits(const float* src, int ld, int n_tok, int K, int swiglu, const float* g, float eps,
                  uint8_t* cells, float* scale, cudaStream_t st) {
    const int slices = K >= 8192 ? 8 : 4;
    const int groups = (n_tok + HX_TC_MAX_TOK - 1) / HX_TC_MAX_TOK;
    k_pf_digits<<<dim3(n_tok, slices), 512, 0, st>>>(src, ld, K, swiglu, g, eps, cells, groups, scale);
    HX_COUNT_LAUNCH(1);
}

void hx_pf_qkpost(float* qkv, int ld, int n_tok, HxPfWhere wh, int NH, int NKV, int DH, const float* qn_g, const float* kn_g,
                  float eps, const float* cosT, const float* sinT, float* kc, float* vc, int cap, cudaStream_t st) {
    const int threads = ((DH + 31) / 32) * 32;
    k_pf_qkpost<<<dim3(NH + 2 * NKV, n_tok), threads, 0, st>>>(qkv, ld, wh, NH, NKV, DH, qn_g, kn_g, eps, cosT, sinT, kc, vc, cap);
    HX_COUNT_LAUNCH(1);
}

size_t hx_pf_attn_scratch(int n_tok, int NH, int NKV, int DH) {
    return (size_t)n_tok * NKV * PF_NS_MAX * (NH / NKV) * (DH + 2);
}

template <int GRP, int TG>
static int pf_attn_launch(dim3 grid, size_t smem, cudaStream_t st, const float* qkv, int ld, HxPfWhere wh, int n_tok, int NH, int DH, const float* kc,
                          const float* vc, int cap, float scale, float* ctx, int ld_ctx, float* part, unsigned* tickets, int* err) {
    static std::atomic<unsigned long long> attr_seen{0};
    if (hx_first_on_device(attr_seen)) HX_CUDA(cudaFuncSetAttribute(k_pf_attn<GRP, TG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));      // the kernel has some static shared memory too
    k_pf_attn<GRP, TG><<<grid, PF_AT, smem, st>>>(qkv, ld, wh, n_tok, NH, DH, kc, vc, cap, scale, ctx, ld_ctx, part, tickets, err);
    return HX_OK;
}

int hx_pf_attn(const float* qkv, int ld, int n_tok, HxPfWhere wh, int NH, int NKV, int DH, const float* kc, const float* vc,
               int cap, float scale, float* ctx, int ld_ctx, float* part, unsigned* tickets, int* err, cudaStream_t st) {
    const int GRP = NH / NKV;
    if (DH > 256 || DH % 32) return hx_fail(HX_ERR_ARG, "batched prefill attention: head_dim %d is not a multiple of 32 up to 256", DH);
    if (PF_AT % DH) return hx_fail(HX_ERR_ARG, "batched prefill attention: head_dim %d does not divide %d", DH, PF_AT);
    if (!part || !tickets) return hx_fail(HX_ERR_ARG, "batched prefill attention: no scratch for the key runs");
    // a prefill chunk (one sequence, consecutive positions): four tokens share the tiles of a CTA
    auto smem_of = [&](int tg) { return (size_t)PF_ST * 2 * PF_TILE_BYTES + ((size_t)tg * GRP * DH + (size_t)tg * GRP * 128 + (size_t)(PF_AT / DH) * GRP * DH) * 4; };
    const size_t smem_max = 226 * 1024;
    const int TG = (wh.pos_arr || smem_of(4) > smem_max) ? 1 : 4;
    const int groups = (n_tok + TG - 1) / TG;
    const size_t smem = smem_of(TG);
    if (smem > smem_max) return hx_fail(HX_ERR_ARG, "batched prefill attention: %zu bytes of shared memory", smem);
    // runs of key tiles per (token group, kv head): about two CTAs per SM, no more than the cache has tiles
    const int KT = 128 < PF_TILE_BYTES / (DH * 4) ? 128 : PF_TILE_BYTES / (DH * 4);
    int ns = (2 * 148 + NKV * groups - 1) / (NKV * groups);
    const int cap_tiles = (cap + KT - 1) / KT;
    if (ns > cap_tiles) ns = cap_tiles;
    if (ns > PF_NS_MAX) ns = PF_NS_MAX;
    if (ns < 1) ns = 1;
    dim3 grid(NKV, groups, ns);
    int rc;
#define HX_PF_ATTN(G) case G: rc = TG == 1 ? pf_attn_launch<G, 1>(grid, smem, st, qkv, ld, wh, n_tok, NH, DH, kc, vc, cap, scale, ctx, ld_ctx, part, tickets, err) \
                                            : pf_attn_launch<G, 4>(grid, smem, st, qkv, ld, wh, n_tok, NH, DH, kc, vc, cap, scale, ctx, ld_ctx, part, tickets, err); break;
    switch (GRP) {
        HX_PF_ATTN(1) HX_PF_ATTN(2) HX_PF_ATTN(3) HX_PF_ATTN(4) HX_PF_ATTN(5) HX_PF_ATTN(6) HX_PF_ATTN(7) HX_PF_ATTN(8)
        default: return hx_fail(HX_ERR_ARG, "batched prefill attention: group of %d query heads per kv head not supported", GRP);
    }
#undef HX_PF_ATTN
    if (rc) return rc;
    HX_COUNT_LAUNCH(1);
    return HX_OK;
}

void hx_pf_tp_reduce(const float* part, float* x, unsigned long long* const* peer_areas, int rank, int world, int count, size_t area_pairs,
                     unsigned ep, unsigned wait_limit, int* err, cudaStream_t st) {
    HxPfPeers pe = {};
    for (int w = 0; w < world && w < 8; w++) pe.p[w] = peer_areas[w];
    int g = (count + 255) / 256; if (g > 148 * 4) g = 148 * 4;
    k_pf_tp_reduce<<<g, 256, 0, st>>>(part, x, pe, rank, world, count, area_pairs, ep, wait_limit, err);
    HX_COUNT_LAUNCH(1);
}

void hx_pf_tp_argmax_rows(const float* logits, int n, int ld, int rows, int vocab_off, unsigned long long* const* peer_areas, int rank, int world,
                          size_t area_pairs, unsigned ep, unsigned wait_limit, int* err, int* next, int* pos_arr, cudaStream_t st) {
    HxPfPeers pe = {};
    for (int w = 0; w < world && w < 8; w++) pe.p[w] = peer_areas[w];
    k_pf_tp_argmax_rows<<<rows, 1024, 0, st>>>(logits, n, ld, vocab_off, pe, rank, world, area_pairs, ep, wait_limit, err, next, pos_arr);
    HX_COUNT_LAUNCH(1);
}

void hx_pf_advance(int* posp, int n, cudaStream_t st) {
    k_pf_advance<<<1, 32, 0, st>>>(posp, n);
    HX_COUNT_LAUNCH(1);
}

void hx_pf_argmax(const float* logits, int n, int* tok, int* hist, int* pos_out, int pos, cudaStream_t st) {
    k_pf_argmax<<<1, 1024, 0, st>>>(logits, n, tok, hist, pos_out, pos);
    HX_COUNT_LAUNCH(1);
}

void hx_pf_top2_rows(const float* logits, int n, int ld, int rows, int* next, float* margin, cudaStream_t st) {
    k_pf_top2_rows<<<rows, 1024, 0, st>>>(logits, n, ld, next, margin);
    HX_COUNT_LAUNCH(1);
}

void hx_pf_argmax_rows(const float* logits, int n, int ld, int rows, int* next, int* pos_arr, cudaStream_t st) {
    k_pf_argmax_rows<<<rows, 1024, 0, st>>>(logits, n, ld, next, pos_arr);
    HX_COUNT_LAUNCH(1);
}
