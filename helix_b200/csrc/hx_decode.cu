// hx_decode.cu -- the batch-1 decode kernels over HBM-resident NVFP4 weights.
//
// These replace, for one token, the kernel sequence of decode_step_llama
// (helixc/runtime/gpt2_infer.c:1341-1613): rms_norm_k + fused_gemv (q,k,v), QK-norm, rope_at, the
// KV appends, fused_decode_attn, fused_gemv (o) + vadd, rms_norm_k + fused_gemv (gate, up) +
// silu_mul_k, fused_gemv (down) + vadd, final norm + fused_lm_head + the host argmax.
//
// k_linear: y = epilogue(W . norm(x)).  HBM-bound; each weight byte is read once with a 128-bit
// load, decoded in registers (cvt.rn.f16x2.e2m1x2) and multiplied in f32.  Algorithmic bytes per
// weight: 0.5 (code) + 1/16 (scale) = 0.5625.
#include "hx_kernels.cuh"
#include <cuda_fp16.h>
#include <limits.h>

#define LIN_THREADS 256
#define LIN_WARPS 8
#define PIECE_PAD 36      // a 32-float piece of x occupies 36 floats of shared memory (bank spread)

// ---- loads ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_stream_v4(const uint4* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ uint32_t ld_stream_u16(const uint8_t* p) {
    unsigned short r;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(r) : "l"(p));
    return r;
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" :: "l"(p));
}

// ---- in-register decode --------------------------------------------------------------------------
// Four bytes = eight E2M1 codes -> four f16x2 (low nibble of each byte in the low half).
__device__ __forceinline__ void e2m1x8_to_f16x2(uint32_t w, uint32_t& h0, uint32_t& h1, uint32_t& h2, uint32_t& h3) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3) : "r"(w));
}
// Two E4M3 bytes -> two f32 (every E4M3 value is exact in f16).
__device__ __forceinline__ float2 e4m3x2_to_f32(uint32_t s16) {
    uint32_t h;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"((unsigned short)s16));
    return __half22float2(*reinterpret_cast<__half2*>(&h));
}
// sum of x[0..7] * mag(code_i) over the eight codes of w, added to part
__device__ __forceinline__ float dot8(uint32_t w, const float4 xa, const float4 xb, float part) {
    uint32_t h0, h1, h2, h3;
    e2m1x8_to_f16x2(w, h0, h1, h2, h3);
    float2 f;
    f = __half22float2(*reinterpret_cast<__half2*>(&h0)); part = fmaf(xa.x, f.x, part); part = fmaf(xa.y, f.y, part);
    f = __half22float2(*reinterpret_cast<__half2*>(&h1)); part = fmaf(xa.z, f.x, part); part = fmaf(xa.w, f.y, part);
    f = __half22float2(*reinterpret_cast<__half2*>(&h2)); part = fmaf(xb.x, f.x, part); part = fmaf(xb.y, f.y, part);
    f = __half22float2(*reinterpret_cast<__half2*>(&h3)); part = fmaf(xb.z, f.x, part); part = fmaf(xb.w, f.y, part);
    return part;
}

__device__ __forceinline__ float block_sum(float v, float* red /*[LIN_WARPS]*/) {
    v = hx_warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < LIN_WARPS; i++) s += red[i];
    return s;
}

__device__ __forceinline__ float silu_mul(float g, float u) {
    // gpu_silu_mul_kernel.hx:20-31: sigmoid(g) = 0.5*(1 + sgn*(1-e)/(1+e)), e = exp(-|g|)
    const float sgn = g < 0.0f ? -1.0f : 1.0f;
    const float e = __expf(-(sgn * g));
    const float th = sgn * ((1.0f - e) / (1.0f + e));
    return g * (0.5f * (1.0f + th)) * u;
}
__device__ __forceinline__ float gelu_new(float xi) {
    // gpu_gelu_stable_kernel.hx:15-28
    const float inner = 0.7978846f * (xi + (0.044715f * (xi * xi * xi)));
    const float two = 2.0f * inner;
    const float sgn = inner < 0.0f ? -1.0f : 1.0f;
    const float e = __expf(-(sgn * two));
    const float th = sgn * ((1.0f - e) / (1.0f + e));
    return 0.5f * xi * (1.0f + th);
}

__device__ __forceinline__ bool better(float av, int ai, float bv, int bi) {
    return av > bv || (av == bv && ai < bi);
}

// ------------------------------------------------------------------------------------------------
// k_linear<R>: a warp owns R consecutive rows at a time; lane l walks the pieces l, l+32, ... of
// those rows (one 16-byte load of 32 codes and one 2-byte load of 2 scales per row and piece), the
// x piece is read once from shared memory for all R rows.  Per 16-element block the products are
// summed first and the block scale applied once; the tensor scale is applied to the row sum.
// ------------------------------------------------------------------------------------------------
template <int R>
__global__ void __launch_bounds__(LIN_THREADS, 2) k_linear(const __grid_constant__ HxLinear a) {
    extern __shared__ __align__(16) float xs[];
    __shared__ float red[LIN_WARPS];
    __shared__ float s_bv[LIN_WARPS];
    __shared__ int s_bi[LIN_WARPS];
    __shared__ unsigned s_ticket;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int npiece = a.Kd >> 5, nsc = a.Kd >> 4;
    const int ngroups = (a.N + R - 1) / R;
    const int nwarps = gridDim.x * LIN_WARPS;
    const int gw = blockIdx.x * LIN_WARPS + warp;

    // Weights never depend on the previous kernel: pull this warp's first rows toward L2 before
    // waiting for it, then let the next kernel do the same.
    if (gw < ngroups) {
        const int row0 = gw * R;
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int rr = min(row0 + r, a.N - 1);
            const char* base = reinterpret_cast<const char*>(a.codes + (size_t)rr * npiece);
            for (int off = lane * 128; off < npiece * 16; off += 32 * 128) prefetch_l2(base + off);
        }
    }
    hx_grid_dep_launch();
    hx_grid_dep_wait();

    // ---- stage norm(x) into shared memory, 36 floats per 32-element piece ----
    {
        const int n4 = a.Kd >> 2;
        float s1 = 0.0f;
        for (int k4 = tid; k4 < n4; k4 += LIN_THREADS) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (4 * k4 < a.K) v = *reinterpret_cast<const float4*>(a.x + 4 * k4);
            *reinterpret_cast<float4*>(xs + (k4 >> 3) * PIECE_PAD + (k4 & 7) * 4) = v;
            if (a.norm == HX_NORM_RMS) s1 += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            else if (a.norm == HX_NORM_LAYER) s1 += v.x + v.y + v.z + v.w;
        }
        if (a.norm != HX_NORM_NONE) {
            float mean = 0.0f, inv;
            if (a.norm == HX_NORM_RMS) {
                const float ss = block_sum(s1, red);
                inv = rsqrtf(ss / (float)a.K + a.eps);
            } else {
                mean = block_sum(s1, red) / (float)a.K;
                float s2 = 0.0f;
                for (int k4 = tid; k4 < n4; k4 += LIN_THREADS) {
                    if (4 * k4 < a.K) {
                        const float4 v = *reinterpret_cast<const float4*>(xs + (k4 >> 3) * PIECE_PAD + (k4 & 7) * 4);
                        s2 += (v.x - mean) * (v.x - mean) + (v.y - mean) * (v.y - mean) + (v.z - mean) * (v.z - mean) +
                              (v.w - mean) * (v.w - mean);
                    }
                }
                inv = rsqrtf(block_sum(s2, red) / (float)a.K + a.eps);
            }
            for (int k4 = tid; k4 < n4; k4 += LIN_THREADS) {
                if (4 * k4 < a.K) {
                    float4* p = reinterpret_cast<float4*>(xs + (k4 >> 3) * PIECE_PAD + (k4 & 7) * 4);
                    float4 v = *p;
                    const float4 g = *reinterpret_cast<const float4*>(a.norm_g + 4 * k4);
                    v.x = g.x * ((v.x - mean) * inv); v.y = g.y * ((v.y - mean) * inv);
                    v.z = g.z * ((v.z - mean) * inv); v.w = g.w * ((v.w - mean) * inv);
                    if (a.norm == HX_NORM_LAYER) {
                        const float4 b = *reinterpret_cast<const float4*>(a.norm_b + 4 * k4);
                        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
                    }
                    *p = v;
                }
            }
        }
        __syncthreads();
    }

    float best_v = -INFINITY; int best_i = INT_MAX;

    for (int grp = gw; grp < ngroups; grp += nwarps) {
        const int row0 = grp * R;
        float acc[R];
        const uint4* cp[R]; const uint8_t* sp[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            acc[r] = 0.0f;
            const int rr = min(row0 + r, a.N - 1);
            cp[r] = a.codes + (size_t)rr * npiece;
            sp[r] = a.scales + (size_t)rr * nsc;
        }
#pragma unroll 2
        for (int p = lane; p < npiece; p += 32) {
            uint4 q[R]; uint32_t s[R];
#pragma unroll
            for (int r = 0; r < R; r++) { q[r] = ld_stream_v4(cp[r] + p); s[r] = ld_stream_u16(sp[r] + 2 * p); }
            const float4* xp = reinterpret_cast<const float4*>(xs + p * PIECE_PAD);
            const float4 x0 = xp[0], x1 = xp[1], x2 = xp[2], x3 = xp[3], x4 = xp[4], x5 = xp[5], x6 = xp[6], x7 = xp[7];
#pragma unroll
            for (int r = 0; r < R; r++) {
                float pa = dot8(q[r].x, x0, x1, 0.0f); pa = dot8(q[r].y, x2, x3, pa);
                float pb = dot8(q[r].z, x4, x5, 0.0f); pb = dot8(q[r].w, x6, x7, pb);
                const float2 sc = e4m3x2_to_f32(s[r]);
                acc[r] = fmaf(pa, sc.x, acc[r]);
                acc[r] = fmaf(pb, sc.y, acc[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < R; r++) acc[r] = hx_warp_sum(acc[r]);

        if (a.epi == HX_EPI_SWIGLU) {
            // rows (2i, 2i+1) = (gate_i, up_i)
            if (lane < R / 2) {
                float g = acc[0], u = acc[1];
#pragma unroll
                for (int j = 1; j < R / 2; j++) if (lane == j) { g = acc[2 * j]; u = acc[2 * j + 1]; }
                const int i = row0 / 2 + lane;
                if (2 * i + 1 < a.N) a.y[i] = silu_mul(g * a.ts[0], u * a.ts[1]);
            }
        } else if (lane < R) {
            float v = acc[0];
#pragma unroll
            for (int r = 1; r < R; r++) if (lane == r) v = acc[r];
            const int row = row0 + lane;
            if (row < a.N) {
                v *= (row < a.bound0) ? a.ts[0] : (row < a.bound1 ? a.ts[1] : a.ts[2]);
                if (a.bias) v += a.bias[row];
                if (a.epi == HX_EPI_RESID) v = a.resid[row] + v;
                else if (a.epi == HX_EPI_GELU) v = gelu_new(v);
                a.y[row] = v;
                if (a.epi == HX_EPI_ARGMAX && better(v, row, best_v, best_i)) { best_v = v; best_i = row; }
            }
        }
    }

    if (a.epi == HX_EPI_ARGMAX) {
        // block-level best, then the last CTA to arrive folds the per-CTA partials (no waiting)
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best_v, d);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, d);
            if (better(ov, oi, best_v, best_i)) { best_v = ov; best_i = oi; }
        }
        if (lane == 0) { s_bv[warp] = best_v; s_bi[warp] = best_i; }
        __syncthreads();
        if (tid == 0) {
            float bv = s_bv[0]; int bi = s_bi[0];
            for (int i = 1; i < LIN_WARPS; i++) if (better(s_bv[i], s_bi[i], bv, bi)) { bv = s_bv[i]; bi = s_bi[i]; }
            a.part_val[blockIdx.x] = bv; a.part_idx[blockIdx.x] = bi;
            __threadfence();
            s_ticket = atomicAdd(a.counter, 1u);
        }
        __syncthreads();
        if (s_ticket == gridDim.x - 1) {
            __threadfence();
            float bv = -INFINITY; int bi = INT_MAX;
            for (int i = tid; i < (int)gridDim.x; i += LIN_THREADS) {
                const float ov = __ldcg(a.part_val + i); const int oi = __ldcg(a.part_idx + i);
                if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, d);
                if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
            __syncthreads();
            if (lane == 0) { s_bv[warp] = bv; s_bi[warp] = bi; }
            __syncthreads();
            if (tid == 0) {
                for (int i = 1; i < LIN_WARPS; i++) if (better(s_bv[i], s_bi[i], bv, bi)) { bv = s_bv[i]; bi = s_bi[i]; }
                const int nt = (bi == INT_MAX) ? 0 : bi;
                *a.next_tok = nt;
                if (a.pos_inc) {
                    const int np = *a.pos_inc + 1;          // position the new token will occupy
                    *a.pos_inc = np;
                    if (a.hist) a.hist[np] = nt;
                }
                *a.counter = 0u;
            }
        }
    }
}

size_t hx_linear_smem_bytes(int Kd) { return (size_t)(Kd / 32) * PIECE_PAD * sizeof(float); }

static int g_sm_count = 0;
static int sm_count() {
    if (!g_sm_count) {
        int dev = 0; cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    return g_sm_count;
}

template <typename... KArgs, typename... Args>
static cudaError_t launch_ex(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                             Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl ? 1 : 0;
    HX_COUNT_LAUNCH(1);
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

int hx_launch_linear(const HxLinear& a, cudaStream_t st, bool pdl) {
    HX_CHECK_ARG(a.codes && a.scales && a.x && a.y && a.N > 0 && a.K > 0);
    HX_CHECK_ARG(a.Kd % 64 == 0 && a.Kd >= a.K && a.K % 4 == 0);
    HX_CHECK_ARG((((uintptr_t)a.x) & 15) == 0 && (((uintptr_t)a.codes) & 15) == 0 && (((uintptr_t)a.scales) & 1) == 0);
    const size_t smem = hx_linear_smem_bytes(a.Kd);
    if (smem > 200 * 1024) return hx_fail(HX_ERR_ARG, "K=%d too large for the shared-memory staging of x", a.K);
    static std::atomic<unsigned long long> attr_seen{0};
    if (hx_first_on_device(attr_seen))
        HX_CUDA(cudaFuncSetAttribute(k_linear<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    const int R = 4;
    const int ngroups = (a.N + R - 1) / R;
    int grid = (ngroups + LIN_WARPS - 1) / LIN_WARPS;
    const int cap = sm_count() * 2;
    if (grid > cap) grid = cap;
    if (a.epi == HX_EPI_SWIGLU) HX_CHECK_ARG(a.N % 2 == 0);
    HX_CUDA(launch_ex(k_linear<4>, dim3(grid), dim3(LIN_THREADS), smem, st, pdl, a));
    return HX_OK;
}

// ------------------------------------------------------------------------------------------------
// k_qk_prep: one CTA per head (NH query heads, then NKV key heads), DH threads.  Query heads:
// per-head RMSNorm (Qwen3), RoPE at *pos, result to q_rot.  Key heads: the same on k, appended to
// the cache at *pos together with the raw v.  Replaces rms_norm_k over NH/NKV rows, NH+NKV rope_at
// launches and 2*NKV device copies per layer (gpt2_infer.c:1500-1511).
// RoPE: rotate_half pairs (i, i+DH/2) with table row *pos (gpu_rope_rot_kernel.hx:23-38).
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_qk_prep(const __grid_constant__ HxAttn a) {
    __shared__ float buf[256];
    __shared__ float red[8];
    hx_grid_dep_launch();
    hx_grid_dep_wait();
    const int h = blockIdx.x, d = threadIdx.x, DH = a.DH, half = DH >> 1;
    const bool isq = h < a.NH;
    const int kvh = h - a.NH;
    const int pos = *a.pos;
    const float* src = isq ? a.qkv + (size_t)h * DH : a.qkv + (size_t)a.NH * DH + (size_t)kvh * DH;
    float v = src[d];
    const float* g = isq ? a.qn_g : a.kn_g;
    if (g) {
        float ss = hx_warp_sum(v * v);
        if ((d & 31) == 0) red[d >> 5] = ss;
        __syncthreads();
        float tot = 0.0f;
        for (int i = 0; i < (DH >> 5); i++) tot += red[i];
        v = g[d] * (v * rsqrtf(tot / (float)DH + a.eps));
    }
    if (a.cosT) {
        buf[d] = v;
        __syncthreads();
        const int i = d < half ? d : d - half;
        const float c = a.cosT[(size_t)pos * half + i], s = a.sinT[(size_t)pos * half + i];
        const float lo = buf[i], hi = buf[i + half];
        v = d < half ? lo * c - hi * s : hi * c + lo * s;
    }
    if (isq) a.q_rot[(size_t)h * DH + d] = v;
    else {
        const size_t o = ((size_t)kvh * a.cap + pos) * DH + d;
        a.kc[o] = v;
        a.vc[o] = a.qkv[(size_t)a.NH * DH + (size_t)a.NKV * DH + (size_t)kvh * DH + d];
    }
}

int hx_launch_qk_prep(const HxAttn& a, cudaStream_t st, bool pdl) {
    HX_CHECK_ARG(a.DH % 32 == 0 && a.DH <= 256 && a.NH % a.NKV == 0);
    HX_CUDA(launch_ex(k_qk_prep, dim3(a.NH + a.NKV), dim3(a.DH), 0, st, pdl, a));
    return HX_OK;
}

// ------------------------------------------------------------------------------------------------
// k_attn<GRP>: one CTA per (kv head, split of the cached positions); the GRP query heads that share
// the kv head are processed together so K and V are read once.  Within the CTA the split is walked
// in tiles of ATT_TILE positions with the online-softmax recurrence of the reference's fused kernel
// (fused_decode_attn_kernel.hx:74-102: running max seeded -1e8, rescale by exp(m - m_new)); the
// per-split partial (m, l, acc) goes to scratch and the last CTA of a kv head to finish merges the
// splits and writes ctx.  HBM-bound: 2*T*DH*4 bytes per kv head.
// ------------------------------------------------------------------------------------------------
#define ATT_THREADS 128
#define ATT_TILE 128

template <int GRP>
__global__ void __launch_bounds__(ATT_THREADS) k_attn(const __grid_constant__ HxAttn a) {
    __shared__ __align__(16) float sq[GRP][256];
    __shared__ float sp[GRP][ATT_TILE];
    __shared__ float sm_m[GRP], sm_l[GRP], sm_r[GRP];
    __shared__ unsigned s_ticket;
    hx_grid_dep_launch();
    hx_grid_dep_wait();
    const int kv = blockIdx.x, split = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int DH = a.DH, T = *a.pos + 1;
    const int chunk = (T + a.nsplit - 1) / a.nsplit;
    const int t0 = split * chunk, t1 = min(T, t0 + chunk);
    const float* kb = a.kc + (size_t)kv * a.cap * DH;
    const float* vb = a.vc + (size_t)kv * a.cap * DH;
    for (int i = tid; i < GRP * DH; i += ATT_THREADS) sq[i / DH][i % DH] = a.q_rot[(size_t)kv * GRP * DH + i];
    if (tid < GRP) { sm_m[tid] = -100000000.0f; sm_l[tid] = 0.0f; }
    __syncthreads();

    // each thread owns output dims d = tid and tid + 128 (DH <= 256)
    float acc0[GRP], acc1[GRP];
#pragma unroll
    for (int g = 0; g < GRP; g++) { acc0[g] = 0.0f; acc1[g] = 0.0f; }

    for (int tb = t0; tb < t1; tb += ATT_TILE) {
        const int nt = min(ATT_TILE, t1 - tb);
        // scores: a warp takes positions warp, warp+4, ...; lanes split the head dimension
        for (int t = warp; t < nt; t += ATT_THREADS / 32) {
            const float* kr = kb + (size_t)(tb + t) * DH;
            float dot[GRP];
#pragma unroll
            for (int g = 0; g < GRP; g++) dot[g] = 0.0f;
            for (int e = lane * 4; e < DH; e += 128) {
                const float4 k4 = *reinterpret_cast<const float4*>(kr + e);
#pragma unroll
                for (int g = 0; g < GRP; g++) {
                    const float4 q4 = *reinterpret_cast<const float4*>(&sq[g][e]);
                    dot[g] = fmaf(q4.x, k4.x, dot[g]); dot[g] = fmaf(q4.y, k4.y, dot[g]);
                    dot[g] = fmaf(q4.z, k4.z, dot[g]); dot[g] = fmaf(q4.w, k4.w, dot[g]);
                }
            }
#pragma unroll
            for (int g = 0; g < GRP; g++) {
                const float s = hx_warp_sum(dot[g]);
                if (lane == 0) sp[g][t] = s * a.scale;
            }
        }
        __syncthreads();
        // per head: new running max, rescale factor, probabilities in place
        for (int g = warp; g < GRP; g += ATT_THREADS / 32) {
            float mx = -INFINITY;
            for (int t = lane; t < nt; t += 32) mx = fmaxf(mx, sp[g][t]);
            mx = hx_warp_max(mx);
            const float mo = sm_m[g], mn = fmaxf(mo, mx);
            float ls = 0.0f;
            for (int t = lane; t < nt; t += 32) { const float p = __expf(sp[g][t] - mn); sp[g][t] = p; ls += p; }
            ls = hx_warp_sum(ls);
            if (lane == 0) { const float r = __expf(mo - mn); sm_r[g] = r; sm_l[g] = sm_l[g] * r + ls; sm_m[g] = mn; }
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < GRP; g++) { const float r = sm_r[g]; acc0[g] *= r; acc1[g] *= r; }
        for (int t = 0; t < nt; t++) {
            const float* vr = vb + (size_t)(tb + t) * DH;
            const float v0 = tid < DH ? vr[tid] : 0.0f;
            const float v1 = tid + ATT_THREADS < DH ? vr[tid + ATT_THREADS] : 0.0f;
#pragma unroll
            for (int g = 0; g < GRP; g++) { const float p = sp[g][t]; acc0[g] = fmaf(p, v0, acc0[g]); acc1[g] = fmaf(p, v1, acc1[g]); }
        }
        __syncthreads();
    }

    // partials of this split
#pragma unroll
    for (int g = 0; g < GRP; g++) {
        const size_t hs = (size_t)(kv * GRP + g) * a.nsplit + split;
        if (tid < DH) a.part_acc[hs * DH + tid] = acc0[g];
        if (tid + ATT_THREADS < DH) a.part_acc[hs * DH + tid + ATT_THREADS] = acc1[g];
        if (tid == 0) { a.part_m[hs] = sm_m[g]; a.part_l[hs] = sm_l[g]; }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(a.counters + kv, 1u);
    __syncthreads();
    if (s_ticket != (unsigned)a.nsplit - 1) return;
    __threadfence();
    // merge: out = sum_s acc_s * exp(m_s - M) / sum_s l_s * exp(m_s - M)
    for (int g = 0; g < GRP; g++) {
        const size_t h0 = (size_t)(kv * GRP + g) * a.nsplit;
        float M = -INFINITY;
        for (int s = 0; s < a.nsplit; s++) M = fmaxf(M, __ldcg(a.part_m + h0 + s));
        float L = 0.0f, o0 = 0.0f, o1 = 0.0f;
        for (int s = 0; s < a.nsplit; s++) {
            const float w = __expf(__ldcg(a.part_m + h0 + s) - M);
            L = fmaf(__ldcg(a.part_l + h0 + s), w, L);
            if (tid < DH) o0 = fmaf(__ldcg(a.part_acc + (h0 + s) * DH + tid), w, o0);
            if (tid + ATT_THREADS < DH) o1 = fmaf(__ldcg(a.part_acc + (h0 + s) * DH + tid + ATT_THREADS), w, o1);
        }
        if (tid < DH) a.ctx[(size_t)(kv * GRP + g) * DH + tid] = o0 / L;
        if (tid + ATT_THREADS < DH) a.ctx[(size_t)(kv * GRP + g) * DH + tid + ATT_THREADS] = o1 / L;
    }
    if (tid == 0) a.counters[kv] = 0u;
}

int hx_launch_attn(const HxAttn& a, cudaStream_t st, bool pdl) {
    HX_CHECK_ARG(a.DH % 4 == 0 && a.DH <= 256 && a.NH % a.NKV == 0 && a.nsplit >= 1);
    const int grp = a.NH / a.NKV;
    dim3 grid(a.NKV, a.nsplit), block(ATT_THREADS);
    cudaError_t e;
    switch (grp) {
        case 1: e = launch_ex(k_attn<1>, grid, block, 0, st, pdl, a); break;
        case 2: e = launch_ex(k_attn<2>, grid, block, 0, st, pdl, a); break;
        case 3: e = launch_ex(k_attn<3>, grid, block, 0, st, pdl, a); break;
        case 4: e = launch_ex(k_attn<4>, grid, block, 0, st, pdl, a); break;
        case 5: e = launch_ex(k_attn<5>, grid, block, 0, st, pdl, a); break;
        case 6: e = launch_ex(k_attn<6>, grid, block, 0, st, pdl, a); break;
        case 7: e = launch_ex(k_attn<7>, grid, block, 0, st, pdl, a); break;
        case 8: e = launch_ex(k_attn<8>, grid, block, 0, st, pdl, a); break;
        default: return hx_fail(HX_ERR_ARG, "unsupported GQA group size %d (1..8)", grp);
    }
    HX_CUDA(e);
    return HX_OK;
}

// ------------------------------------------------------------------------------------------------
// small ops
// ------------------------------------------------------------------------------------------------
__global__ void k_embed(const float* __restrict__ emb, const float* __restrict__ wpe, const int* __restrict__ tok,
                        const int* __restrict__ pos, int index_by_pos, float* __restrict__ x, int DM) {
    hx_grid_dep_launch();
    hx_grid_dep_wait();
    const size_t t = (size_t)tok[index_by_pos ? pos[0] : 0];
    const size_t p = wpe ? (size_t)pos[0] : 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < DM; i += gridDim.x * blockDim.x)
        x[i] = wpe ? emb[t * DM + i] + wpe[p * DM + i] : emb[t * DM + i];
}
int hx_launch_embed(const float* emb, const float* wpe, const int* tok, const int* pos, int index_by_pos, float* x,
                    int DM, cudaStream_t st, bool pdl) {
    HX_CUDA(launch_ex(k_embed, dim3((DM + 255) / 256), dim3(256), 0, st, pdl, emb, wpe, tok, pos, index_by_pos, x, DM));
    return HX_OK;
}

// Counter-based N(0, sigma): splitmix64 of (seed, pair index) -> two uniforms -> Box-Muller.
__device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__global__ void k_fill_normal(float* __restrict__ p, size_t n, float sigma, uint64_t seed) {
    const size_t npair = (n + 1) / 2;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < npair; i += (size_t)gridDim.x * blockDim.x) {
        const uint64_t r = splitmix64(seed * 0xD1342543DE82EF95ull + i);
        const float u1 = ((float)(uint32_t)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);   // (0,1)
        const float u2 = ((float)(uint32_t)((r >> 8) & 0xFFFFFF)) * (1.0f / 16777216.0f);
        const float rad = sqrtf(-2.0f * logf(u1)) * sigma;
        float sn, cs; sincospif(2.0f * u2, &sn, &cs);
        p[2 * i] = rad * cs;
        if (2 * i + 1 < n) p[2 * i + 1] = rad * sn;
    }
}
int hx_launch_fill_normal(float* p, size_t n, float sigma, uint64_t seed, cudaStream_t st) {
    size_t np = (n + 1) / 2;
    int g = (int)((np + 255) / 256); if (g > 148 * 16) g = 148 * 16; if (g < 1) g = 1;
    k_fill_normal<<<g, 256, 0, st>>>(p, n, sigma, seed);
    HX_COUNT_LAUNCH(1);
    HX_CUDA(cudaGetLastError());
    return HX_OK;
}
__global__ void k_fill_const(float* __restrict__ p, size_t n, float v) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = v;
}
int hx_launch_fill_const(float* p, size_t n, float v, cudaStream_t st) {
    int g = (int)((n + 255) / 256); if (g > 148 * 16) g = 148 * 16; if (g < 1) g = 1;
    k_fill_const<<<g, 256, 0, st>>>(p, n, v);
    HX_COUNT_LAUNCH(1);
    HX_CUDA(cudaGetLastError());
    return HX_OK;
}

// Stand-alone GEMV over the dense layout (C-ABI, device pointers).
HX_API int hx_gemv_d16(const float* x, const uint8_t* codes, const uint8_t* scales, const float* ts,
                       float* y, int N, int Kd, void* stream) {
    HX_CHECK_ARG(x && codes && scales && ts && y && N > 0 && Kd > 0 && Kd % 64 == 0);
    float tsv = 0.0f;
    HX_CUDA(cudaMemcpyAsync(&tsv, ts, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    HX_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    HxLinear a = {};
    a.codes = reinterpret_cast<const uint4*>(codes); a.scales = scales;
    a.ts[0] = a.ts[1] = a.ts[2] = tsv; a.bound0 = a.bound1 = N;
    a.N = N; a.K = Kd; a.Kd = Kd; a.x = x; a.norm = HX_NORM_NONE; a.y = y; a.epi = HX_EPI_STORE;
    return hx_launch_linear(a, (cudaStream_t)stream, false);
}
