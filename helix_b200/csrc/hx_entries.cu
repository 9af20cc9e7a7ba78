// hx_entries.cu -- the kernel-entry ABI of the Helix inference worker, for sm_100a.
//
// The reference's C host programs load a module with cuModuleLoadData, look entries up by name with
// cuModuleGetFunction and launch them with fixed grid/block shapes, zero dynamic shared memory and
// the NULL stream (helixc/runtime/gpt2_infer.c:373-470, 1944-1964, 2281-2326;
// helixc/runtime/cuda_launch.c:1087-1088).  This file is compiled to helix_b200_kernels.fatbin,
// which can be passed wherever the reference passes its emitted PTX: every entry below has the
// name, parameter order and parameter types of the corresponding emitted kernel (pointers are
// 64-bit device pointers, scalars are 32-bit), uses static shared memory only, never allocates and
// never traps.  Index arithmetic follows the caller's geometry (one thread per row / element /
// output where the reference launches it that way), so each entry is correct under exactly the
// launch shapes the worker and the test launcher use.
//
// Arithmetic order follows the kernel sources under helixc/examples and the emitters in
// helixc/bootstrap/kovc.hx (fused GEMV: :14432-14692, softmax/norm intrinsics: :12276-12318):
// f32 throughout, ascending sums, exp as ex2.approx(x*log2e), rsqrt.approx for the norms.
#include "hx_common.cuh"

// nvfp4_dequant_kernel.hx:35-51 -- grid=(M) block=(K).
extern "C" __global__ void nvfp4_dequant(const int* w, const float* sc, float* out, int mm, int kk, int nn) {
    const int row = blockIdx.x, col = threadIdx.x;
    const int word = col / 7, slot = col - word * 7;
    const unsigned wv = (unsigned)w[row * (kk / 7) + word];
    const int code = (wv >> (4 * slot)) & 15;
    out[row * kk + col] = __fmul_rn(hx_e2m1_dec(code), sc[row * (kk / 16) + col / 16]);
}

// nvfp4_dequant_tiled_kernel.hx:24-43 -- grid=(rows*ceil(kk/nn)) block=(nn).
extern "C" __global__ void nvfp4_dequant_tiled(const int* w, const float* sc, float* out, int mm, int kk, int nn) {
    const int lb = blockIdx.x, ntile = (kk + nn - 1) / nn;
    const int row = lb / ntile, col = (lb - row * ntile) * nn + threadIdx.x;
    const int word = col / 7, slot = col - word * 7;
    const unsigned wv = (unsigned)w[(size_t)row * (kk / 7) + word];
    const int code = (wv >> (4 * slot)) & 15;
    out[(size_t)row * kk + col] = __fmul_rn(hx_e2m1_dec(code), sc[(size_t)row * (kk / 16) + col / 16]);
}

// gemv_abt_nvfp4_kernel.hx:25-50 -- one thread per output, collapsed f32 scales.
extern "C" __global__ void gemv_abt_nvfp4(const float* x, const int* w, const float* sc, float* y, int kpad) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int kwords = kpad / 7;
    const size_t wbase = (size_t)n * kwords, scbase = (size_t)n * (kpad / 16);
    float acc = 0.0f;
    for (int word = 0; word < kwords; word++) {
        const unsigned wv = (unsigned)w[wbase + word];
#pragma unroll
        for (int s = 0; s < 7; s++) {
            const int col = word * 7 + s;
            const float wt = __fmul_rn(hx_e2m1_dec((wv >> (4 * s)) & 15), sc[scbase + col / 16]);
            acc = acc + x[col] * wt;
        }
    }
    y[n] = acc;
}

// One lane's share of a row: words first, first+stride, ...; the seven slots of a word in order,
// each step fma(x, mag*scale, acc) with scale = e4m3(micro)*ts decoded in the kernel
// (kovc.hx:14357-14393, 14639-14679).  micro is four codes per int32, low byte first, row stride
// ceil(kblk/4) words.
__device__ __forceinline__ float hx_row_partial(const float* __restrict__ x, const int* __restrict__ w,
                                                const int* __restrict__ micro, float ts, int row, int kpad,
                                                int first, int stride) {
    const int kwords = kpad / 7, mst = (kpad / 16 + 3) / 4;
    const int* wr = w + (size_t)row * kwords;
    const int* mr = micro + (size_t)row * mst;
    float acc = 0.0f;
    for (int word = first; word < kwords; word += stride) {
        const unsigned wv = (unsigned)wr[word];
        const int col0 = word * 7;
        int blk = col0 >> 4;
        unsigned mw = (unsigned)mr[blk >> 2];
        float scale = __fmul_rn(hx_e4m3_dec((mw >> (8 * (blk & 3))) & 0xFF), ts);
#pragma unroll
        for (int s = 0; s < 7; s++) {
            const int col = col0 + s;
            if ((col >> 4) != blk) {              // a word straddles at most one block boundary
                blk = col >> 4;
                mw = (unsigned)mr[blk >> 2];
                scale = __fmul_rn(hx_e4m3_dec((mw >> (8 * (blk & 3))) & 0xFF), ts);
            }
            acc = fmaf(x[col], __fmul_rn(hx_e2m1_dec((wv >> (4 * s)) & 15), scale), acc);
        }
    }
    return acc;
}

// kovc.hx:14583-14692 -- grid=(ceil(N/8)) block=(32,8): one warp per output row, the lane
// partials are folded with shfl.down 16,8,4,2,1 and lane 0 stores.
extern "C" __global__ void dequant_gemv_warp(const float* x, const int* w_packed, const int* micro,
                                              const float* ts, float* y, int kpad) {
    const int lane = threadIdx.x, row = blockIdx.x * 8 + threadIdx.y;
    float acc = hx_row_partial(x, w_packed, micro, ts[0], row, kpad, lane, 32);
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) acc = acc + __shfl_down_sync(0xffffffffu, acc, d);
    if (lane == 0) y[row] = acc;
}

// kovc.hx:14432-14538 -- grid=(N) block=(256): 256 partials (word stride 256), then an 8-level
// shared-memory tree (kovc.hx:13597-13629).
extern "C" __global__ void dequant_gemv_blockred(const float* x, const int* w_packed, const int* micro,
                                                  const float* ts, float* y, int kpad) {
    __shared__ float red[256];
    const int t = threadIdx.x, row = blockIdx.x;
    red[t] = hx_row_partial(x, w_packed, micro, ts[0], row, kpad, t, 256);
    __syncthreads();
    for (int s = 128; s >= 1; s >>= 1) {
        if (t < s) red[t] = red[t] + red[t + s];
        __syncthreads();
    }
    if (t == 0) y[row] = red[0];
}

// fused_decode_attn_kernel.hx:74-102 -- grid=(NH) block=(DH).  Same online softmax recurrence
// (m seeded -1e8); the score, which the source recomputes in every lane, is computed once per
// position by the block (ascending dot product per lane-chunk is replaced by a warp reduction, the
// result differs from the source only by f32 summation order).
extern "C" __global__ void fused_decode_attn(const float* q, const float* kc, const float* vc, float* out,
                                              const float* sc, int T, int DH, int koff, int grp, int kvstride) {
    __shared__ float s_part[32];
    __shared__ float s_score;
    const int h = blockIdx.x, d = threadIdx.x, nw = (blockDim.x + 31) >> 5;
    const size_t base = (size_t)koff + (size_t)(h / grp) * (size_t)kvstride;
    const float scale = sc[0];
    const float qd = (d < DH) ? q[h * DH + d] : 0.0f;
    float m = -100000000.0f, l = 0.0f, acc = 0.0f;
    for (int t = 0; t < T; t++) {
        float p = (d < DH) ? qd * kc[base + (size_t)t * DH + d] : 0.0f;
        p = hx_warp_sum(p);
        if ((d & 31) == 0) s_part[d >> 5] = p;
        __syncthreads();
        if (d == 0) { float s = 0.0f; for (int i = 0; i < nw; i++) s = s + s_part[i]; s_score = s * scale; }
        __syncthreads();
        const float s = s_score;
        const float mn = s > m ? s : m;
        const float r = __expf(m - mn), pw = __expf(s - mn);
        if (d < DH) acc = acc * r + pw * vc[base + (size_t)t * DH + d];
        l = l * r + pw;
        m = mn;
    }
    if (d < DH) out[h * DH + d] = acc / l;
}

// softmax_causal_offset_kernel.hx:26-56 -- one thread per row; row r covers columns [0, base+r].
extern "C" __global__ void softmax_causal_offset(const float* x, float* y, int rows, int cols, int base) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    const size_t b = (size_t)row * cols;
    int ext = base + row + 1; if (ext > cols) ext = cols;
    float m = x[b];
    for (int j = 1; j < ext; j++) if (x[b + j] > m) m = x[b + j];
    float s = 0.0f;
    for (int j = 0; j < ext; j++) { float e = __expf(x[b + j] - m); y[b + j] = e; s = s + e; }
    for (int j = 0; j < ext; j++) y[b + j] = y[b + j] / s;
    for (int j = ext; j < cols; j++) y[b + j] = 0.0f;
}

// gpu_softmax_causal_kernel.hx:10-39 -- causal row softmax, zeros above the diagonal.
extern "C" __global__ void gpu_softmax_causal(const float* x, float* y, int rows, int cols) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    const size_t b = (size_t)row * cols;
    int ext = row + 1; if (ext > cols) ext = cols;
    float m = x[b];
    for (int j = 1; j < ext; j++) if (x[b + j] > m) m = x[b + j];
    float s = 0.0f;
    for (int j = 0; j < ext; j++) { float e = __expf(x[b + j] - m); y[b + j] = e; s = s + e; }
    for (int j = 0; j < ext; j++) y[b + j] = y[b + j] / s;
    for (int j = ext; j < cols; j++) y[b + j] = 0.0f;
}

// gpu_softmax_row_kernel.hx:11-34 -- one thread per row, three passes.
extern "C" __global__ void gpu_softmax_row(const float* x, float* y, int cols) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    const size_t b = (size_t)row * cols;
    float m = x[b];
    for (int j = 1; j < cols; j++) if (x[b + j] > m) m = x[b + j];
    float s = 0.0f;
    for (int j = 0; j < cols; j++) { float e = __expf(x[b + j] - m); y[b + j] = e; s = s + e; }
    for (int j = 0; j < cols; j++) y[b + j] = y[b + j] / s;
}

// gpu_gemv_abt_kernel.hx:13-24 -- y[n] = sum_j x[j]*w[n*k+j], one thread per output.
extern "C" __global__ void gpu_gemv_abt(const float* x, const float* w, float* y, int k) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const float* wr = w + (size_t)n * k;
    float acc = 0.0f;
    for (int j = 0; j < k; j++) acc = acc + x[j] * wr[j];
    y[n] = acc;
}

// gpu_gemv_ab_kernel.hx:11-21 -- y[n] = sum_t p[t]*m[t*ncols+n].
extern "C" __global__ void gpu_gemv_ab(const float* p, const float* m, float* y, int tlen, int ncols) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    float acc = 0.0f;
    for (int t = 0; t < tlen; t++) acc = acc + p[t] * m[(size_t)t * ncols + n];
    y[n] = acc;
}

// gpu_rmsnorm_fwd_eps_kernel.hx:18-29 -- eps baked to 1e-5, one thread per row.
extern "C" __global__ void gpu_rmsnorm_fwd_eps(const float* x, float* y, const float* w, int cols) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    const size_t b = (size_t)row * cols;
    float ss = 0.0f;
    for (int j = 0; j < cols; j++) ss = ss + x[b + j] * x[b + j];
    const float inv = rsqrtf(ss / (float)cols + 0.00001f);
    for (int j = 0; j < cols; j++) y[b + j] = w[j] * (x[b + j] * inv);
}

// gpu_layernorm_fwd_eps_kernel.hx:9-25 -- population variance, two passes, eps 1e-5.
extern "C" __global__ void gpu_layernorm_fwd_eps(const float* x, float* y, const float* gamma, const float* beta, int cols) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    const size_t b = (size_t)row * cols;
    float sm = 0.0f;
    for (int j = 0; j < cols; j++) sm = sm + x[b + j];
    const float mean = sm / (float)cols;
    float vs = 0.0f;
    for (int j = 0; j < cols; j++) vs = vs + (x[b + j] - mean) * (x[b + j] - mean);
    const float inv = rsqrtf(vs / (float)cols + 0.00001f);
    for (int j = 0; j < cols; j++) y[b + j] = gamma[j] * ((x[b + j] - mean) * inv) + beta[j];
}

// gpu_rope_rot_kernel.hx:23-38 -- rotate_half pairs (i, i+half), in place, one thread per row.
extern "C" __global__ void gpu_rope_rot(float* q, const float* cosT, const float* sinT, int half) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    const size_t b = (size_t)row * (half + half), tb = (size_t)row * half;
    for (int i = 0; i < half; i++) {
        const float a = q[b + i], c = q[b + half + i], cv = cosT[tb + i], sv = sinT[tb + i];
        q[b + i] = a * cv - c * sv;
        q[b + half + i] = c * cv + a * sv;
    }
}

// gpu_silu_mul_kernel.hx:20-31 -- one thread per element, no bounds guard (exact tiling).
extern "C" __global__ void gpu_silu_mul(const float* g, const float* u, float* y, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const float gi = g[i];
    const float sgn = gi < 0.0f ? -1.0f : 1.0f;
    const float e = __expf(0.0f - sgn * gi);
    const float th = sgn * ((1.0f - e) / (1.0f + e));
    y[i] = gi * (0.5f * (1.0f + th)) * u[i];
}

// gpu_gelu_stable_kernel.hx:15-28 -- gelu_new with the overflow-safe tanh.
extern "C" __global__ void gpu_gelu_stable(const float* x, float* y, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const float xi = x[i];
    const float inner = 0.7978846f * (xi + (0.044715f * (xi * xi * xi)));
    const float two = 2.0f * inner;
    const float sgn = inner < 0.0f ? -1.0f : 1.0f;
    const float e = __expf(0.0f - sgn * two);
    const float th = sgn * ((1.0f - e) / (1.0f + e));
    y[i] = 0.5f * xi * (1.0f + th);
}

// gpu_add_bias_rowbcast_kernel.hx:17-27 -- y[i] += bias[i mod cols], guarded by n.
extern "C" __global__ void gpu_add_bias_rowbcast(float* y, const float* bias, int n, int cols) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = y[i] + bias[i % cols];
}

// vector_add_kernel.hx:18-22 and gpu_scale_rt_kernel.hx:9-13 -- exact tiling, no guard.
extern "C" __global__ void vector_add(const float* a, const float* b, float* c, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    c[i] = a[i] + b[i];
}
extern "C" __global__ void gpu_scale_rt(float* a, const float* s, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    a[i] = a[i] * s[0];
}

// tiled_matmul_kernel.hx:17-20 / tiled_matmul_abt_kernel.hx:20-23 -- grid=(N/64, M/64)
// block=(16,16): a 64x64 tile per CTA, 4x4 outputs per thread, k in steps of 8 ascending with one
// f32 accumulator per output (kovc.hx:13061-13200, 13424-13520).  M, N multiples of 64, K of 8.
template <bool BT>
__device__ __forceinline__ void hx_tile_mm(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                                           int M, int K, int N) {
    __shared__ float As[8][64 + 4];
    __shared__ float Bs[8][64 + 4];
    const int tx = threadIdx.x, ty = threadIdx.y, tid = ty * 16 + tx;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 8) {
        // 512 elements per operand tile, two per thread
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int e = tid + i * 256;
            { const int r = e >> 3, kk = e & 7; As[kk][r] = a[(size_t)(m0 + r) * K + k0 + kk]; }
            if (BT) { const int r = e >> 3, kk = e & 7; Bs[kk][r] = b[(size_t)(n0 + r) * K + k0 + kk]; }
            else    { const int kk = e >> 6, cc = e & 63; Bs[kk][cc] = b[(size_t)(k0 + kk) * N + n0 + cc]; }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { av[i] = As[kk][ty * 4 + i]; bv[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) c[(size_t)(m0 + ty * 4 + i) * N + n0 + tx * 4 + j] = acc[i][j];
}
extern "C" __global__ void tiled_matmul(const float* a, const float* b, float* c, int M, int K, int N) {
    hx_tile_mm<false>(a, b, c, M, K, N);
}
extern "C" __global__ void tiled_matmul_abt(const float* a, const float* b, float* c, int M, int K, int N) {
    hx_tile_mm<true>(a, b, c, M, K, N);
}

// ---- library-side launcher over the committed layout (guards the row count) --------------------
#ifndef HX_ENTRIES_ONLY
__global__ void __launch_bounds__(256) k_gemv_committed(const float* x, const int* w_packed, const int* micro,
                                                         const float* ts, float* y, int kpad, int N) {
    const int lane = threadIdx.x, row = blockIdx.x * 8 + threadIdx.y;
    if (row >= N) return;                          // whole warps leave together
    float acc = hx_row_partial(x, w_packed, micro, ts[0], row, kpad, lane, 32);
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) acc = acc + __shfl_down_sync(0xffffffffu, acc, d);
    if (lane == 0) y[row] = acc;
}

HX_API int hx_gemv_nvfp4(const float* x, const int32_t* words, const int32_t* micro4, const float* ts,
                         float* y, int N, int Kpad, void* stream) {
    HX_CHECK_ARG(x && words && micro4 && ts && y && N > 0 && Kpad > 0 && Kpad % 112 == 0);
    k_gemv_committed<<<(N + 7) / 8, dim3(32, 8), 0, (cudaStream_t)stream>>>(x, words, micro4, ts, y, Kpad, N);
    HX_COUNT_LAUNCH(1);
    HX_CUDA(cudaGetLastError());
    return HX_OK;
}
#endif
