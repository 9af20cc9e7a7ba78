// hx_quant.cu -- NVFP4 forward quantizer, dequantizer and layout converters on the GPU.
//
// Reference: nvfp4_quantize_tensor / nvfp4_host_dequant, helixc/runtime/gpt2_pack.c:350-387;
// v3_dequant_packed / v3_pack_micro, helixc/runtime/gpt2_infer.c:109-122, 2151-2161.
//
// The quantizer is bit-exact with the reference: the five float operations that decide a code
// (amax/2688, ts*6, bamax/(ts*6), decode(micro)*ts, v/eff) are issued as separately rounded IEEE
// operations (__fdiv_rn / __fmul_rn are never contracted), the rest is compares and integers.
//
// Data flow (HBM-bound): pass 1 reads the tensor once for the per-tensor amax; pass 2 reads it again
// (from L2 when the tensor is smaller than L2) and writes 4.57 bits of codes + 0.5 bits of scale
// per element.
#include "hx_common.cuh"

unsigned long long g_hx_launches = 0;

// ------------------------------------------------------------------------------------------------
// pass 1: amax over rows*K.  Non-negative floats order like their bit patterns, so the final
// combine is an integer atomicMax.  NaN never wins (the reference's `a > amax` is false for NaN).
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_amax(const float* __restrict__ w, size_t n, unsigned* __restrict__ out_bits) {
    float m = 0.0f;
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    if ((((uintptr_t)w) & 15) == 0) {
        const float4* w4 = reinterpret_cast<const float4*>(w);
        size_t n4 = n / 4;
        for (size_t i = tid; i < n4; i += nth) {
            float4 v = __ldg(w4 + i);
            // fmaxf returns the non-NaN operand, like the reference's compare-and-keep
            m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
        for (size_t i = n4 * 4 + tid; i < n; i += nth) m = fmaxf(m, fabsf(w[i]));
    } else {
        for (size_t i = tid; i < n; i += nth) m = fmaxf(m, fabsf(w[i]));
    }
    m = hx_warp_max(m);
    __shared__ float sm[8];
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 8) {
        m = sm[threadIdx.x];
#pragma unroll
        for (int d = 4; d >= 1; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffu, m, d));
        if (threadIdx.x == 0) atomicMax(out_bits, __float_as_uint(m));
    }
}

// ------------------------------------------------------------------------------------------------
// pass 2: one CTA iteration covers a "span" of 1792 columns of one row (112 blocks = 256 words, the
// largest span below 2048 on which 16-element blocks and 7-code words both end).  448 threads:
// thread t holds columns 4t..4t+3 (one float4, fully coalesced); four neighbouring threads form a
// 16-block, its amax comes from two shuffles.  The 4-bit codes go to shared memory as one dense
// nibble stream; threads 0..255 then cut 28-bit words out of it with a funnel shift.
// ------------------------------------------------------------------------------------------------
#define QSPAN 1792
#define QTHREADS 448

__global__ void __launch_bounds__(QTHREADS) k_quantize(const float* __restrict__ w, int rows, int K, int Kpad,
                                                        const unsigned* __restrict__ amax_bits,
                                                        int32_t* __restrict__ words, uint8_t* __restrict__ micro,
                                                        float* __restrict__ sc, float* __restrict__ ts_out) {
    __shared__ uint32_t nib[QSPAN / 8 + 2];   // dense nibble stream of the span (+ slack for the funnel)
    const int t = threadIdx.x;
    const int spans = (Kpad + QSPAN - 1) / QSPAN;
    const int kwords = Kpad / 7, kblk = Kpad / 16;
    float amax = __uint_as_float(*amax_bits);
    float ts = __fdiv_rn(amax, 2688.0f);          // 6.0f*448.0f folds to 2688.0f in the reference build
    if (!(ts > 0.0f)) ts = 1.0f;                  // `if (ts <= 0) ts = 1`; amax is never NaN
    if (blockIdx.x == 0 && t == 0 && ts_out) *ts_out = ts;
    const float ts6 = __fmul_rn(ts, 6.0f);
    const bool vec = ((K & 3) == 0) && ((((uintptr_t)w) & 15) == 0);
    if (t < 2) nib[QSPAN / 8 + t] = 0;

    for (long item = blockIdx.x; item < (long)rows * spans; item += gridDim.x) {
        const int r = (int)(item / spans), sp = (int)(item % spans);
        const int col0 = sp * QSPAN + 4 * t;
        const float* wr = w + (size_t)r * K;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (col0 < Kpad) {
            if (vec && col0 + 3 < K) v = __ldg(reinterpret_cast<const float4*>(wr + col0));
            else {
                if (col0 + 0 < K) v.x = wr[col0 + 0];
                if (col0 + 1 < K) v.y = wr[col0 + 1];
                if (col0 + 2 < K) v.z = wr[col0 + 2];
                if (col0 + 3 < K) v.w = wr[col0 + 3];
            }
        }
        // block amax with the reference's compare (NaN never replaces the running maximum)
        float bm = 0.0f, a;
        a = fabsf(v.x); if (a > bm) bm = a;
        a = fabsf(v.y); if (a > bm) bm = a;
        a = fabsf(v.z); if (a > bm) bm = a;
        a = fabsf(v.w); if (a > bm) bm = a;
        a = __shfl_xor_sync(0xffffffffu, bm, 1); if (a > bm) bm = a;
        a = __shfl_xor_sync(0xffffffffu, bm, 2); if (a > bm) bm = a;
        const int mc = hx_e4m3_enc(__fdiv_rn(bm, ts6));
        const float eff = __fmul_rn(hx_e4m3_dec(mc), ts);
        uint32_t c4 = 0;
        if (eff > 0.0f) {
            c4 = (uint32_t)hx_e2m1_enc(__fdiv_rn(v.x, eff)) | ((uint32_t)hx_e2m1_enc(__fdiv_rn(v.y, eff)) << 4) |
                 ((uint32_t)hx_e2m1_enc(__fdiv_rn(v.z, eff)) << 8) | ((uint32_t)hx_e2m1_enc(__fdiv_rn(v.w, eff)) << 12);
        }
        // two neighbouring threads share one 32-bit word of the nibble stream
        uint32_t other = __shfl_xor_sync(0xffffffffu, c4, 1);
        __syncthreads();                          // previous iteration's readers are done
        if ((t & 1) == 0) nib[t >> 1] = c4 | (other << 16);
        if ((t & 3) == 0 && col0 < Kpad) {
            const size_t bi = (size_t)r * kblk + (size_t)(col0 >> 4);
            if (micro) micro[bi] = (uint8_t)mc;
            if (sc) sc[bi] = eff;
        }
        __syncthreads();
        if (t < 256) {
            const int wi = sp * 256 + t;          // word index in the row
            if (wi < kwords) {
                const int bit = 28 * t;
                const uint32_t lo = nib[bit >> 5], hi = nib[(bit >> 5) + 1];
                const uint32_t word = __funnelshift_r(lo, hi, bit & 31) & 0x0FFFFFFFu;
                words[(size_t)r * kwords + wi] = (int32_t)word;
            }
        }
    }
}

HX_API int hx_kpad(int K) { return ((K + 111) / 112) * 112; }
HX_API int hx_kd(int K) { return ((K + 63) / 64) * 64; }

// Scratch for the tensor's amax: 64 words per device handed out in turn, so calls that overlap on different
// streams do not share a word (up to 64 of them in flight per device); zeroed before every use on the caller's stream.
static unsigned* amax_scratch() {
    static unsigned* p[64] = {0};
    static std::atomic<unsigned> turn{0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!p[dev] && cudaMalloc(&p[dev], 256) != cudaSuccess) return nullptr;
    return p[dev] + (turn.fetch_add(1u) & 63u);
}

HX_API int hx_quantize_nvfp4(const float* w, int rows, int K, int32_t* words, uint8_t* micro, float* sc,
                             float* ts, void* stream) {
    HX_CHECK_ARG(w && words && rows > 0 && K > 0);
    cudaStream_t st = (cudaStream_t)stream;
    unsigned* am = amax_scratch();
    if (!am) return hx_fail(HX_ERR_CUDA, "no CUDA device / scratch allocation failed");
    const int Kpad = hx_kpad(K);
    HX_CUDA(cudaMemsetAsync(am, 0, 4, st));
    size_t n = (size_t)rows * K;
    int g1 = (int)((n / 4 + 255) / 256); if (g1 > 148 * 8) g1 = 148 * 8; if (g1 < 1) g1 = 1;
    k_amax<<<g1, 256, 0, st>>>(w, n, am);
    long items = (long)rows * ((Kpad + QSPAN - 1) / QSPAN);
    int g2 = (int)(items < 148L * 16 ? items : 148L * 16);
    k_quantize<<<g2, QTHREADS, 0, st>>>(w, rows, K, Kpad, am, words, micro, sc, ts);
    HX_COUNT_LAUNCH(2);
    HX_CUDA(cudaGetLastError());
    return HX_OK;
}

// ------------------------------------------------------------------------------------------------
// Quantizer that allocates nothing.
//
// hx_quantize_nvfp4 takes its amax word from cudaMalloc on its first call per device.  Some hosts cannot
// accept that: a worker that gave all device memory to its own arena when it started (the reference's
// worker sizes every buffer once and never allocates inside its token loop), or a service that shares the
// GPU with other streams and cannot afford the device-wide stall an allocation implies.  This variant finds
// the tensor's amax through a scratch array that is part of the library image: one word per row, then one
// word for the whole tensor.  The array is obtained with cudaGetSymbolAddress, which only looks a symbol
// up; it is looked up once per device and cached.
//
//   * size limit: rows <= HX_NOALLOC_MAX_ROWS (1 MiB of row maxima + 256 B); more rows are refused.
//   * the first call on a device performs the symbol look-up (and loads the library's device code if
//     nothing did before); make that call during start-up, before any stream capture.
//   * the array is shared by every caller of the process and keeps what the last call left; nothing has to
//     start at zero, because a call writes words [0, rows) and the tensor word before it reads them and
//     never reads beyond.
//   * two calls that overlap in time on one device (different streams or threads) race on the array; calls
//     on one stream are ordered by the stream.
// ------------------------------------------------------------------------------------------------
#define HX_NOALLOC_MAX_ROWS (1 << 18)
static __device__ __align__(256) unsigned g_noalloc_scratch[HX_NOALLOC_MAX_ROWS + 64];

// amax of each row: G threads per row (32 or 256), rows dealt to groups grid-stride.
template <int G>
__global__ void __launch_bounds__(256) k_row_amax(const float* __restrict__ w, int rows, int K, unsigned* __restrict__ row_bits) {
    const int groups_per_block = 256 / G, gl = threadIdx.x / G, t = threadIdx.x % G;
    __shared__ float sm[8];
    for (int r = blockIdx.x * groups_per_block + gl; r < rows; r += gridDim.x * groups_per_block) {   // uniform per block when G = 256
        const float* wr = w + (size_t)r * K;
        float m = 0.0f;
        if (((((uintptr_t)wr) & 15) == 0)) {
            const float4* w4 = reinterpret_cast<const float4*>(wr);
            const int n4 = K / 4;
            for (int i = t; i < n4; i += G) {
                const float4 v = __ldg(w4 + i);
                m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
            for (int i = n4 * 4 + t; i < K; i += G) m = fmaxf(m, fabsf(wr[i]));
        } else {
            for (int i = t; i < K; i += G) m = fmaxf(m, fabsf(wr[i]));
        }
        m = hx_warp_max(m);
        if (G == 32) {
            if (t == 0) row_bits[r] = __float_as_uint(m);
        } else {
            if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = m;
            __syncthreads();
            if (threadIdx.x == 0) {
                float mm = sm[0];
#pragma unroll
                for (int i = 1; i < 8; i++) mm = fmaxf(mm, sm[i]);
                row_bits[r] = __float_as_uint(mm);
            }
            __syncthreads();
        }
    }
}

// max of the row words -> tensor_bits[0]; one block.  Non-negative floats order like their bit patterns.
__global__ void __launch_bounds__(1024) k_fold_amax(const unsigned* __restrict__ row_bits, int rows, unsigned* __restrict__ tensor_bits) {
    unsigned m = 0u;
    for (int i = threadIdx.x; i < rows; i += 1024) m = max(m, row_bits[i]);
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, d));
    __shared__ unsigned sm[32];
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = sm[threadIdx.x];
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, d));
        if (threadIdx.x == 0) tensor_bits[0] = m;
    }
}

// Address of the library's scratch array on the current device (looked up once per device).
static int noalloc_scratch(unsigned** out) {
    static unsigned* cached[64] = {0};
    int dev = 0;
    HX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return hx_fail(HX_ERR_ARG, "device index %d not supported", dev);
    if (!cached[dev]) {
        unsigned* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || !ptr) return hx_fail(HX_ERR_CUDA, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return HX_OK;
}

HX_API int hx_noalloc_max_rows(void) { return HX_NOALLOC_MAX_ROWS; }

HX_API int hx_quantize_nvfp4_noalloc(const float* w, int rows, int K, int32_t* words, uint8_t* micro, float* sc,
                                     float* ts, void* stream) {
    HX_CHECK_ARG(w && words && rows > 0 && K > 0);
    if (rows > HX_NOALLOC_MAX_ROWS)
        return hx_fail(HX_ERR_ARG, "hx_quantize_nvfp4_noalloc: %d rows exceed the built-in scratch of %d rows; "
                                   "quantize the tensor with hx_quantize_nvfp4", rows, HX_NOALLOC_MAX_ROWS);
    cudaStream_t st = (cudaStream_t)stream;
    unsigned* scr = nullptr;
    int rc = noalloc_scratch(&scr); if (rc) return rc;
    unsigned* tensor_bits = scr + HX_NOALLOC_MAX_ROWS;
    const int Kpad = hx_kpad(K);
    if (K >= 2048) {
        int g = rows < 148 * 8 ? rows : 148 * 8;
        k_row_amax<256><<<g, 256, 0, st>>>(w, rows, K, scr);
    } else {
        int g = (rows + 7) / 8; if (g > 148 * 8) g = 148 * 8;
        k_row_amax<32><<<g, 256, 0, st>>>(w, rows, K, scr);
    }
    k_fold_amax<<<1, 1024, 0, st>>>(scr, rows, tensor_bits);
    long items = (long)rows * ((Kpad + QSPAN - 1) / QSPAN);
    int g2 = (int)(items < 148L * 16 ? items : 148L * 16);
    k_quantize<<<g2, QTHREADS, 0, st>>>(w, rows, K, Kpad, tensor_bits, words, micro, sc, ts);
    HX_COUNT_LAUNCH(3);
    HX_CUDA(cudaGetLastError());
    return HX_OK;
}

HX_API int hx_quantize_nvfp4_host(const float* w, int rows, int K, int32_t* words, uint8_t* micro, float* sc,
                                  float* ts) {
    HX_CHECK_ARG(w && words && rows > 0 && K > 0);
    const int Kpad = hx_kpad(K);
    const size_t nw = (size_t)rows * K * 4, nq = (size_t)rows * (Kpad / 7) * 4, nm = (size_t)rows * (Kpad / 16);
    float* dw = nullptr; int32_t* dq = nullptr; uint8_t* dm = nullptr; float* ds = nullptr; float* dts = nullptr;
    int rc = HX_OK;
    auto cleanup = [&]() { cudaFree(dw); cudaFree(dq); cudaFree(dm); cudaFree(ds); cudaFree(dts); };
#define HXQ(call) do { cudaError_t _e = (call); if (_e != cudaSuccess) { cleanup(); return hx_fail(HX_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(_e)); } } while (0)
    HXQ(cudaMalloc(&dw, nw)); HXQ(cudaMalloc(&dq, nq)); HXQ(cudaMalloc(&dm, nm)); HXQ(cudaMalloc(&dts, 4));
    if (sc) HXQ(cudaMalloc(&ds, nm * 4));
    HXQ(cudaMemcpy(dw, w, nw, cudaMemcpyHostToDevice));
    rc = hx_quantize_nvfp4(dw, rows, K, dq, dm, ds, dts, nullptr);
    if (rc) { cleanup(); return rc; }
    HXQ(cudaMemcpy(words, dq, nq, cudaMemcpyDeviceToHost));
    if (micro) HXQ(cudaMemcpy(micro, dm, nm, cudaMemcpyDeviceToHost));
    if (sc) HXQ(cudaMemcpy(sc, ds, nm * 4, cudaMemcpyDeviceToHost));
    if (ts) HXQ(cudaMemcpy(ts, dts, 4, cudaMemcpyDeviceToHost));
#undef HXQ
    cleanup();
    return HX_OK;
}

// ------------------------------------------------------------------------------------------------
// dequant to f32: out[r,col] = sign*mag*(e4m3(micro)*ts), or sign*mag*sc with collapsed scales.
// One thread per 7-code word keeps the word reads coalesced.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_dequant(const int32_t* __restrict__ words, const uint8_t* __restrict__ micro,
                                                  const float* __restrict__ ts, const float* __restrict__ sc,
                                                  float* __restrict__ out, int rows, int Kpad) {
    const int kwords = Kpad / 7, kblk = Kpad / 16;
    const float tsv = ts ? *ts : 1.0f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)rows * kwords;
         i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / kwords), wd = (int)(i % kwords);
        uint32_t wv = (uint32_t)words[i];
#pragma unroll
        for (int s = 0; s < 7; s++) {
            const int col = wd * 7 + s;
            const int code = (wv >> (4 * s)) & 15;
            const size_t bi = (size_t)r * kblk + (col >> 4);
            const float eff = sc ? sc[bi] : __fmul_rn(hx_e4m3_dec(micro[bi]), tsv);
            out[(size_t)r * Kpad + col] = __fmul_rn(hx_e2m1_dec(code), eff);
        }
    }
}

HX_API int hx_dequant_nvfp4(const int32_t* words, const uint8_t* micro, const float* ts, const float* sc,
                            float* out, int rows, int Kpad, void* stream) {
    HX_CHECK_ARG(words && out && rows > 0 && Kpad > 0 && Kpad % 112 == 0);
    HX_CHECK_ARG(sc || (micro && ts));
    size_t n = (size_t)rows * (Kpad / 7);
    int g = (int)((n + 255) / 256); if (g > 148 * 16) g = 148 * 16;
    k_dequant<<<g, 256, 0, (cudaStream_t)stream>>>(words, micro, ts, sc, out, rows, Kpad);
    HX_COUNT_LAUNCH(1);
    HX_CUDA(cudaGetLastError());
    return HX_OK;
}

// micro bytes -> 4 per int32, low byte first, row stride ceil(kblk/4) words.
__global__ void k_pack_micro(const uint8_t* __restrict__ micro, int rows, int kblk, int32_t* __restrict__ dst) {
    const int mst = (kblk + 3) / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)rows * mst;
         i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / mst), wi = (int)(i % mst);
        uint32_t v = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int b = wi * 4 + j;
            if (b < kblk) v |= (uint32_t)micro[(size_t)r * kblk + b] << (8 * j);
        }
        dst[i] = (int32_t)v;
    }
}

HX_API int hx_pack_micro(const uint8_t* micro, int rows, int kblk, int32_t* dst, void* stream) {
    HX_CHECK_ARG(micro && dst && rows > 0 && kblk > 0);
    size_t n = (size_t)rows * ((kblk + 3) / 4);
    int g = (int)((n + 255) / 256); if (g > 148 * 16) g = 148 * 16;
    k_pack_micro<<<g, 256, 0, (cudaStream_t)stream>>>(micro, rows, kblk, dst);
    HX_COUNT_LAUNCH(1);
    HX_CUDA(cudaGetLastError());
    return HX_OK;
}

// ------------------------------------------------------------------------------------------------
// committed layout -> dense decode layout: per row Kd/2 code bytes (two codes per byte, low nibble
// first) and Kd/16 scale bytes, Kd = K rounded up to 64.  One thread per 8 codes (one u32 out).
// Columns at or beyond K are written as zero codes / zero scales.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_repack_d16(const int32_t* __restrict__ words, const uint8_t* __restrict__ micro,
                                                     int rows, int K, int Kpad, uint32_t* __restrict__ codes,
                                                     uint8_t* __restrict__ scales, int row_mul, int row_off) {
    const int Kd = ((K + 63) / 64) * 64;
    const int kwords = Kpad / 7, kblk = Kpad / 16, c8 = Kd / 8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)rows * c8;
         i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / c8), g = (int)(i % c8);
        uint32_t o = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int col = g * 8 + j;
            uint32_t code = 0;
            if (col < K) {
                const int wd = col / 7, s = col - wd * 7;
                code = ((uint32_t)words[(size_t)r * kwords + wd] >> (4 * s)) & 15u;
            }
            o |= code << (4 * j);
        }
        const size_t dr = (size_t)r * row_mul + row_off;     // destination row (fused / interleaved tensors)
        codes[dr * c8 + g] = o;
        if ((g & 1) == 0) {
            const int b = g >> 1;
            scales[dr * (Kd / 16) + b] = (b < kblk && b * 16 < K) ? micro[(size_t)r * kblk + b] : (uint8_t)0;
        }
    }
}

HX_API int hx_repack_d16(const int32_t* words, const uint8_t* micro, int rows, int K, int Kpad,
                         uint8_t* codes, uint8_t* scales, void* stream) {
    HX_CHECK_ARG(words && micro && codes && scales && rows > 0 && K > 0 && Kpad == hx_kpad(K));
    size_t n = (size_t)rows * (hx_kd(K) / 8);
    int g = (int)((n + 255) / 256); if (g > 148 * 16) g = 148 * 16;
    k_repack_d16<<<g, 256, 0, (cudaStream_t)stream>>>(words, micro, rows, K, Kpad, (uint32_t*)codes, scales, 1, 0);
    HX_COUNT_LAUNCH(1);
    HX_CUDA(cudaGetLastError());
    return HX_OK;
}

// Source row r lands on destination row r*row_mul + row_off (q|k|v stacking, gate/up interleave).
void hx_repack_rows(const int32_t* words, const uint8_t* micro, int rows, int K, int Kpad, uint8_t* codes,
                    uint8_t* scales, int row_mul, int row_off, cudaStream_t st) {
    size_t n = (size_t)rows * (hx_kd(K) / 8);
    int g = (int)((n + 255) / 256); if (g > 148 * 16) g = 148 * 16;
    k_repack_d16<<<g, 256, 0, st>>>(words, micro, rows, K, Kpad, (uint32_t*)codes, scales, row_mul, row_off);
    HX_COUNT_LAUNCH(1);
}
