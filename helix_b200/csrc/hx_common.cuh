// hx_common.cuh -- shared declarations of libhelix_b200: error plumbing, the NVFP4 codecs
// (host + device) and small device helpers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <math.h>
#include "../../include/helix_b200.h"

#define HX_API extern "C" __attribute__((visibility("default")))

// ---- error plumbing -----------------------------------------------------------------------------
void hx_set_error(const char* fmt, ...);
int  hx_fail(int code, const char* fmt, ...);

#define HX_CUDA(call)                                                                         \
    do {                                                                                      \
        cudaError_t _e = (call);                                                              \
        if (_e != cudaSuccess)                                                                \
            return hx_fail(HX_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(_e), \
                           __FILE__, __LINE__);                                               \
    } while (0)

#define HX_CHECK_ARG(cond)                                                                    \
    do {                                                                                      \
        if (!(cond)) return hx_fail(HX_ERR_ARG, "bad argument: %s (%s:%d)", #cond, __FILE__, __LINE__); \
    } while (0)

// A function attribute belongs to the device that is current when it is set, so "done once" is tracked per
// device: returns true the first time it is called for `seen` on the current device (devices 0..63).
#include <atomic>
static inline bool hx_first_on_device(std::atomic<unsigned long long>& seen) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev > 63) return true;
    const unsigned long long bit = 1ull << dev;
    return (seen.fetch_or(bit) & bit) == 0;
}

// Count of kernels this library launched (reported by the benchmark as gpu_launches).
extern unsigned long long g_hx_launches;
#define HX_COUNT_LAUNCH(n) (g_hx_launches += (n))

// ---- codecs -------------------------------------------------------------------------------------
// E2M1 magnitudes {0,.5,1,1.5,2,3,4,6}: as_float(mag3 << 22) is mag * 2^-126 (the e=0 codes land on
// f32 subnormals), so one exact multiply by 2^126 decodes all eight without a table.
__host__ __device__ __forceinline__ float hx_e2m1_mag(int c3) {
#ifdef __CUDA_ARCH__
    return __uint_as_float((unsigned)(c3 & 7) << 22) * 8.507059173023462e37f;   // 2^126
#else
    const float MAG[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    return MAG[c3 & 7];
#endif
}
__host__ __device__ __forceinline__ float hx_e2m1_dec(int code) {
    float m = hx_e2m1_mag(code);
    return (code & 8) ? -m : m;
}

// Threshold encoder; a tie takes the smaller magnitude, magnitude 0 never carries a sign, NaN maps
// to code 7 (every comparison false).  Reference: e2m1_encode, gpt2_pack.c:306-318.
__host__ __device__ __forceinline__ int hx_e2m1_enc(float v) {
    float a = v < 0.0f ? -v : v;
    if (a <= 0.25f) return 0;
    int mag = 1 + (int)!(a <= 0.75f) + (int)!(a <= 1.25f) + (int)!(a <= 1.75f) + (int)!(a <= 2.5f) +
              (int)!(a <= 3.5f) + (int)!(a <= 5.0f);
    return mag | (v < 0.0f ? 8 : 0);
}

// E4M3 decode for non-NaN codes: (1+m/8)*2^(e-7), subnormals (m/8)*2^-6.  Built from the bit
// pattern: as_float((c & 0x7F) << 20) is the value times 2^-120 (e=0 lands on f32 subnormals).
// Reference: e4m3_decode, gpt2_pack.c:333-338.
__host__ __device__ __forceinline__ float hx_e4m3_dec(int c) {
    if ((c & 0x7F) == 0x7F) {
#ifdef __CUDA_ARCH__
        return __uint_as_float(0x7FC00000u);
#else
        return nanf("");
#endif
    }
    uint32_t bits = (uint32_t)(c & 0x7F) << 20;
    float mag;
#ifdef __CUDA_ARCH__
    mag = __uint_as_float(bits) * 1.329227995784916e36f;   // 2^120, exact
#else
    float f; memcpy(&f, &bits, 4); mag = f * 1.329227995784916e36f;
#endif
    return (c & 0x80) ? -mag : mag;
}

// E4M3 encode of v with the reference's semantics: the nearest of the 254 non-NaN codes by
// |decode(c) - v| evaluated in f32, the first (lowest) code on a tie, code 0 when no distance is
// below 1e30.  For 0 <= v <= 512 (everything the quantizer can produce: the ratio never exceeds
// 448 by more than rounding) the winner is found in closed form: values are monotonic in the code
// and the distances to the two neighbours are exact (Sterbenz), so the rule is "round to nearest, a
// tie goes to the lower code".  Outside that range f32 rounding of the distances themselves creates
// ties between far-apart codes, so the search is run as written.
// Reference: e4m3_encode, gpt2_pack.c:339-343.
__host__ __device__ __forceinline__ int hx_e4m3_enc_search(float v) {
    int best = 0; float bd = 1.0e30f;
    for (int c = 0; c < 256; c++) {
        if ((c & 0x7F) == 0x7F) continue;
        float d = hx_e4m3_dec(c) - v; if (d < 0) d = -d;
        if (d < bd) { bd = d; best = c; }
    }
    return best;
}
__host__ __device__ __forceinline__ int hx_e4m3_enc(float v) {
    if (!(v >= 0.0f && v <= 512.0f)) return hx_e4m3_enc_search(v);   // negative, huge or NaN: rare
    if (v >= 448.0f) return 0x7E;
    if (v < 0.015625f) {                           // below 2^-6: subnormal codes, step 2^-9
        const float t = v * 512.0f;                // exact
        const int k = (int)t;
        return k + ((t - (float)k) > 0.5f ? 1 : 0);   // 8 rolls into code 0x08 = 2^-6
    }
    uint32_t bits;
#ifdef __CUDA_ARCH__
    bits = __float_as_uint(v);
#else
    memcpy(&bits, &v, 4);
#endif
    const int e = (int)(bits >> 23) - 127 + 7;     // 1..15
    const uint32_t man = bits & 0x7FFFFFu;
    int c = (e << 3) | (int)(man >> 20);
    if ((man & 0xFFFFFu) > 0x80000u) c += 1;       // above the midpoint; carries into the exponent
    return c > 0x7E ? 0x7E : c;
}

// ---- device helpers -----------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ float hx_warp_sum(float v) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}
__device__ __forceinline__ float hx_warp_max(float v) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}
// Programmatic dependent launch: wait for the kernels this one depends on / let dependents start.
__device__ __forceinline__ void hx_grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void hx_grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif
