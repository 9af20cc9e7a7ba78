/* hx_oracle.c -- CPU restatement of the Helix NVFP4 quantized-inference path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: only the test suite,
 * the smoke entry and the benchmark's CPU-baseline / reference legs may build, load or call it.
 * Nothing in the shipped library links against it and it must never be used as a fallback.
 *
 * Every function restates, in plain C, the algorithm of the reference function cited beside it
 * (paths are relative to the Helix source tree).  Parity status: the codecs, the quantizer, the
 * host dequantizer, the micro-scale re-layout, the container layout and SHA-256 are PINNED against
 * the reference's own self-tests / known answers and against the reference sources compiled
 * unmodified (see oracle/Makefile, target `ref`).  The model-level forward (RMSNorm / RoPE / GQA
 * attention / SwiGLU sequencing) restates helixc/runtime/gpt2_infer.c and the kernel sources under
 * helixc/examples and is PINNED by the reference's own GPU worker: gpt2_infer.c compiled unmodified,
 * driving PTX emitted by the reference's own compiler (oracle/mint_ref_ptx.py), was run on a B200 on
 * seeded models; its prefill logits are committed as tests/golden/ref_worker_logits.npz and
 * reproduced by orc_model_prefill to 2e-5 (tests/test_oracle_golden.py), and its fused decode path
 * yields orc_model_generate's tokens (tests/test_ref_worker_gpu.py).
 *
 * Build: gcc -O2 -fopenmp -shared -fPIC (no -march, no -ffast-math: the quantizer's float ops must
 * stay separately rounded, exactly as the reference's plain -O2 x86-64 build rounds them).
 */
#define _GNU_SOURCE
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <stdio.h>
#include <math.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <fcntl.h>
#include <unistd.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------------
 * Codecs.  helixc/runtime/gpt2_pack.c:291-343 (same functions appear in cuda_launch.c:208-228 and
 * gpt2_infer.c:102-107).
 * ---------------------------------------------------------------------------------------------- */

/* E2M1: 1 sign, 2 exponent, 1 mantissa bit.  gpt2_pack.c:291-295. */
ORC_API float orc_e2m1_decode(int code) {
    static const float MAG[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float m = MAG[code & 7];
    return (code & 8) ? -m : m;
}

/* Nearest of the 16 values, first minimum wins.  gpt2_pack.c:297-301. */
ORC_API int orc_e2m1_encode_ref(float v) {
    int best = 0;
    float bestd = 1.0e30f;
    for (int c = 0; c < 16; c++) {
        float d = orc_e2m1_decode(c) - v;
        if (d < 0) d = -d;
        if (d < bestd) { bestd = d; best = c; }
    }
    return best;
}

/* Threshold form: midpoints compare with <= so a tie takes the smaller magnitude; a magnitude of
 * zero never carries the sign bit.  gpt2_pack.c:306-318. */
ORC_API int orc_e2m1_encode(float v) {
    static const float MID[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
    float a = v < 0.0f ? -v : v;
    int mag = 7;
    for (int i = 0; i < 7; i++) if (a <= MID[i]) { mag = i; break; }
    if (mag == 0) return 0;
    return mag | (v < 0.0f ? 8 : 0);
}

/* E4M3 (bias 7, S.1111.111 is NaN, no infinities).  gpt2_pack.c:333-338. */
ORC_API float orc_e4m3_decode(int c) {
    int s = (c >> 7) & 1, e = (c >> 3) & 15, m = c & 7;
    if (e == 15 && m == 7) return nanf("");
    float mag = (e == 0) ? ((float)m / 8.0f) * ldexpf(1.0f, -6)
                         : (1.0f + (float)m / 8.0f) * ldexpf(1.0f, e - 7);
    return s ? -mag : mag;
}

/* Exhaustive nearest search over the 254 non-NaN codes in code order; the first minimum wins.
 * gpt2_pack.c:339-343. */
ORC_API int orc_e4m3_encode(float v) {
    int best = 0;
    float bestd = 1.0e30f;
    for (int c = 0; c < 256; c++) {
        if ((c & 0x7F) == 0x7F) continue;
        float d = orc_e4m3_decode(c) - v;
        if (d < 0) d = -d;
        if (d < bestd) { bestd = d; best = c; }
    }
    return best;
}

/* ------------------------------------------------------------------------------------------------
 * Quantizer.  nvfp4_quantize_tensor, gpt2_pack.c:350-373.
 *   Kpad = K rounded up to a multiple of 112; per tensor ts = amax/(6*448) (1.0 when amax is 0);
 *   per 16-block: micro = e4m3_encode(bamax/(ts*6)), eff = e4m3_decode(micro)*ts,
 *   code = eff>0 ? e2m1_encode(v/eff) : 0; seven codes per int32 word, low nibble first.
 * outSc / outMicro / outTs may each be NULL.  Returns Kpad.
 * ---------------------------------------------------------------------------------------------- */
ORC_API int orc_kpad(int K) { return ((K + 111) / 112) * 112; }

ORC_API int orc_nvfp4_quantize(const float* w, int rows, int K, int32_t* outW, float* outSc,
                               uint8_t* outMicro, float* outTs) {
    int Kpad = orc_kpad(K), kwords = Kpad / 7, kblk = Kpad / 16;
    float amax = 0.0f;
    for (long i = 0; i < (long)rows * K; i++) {
        float a = w[i] < 0 ? -w[i] : w[i];
        if (a > amax) amax = a;
    }
    float ts = amax / (6.0f * 448.0f);
    if (ts <= 0.0f) ts = 1.0f;
    if (outTs) *outTs = ts;
    /* The 254-way search depends only on the block's ratio; rows are independent, so the row loop
     * runs on all cores.  Results are identical to the single-threaded order. */
    #pragma omp parallel
    {
        int* codes = (int*)malloc((size_t)Kpad * sizeof(int));
        #pragma omp for schedule(static)
        for (int r = 0; r < rows; r++) {
            for (int b = 0; b < kblk; b++) {
                float bamax = 0.0f;
                for (int j = 0; j < 16; j++) {
                    int k = b * 16 + j;
                    float v = (k < K) ? w[(long)r * K + k] : 0.0f;
                    float a = v < 0 ? -v : v;
                    if (a > bamax) bamax = a;
                }
                int micro = orc_e4m3_encode(bamax / (ts * 6.0f));
                float eff = orc_e4m3_decode(micro) * ts;
                if (outSc) outSc[(long)r * kblk + b] = eff;
                if (outMicro) outMicro[(long)r * kblk + b] = (uint8_t)micro;
                for (int j = 0; j < 16; j++) {
                    int k = b * 16 + j;
                    float v = (k < K) ? w[(long)r * K + k] : 0.0f;
                    codes[k] = (eff > 0.0f) ? orc_e2m1_encode(v / eff) : 0;
                }
            }
            for (int kw = 0; kw < kwords; kw++) {
                int word = 0, pw = 1;
                for (int j = 0; j < 7; j++) { word += (codes[kw * 7 + j] & 15) * pw; pw *= 16; }
                outW[(long)r * kwords + kw] = word;
            }
        }
        free(codes);
    }
    return Kpad;
}

/* One row of the packed layout -> f32.  The value is sign*mag*(e4m3(micro)*ts) with the two
 * multiplies in that association.  v3_dequant_packed, gpt2_infer.c:109-122. */
static void dequant_row_micro(const int32_t* wr, const uint8_t* mr, float ts, float* out, int Kpad) {
    static const float MAG[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    for (int col = 0; col < Kpad; col++) {
        int wv = wr[col / 7];
        int code = (wv >> (4 * (col % 7))) & 15;   /* words are non-negative: /16 == >>4 */
        float sm = (code & 8) ? -MAG[code & 7] : MAG[code & 7];
        float eff = orc_e4m3_decode(mr[col / 16]) * ts;
        out[col] = sm * eff;
    }
}

ORC_API void orc_nvfp4_dequant_micro(const int32_t* w, const uint8_t* micro, float ts, float* out,
                                     int rows, int Kpad) {
    int kwords = Kpad / 7, kblk = Kpad / 16;
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++)
        dequant_row_micro(w + (long)r * kwords, micro + (long)r * kblk, ts, out + (long)r * Kpad, Kpad);
}

/* Dequant against pre-collapsed f32 scales.  nvfp4_host_dequant, gpt2_pack.c:375-387; this is
 * also what the device kernels nvfp4_dequant / nvfp4_dequant_tiled compute
 * (helixc/examples/nvfp4_dequant_kernel.hx:35-51). */
ORC_API void orc_nvfp4_dequant_sc(const int32_t* w, const float* sc, float* out, int rows, int Kpad) {
    static const float MAG[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    int kwords = Kpad / 7, kblk = Kpad / 16;
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++)
        for (int col = 0; col < Kpad; col++) {
            int wv = w[(long)r * kwords + col / 7];
            int code = (wv >> (4 * (col % 7))) & 15;
            float sm = (code & 8) ? -MAG[code & 7] : MAG[code & 7];
            out[(long)r * Kpad + col] = sm * sc[(long)r * kblk + col / 16];
        }
}

/* Micro-scale bytes -> 4-per-int32 words (low byte first), row stride ceil(kblk/4) words.
 * v3_pack_micro, gpt2_infer.c:2151-2161. */
ORC_API void orc_pack_micro(const uint8_t* micro, long rows, int kblk, int32_t* dst) {
    int micstride = (kblk + 3) / 4;
    memset(dst, 0, (size_t)rows * micstride * 4);
    for (long r = 0; r < rows; r++)
        for (int b = 0; b < kblk; b++)
            dst[r * micstride + (b >> 2)] |= (int32_t)micro[r * kblk + b] << (8 * (b & 3));
}

/* ------------------------------------------------------------------------------------------------
 * SHA-256 (FIPS 180-4).  Restates gpt2_infer.c:137-213; pinned by the three NIST vectors the
 * reference self-test uses (cuda_launch.c:787-805).
 * ---------------------------------------------------------------------------------------------- */
typedef struct { uint32_t h[8]; uint64_t len; uint8_t buf[64]; int fill; } OrcSha;

static const uint32_t SHA_K[64] = {
    0x428a2f98,0x71374491,0xb5c0fbcf,0xe9b5dba5,0x3956c25b,0x59f111f1,0x923f82a4,0xab1c5ed5,
    0xd807aa98,0x12835b01,0x243185be,0x550c7dc3,0x72be5d74,0x80deb1fe,0x9bdc06a7,0xc19bf174,
    0xe49b69c1,0xefbe4786,0x0fc19dc6,0x240ca1cc,0x2de92c6f,0x4a7484aa,0x5cb0a9dc,0x76f988da,
    0x983e5152,0xa831c66d,0xb00327c8,0xbf597fc7,0xc6e00bf3,0xd5a79147,0x06ca6351,0x14292967,
    0x27b70a85,0x2e1b2138,0x4d2c6dfc,0x53380d13,0x650a7354,0x766a0abb,0x81c2c92e,0x92722c85,
    0xa2bfe8a1,0xa81a664b,0xc24b8b70,0xc76c51a3,0xd192e819,0xd6990624,0xf40e3585,0x106aa070,
    0x19a4c116,0x1e376c08,0x2748774c,0x34b0bcb5,0x391c0cb3,0x4ed8aa4a,0x5b9cca4f,0x682e6ff3,
    0x748f82ee,0x78a5636f,0x84c87814,0x8cc70208,0x90befffa,0xa4506ceb,0xbef9a3f7,0xc67178f2};

static inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

static void sha_block(OrcSha* s, const uint8_t* p) {
    uint32_t w[64];
    for (int i = 0; i < 16; i++)
        w[i] = ((uint32_t)p[4*i] << 24) | ((uint32_t)p[4*i+1] << 16) | ((uint32_t)p[4*i+2] << 8) | p[4*i+3];
    for (int i = 16; i < 64; i++) {
        uint32_t s0 = rotr(w[i-15], 7) ^ rotr(w[i-15], 18) ^ (w[i-15] >> 3);
        uint32_t s1 = rotr(w[i-2], 17) ^ rotr(w[i-2], 19) ^ (w[i-2] >> 10);
        w[i] = w[i-16] + s0 + w[i-7] + s1;
    }
    uint32_t a=s->h[0], b=s->h[1], c=s->h[2], d=s->h[3], e=s->h[4], f=s->h[5], g=s->h[6], h=s->h[7];
    for (int i = 0; i < 64; i++) {
        uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
        uint32_t ch = (e & f) ^ (~e & g);
        uint32_t t1 = h + S1 + ch + SHA_K[i] + w[i];
        uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
        uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
        uint32_t t2 = S0 + mj;
        h = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    s->h[0]+=a; s->h[1]+=b; s->h[2]+=c; s->h[3]+=d; s->h[4]+=e; s->h[5]+=f; s->h[6]+=g; s->h[7]+=h;
}

static void sha_init(OrcSha* s) {
    static const uint32_t H0[8] = {0x6a09e667,0xbb67ae85,0x3c6ef372,0xa54ff53a,0x510e527f,0x9b05688c,0x1f83d9ab,0x5be0cd19};
    memcpy(s->h, H0, sizeof(H0)); s->len = 0; s->fill = 0;
}
static void sha_update(OrcSha* s, const uint8_t* p, size_t n) {
    s->len += n;
    while (n) {
        if (s->fill == 0 && n >= 64) { sha_block(s, p); p += 64; n -= 64; continue; }
        size_t take = 64 - (size_t)s->fill; if (take > n) take = n;
        memcpy(s->buf + s->fill, p, take); s->fill += (int)take; p += take; n -= take;
        if (s->fill == 64) { sha_block(s, s->buf); s->fill = 0; }
    }
}
static void sha_final(OrcSha* s, uint8_t out[32]) {
    uint64_t bits = s->len * 8;
    uint8_t pad = 0x80; sha_update(s, &pad, 1);
    uint8_t z = 0; while (s->fill != 56) sha_update(s, &z, 1);
    uint8_t lb[8]; for (int i = 0; i < 8; i++) lb[i] = (uint8_t)(bits >> (56 - 8*i));
    sha_update(s, lb, 8);
    for (int i = 0; i < 8; i++) { out[4*i]=(uint8_t)(s->h[i]>>24); out[4*i+1]=(uint8_t)(s->h[i]>>16); out[4*i+2]=(uint8_t)(s->h[i]>>8); out[4*i+3]=(uint8_t)s->h[i]; }
}

ORC_API void orc_sha256(const uint8_t* data, size_t n, uint8_t out[32]) {
    OrcSha s; sha_init(&s); sha_update(&s, data, n); sha_final(&s, out);
}

ORC_API void orc_sha256_hex(const uint8_t* data, size_t n, char hex[65]) {
    uint8_t d[32]; orc_sha256(data, n, d);
    for (int i = 0; i < 32; i++) sprintf(hex + 2*i, "%02x", d[i]);
    hex[64] = 0;
}

/* ------------------------------------------------------------------------------------------------
 * Elementwise / row operators, restating the kernels the worker launches.
 * ---------------------------------------------------------------------------------------------- */

/* y = w * (x * rsqrt(mean(x^2) + eps)); ascending f32 sum.  gpu_rmsnorm_fwd_eps_kernel.hx:18-29
 * (eps is baked to 1e-5 there; it is a parameter here so that both values can be checked). */
ORC_API void orc_rmsnorm(const float* x, float* y, const float* w, int rows, int cols, float eps) {
    for (int r = 0; r < rows; r++) {
        const float* xr = x + (long)r * cols; float* yr = y + (long)r * cols;
        float ss = 0.0f;
        for (int j = 0; j < cols; j++) ss = ss + xr[j] * xr[j];
        float inv = 1.0f / sqrtf(ss / (float)cols + eps);
        for (int j = 0; j < cols; j++) yr[j] = w[j] * (xr[j] * inv);
    }
}

/* Affine LayerNorm, population variance, two passes.  gpu_layernorm_fwd_eps_kernel.hx:9-25. */
ORC_API void orc_layernorm(const float* x, float* y, const float* g, const float* b, int rows, int cols, float eps) {
    for (int r = 0; r < rows; r++) {
        const float* xr = x + (long)r * cols; float* yr = y + (long)r * cols;
        float sm = 0.0f; for (int j = 0; j < cols; j++) sm = sm + xr[j];
        float mean = sm / (float)cols;
        float vs = 0.0f; for (int j = 0; j < cols; j++) vs = vs + (xr[j] - mean) * (xr[j] - mean);
        float inv = 1.0f / sqrtf(vs / (float)cols + eps);
        for (int j = 0; j < cols; j++) yr[j] = g[j] * ((xr[j] - mean) * inv) + b[j];
    }
}

/* cos/sin tables in double, cast to f32: inv = theta^(-2j/DH), angle = s*inv.
 * gpt2_infer.c:2040-2051. */
ORC_API void orc_rope_tables(float* cosT, float* sinT, int S, int DH, double theta) {
    int half = DH / 2;
    for (int s = 0; s < S; s++)
        for (int j = 0; j < half; j++) {
            double inv = pow(theta, -2.0 * (double)j / (double)DH);
            double ang = (double)s * inv;
            cosT[(long)s * half + j] = (float)cos(ang);
            sinT[(long)s * half + j] = (float)sin(ang);
        }
}

/* rotate_half convention, pairs (i, i+half), in place; table row r pairs with buffer row r.
 * gpu_rope_rot_kernel.hx:23-38. */
ORC_API void orc_rope_rot(float* q, const float* cosT, const float* sinT, int rows, int half) {
    for (int r = 0; r < rows; r++)
        for (int i = 0; i < half; i++) {
            float a = q[(long)r * 2 * half + i], b = q[(long)r * 2 * half + half + i];
            float c = cosT[(long)r * half + i], s = sinT[(long)r * half + i];
            q[(long)r * 2 * half + i] = a * c - b * s;
            q[(long)r * 2 * half + half + i] = b * c + a * s;
        }
}

/* y = g*sigmoid(g)*u with sigmoid(g) = 0.5*(1 + sgn*(1-e)/(1+e)), e = exp(-|g|).
 * gpu_silu_mul_kernel.hx:20-31. */
ORC_API void orc_silu_mul(const float* g, const float* u, float* y, int n) {
    for (int i = 0; i < n; i++) {
        float gi = g[i], sgn = gi < 0.0f ? -1.0f : 1.0f;
        float e = expf(-(sgn * gi));
        float th = sgn * ((1.0f - e) / (1.0f + e));
        y[i] = gi * (0.5f * (1.0f + th)) * u[i];
    }
}

/* gelu_new with the stable tanh form.  gpu_gelu_stable_kernel.hx:15-28. */
ORC_API void orc_gelu(const float* x, float* y, int n) {
    for (int i = 0; i < n; i++) {
        float xi = x[i];
        float inner = 0.7978846f * (xi + 0.044715f * (xi * xi * xi));
        float two = 2.0f * inner, sgn = 1.0f, am = two;
        if (inner < 0.0f) { am = -two; sgn = -1.0f; }
        float e = expf(-am);
        float th = sgn * ((1.0f - e) / (1.0f + e));
        y[i] = 0.5f * xi * (1.0f + th);
    }
}

/* Three-pass row softmax: max from element 0 upward, exp and ascending sum, divide.
 * gpu_softmax_row_kernel.hx:11-34. */
ORC_API void orc_softmax_row(const float* x, float* y, int rows, int cols) {
    for (int r = 0; r < rows; r++) {
        const float* xr = x + (long)r * cols; float* yr = y + (long)r * cols;
        float m = xr[0]; for (int j = 1; j < cols; j++) if (xr[j] > m) m = xr[j];
        float s = 0.0f; for (int j = 0; j < cols; j++) { float e = expf(xr[j] - m); yr[j] = e; s = s + e; }
        for (int j = 0; j < cols; j++) yr[j] = yr[j] / s;
    }
}

/* Causal softmax with an absolute offset: row r normalises over columns [0, base+r], zeros beyond.
 * softmax_causal_offset_kernel.hx:26-56 (base=0 gives gpu_softmax_causal_kernel.hx:10-39). */
ORC_API void orc_softmax_causal_offset(const float* x, float* y, int rows, int cols, int base) {
    for (int r = 0; r < rows; r++) {
        const float* xr = x + (long)r * cols; float* yr = y + (long)r * cols;
        int ext = base + r + 1; if (ext > cols) ext = cols;
        float m = xr[0]; for (int j = 1; j < ext; j++) if (xr[j] > m) m = xr[j];
        float s = 0.0f; for (int j = 0; j < ext; j++) { float e = expf(xr[j] - m); yr[j] = e; s = s + e; }
        for (int j = 0; j < ext; j++) yr[j] = yr[j] / s;
        for (int j = ext; j < cols; j++) yr[j] = 0.0f;
    }
}

/* y[n] = sum_j x[j]*w[n*k+j], one accumulator, ascending.  gpu_gemv_abt_kernel.hx:13-24. */
ORC_API void orc_gemv_abt(const float* x, const float* w, float* y, int N, int K) {
    #pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        float acc = 0.0f; const float* wr = w + (long)n * K;
        for (int j = 0; j < K; j++) acc = fmaf(x[j], wr[j], acc);
        y[n] = acc;
    }
}

/* y[n] = sum_t p[t]*m[t*ncols+n].  gpu_gemv_ab_kernel.hx:11-21. */
ORC_API void orc_gemv_ab(const float* p, const float* m, float* y, int T, int ncols) {
    for (int n = 0; n < ncols; n++) {
        float acc = 0.0f;
        for (int t = 0; t < T; t++) acc = fmaf(p[t], m[(long)t * ncols + n], acc);
        y[n] = acc;
    }
}

/* First maximum wins, NaN never selected.  argmax_row, gpt2_infer.c:1735-1739. */
ORC_API int orc_argmax(const float* v, int n) {
    int a = 0; float best = v[0];
    for (int i = 1; i < n; i++) if (v[i] > best) { best = v[i]; a = i; }
    return a;
}

/* Fused dequant GEMV over the packed layout, y[n] = sum_{col<Kpad} x[col]*deq(W[n,col]); x is
 * Kpad long and zero-tailed.  The weight value is the bit-defined sign*mag*(e4m3*ts); the sum is
 * one ascending f32 accumulator, which is the order of the reference's unfused path and of the CPU
 * oracle in cuda_launch.c:2073 (the fused device kernels reorder the sum across lanes).
 * fused_gemv, gpt2_infer.c:2281-2297. */
ORC_API void orc_gemv_packed(const float* x, const int32_t* W, const uint8_t* micro, float ts,
                             float* y, int N, int Kpad) {
    int kwords = Kpad / 7, kblk = Kpad / 16;
    #pragma omp parallel
    {
        float* row = (float*)malloc((size_t)Kpad * sizeof(float));
        #pragma omp for schedule(static)
        for (int n = 0; n < N; n++) {
            dequant_row_micro(W + (long)n * kwords, micro + (long)n * kblk, ts, row, Kpad);
            float acc = 0.0f;
            for (int j = 0; j < Kpad; j++) acc = fmaf(x[j], row[j], acc);
            y[n] = acc;
        }
        free(row);
    }
}

/* The warp-per-row device order: lane l owns words l, l+32, ...; within a word the seven slots in
 * order, each step fma(x, mag*scale, acc); then acc += shfl_down(acc, d) for d = 16,8,4,2,1.
 * helixc/bootstrap/kovc.hx:14583-14692 (dequant_gemv_warp). */
ORC_API void orc_gemv_packed_warp_order(const float* x, const int32_t* W, const uint8_t* micro, float ts,
                                        float* y, int N, int Kpad) {
    static const float MAG[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    int kwords = Kpad / 7, kblk = Kpad / 16;
    for (int n = 0; n < N; n++) {
        float lane[32];
        for (int l = 0; l < 32; l++) {
            float acc = 0.0f;
            for (int wd = l; wd < kwords; wd += 32) {
                int wv = W[(long)n * kwords + wd];
                for (int s = 0; s < 7; s++) {
                    int col = wd * 7 + s, code = (wv >> (4 * s)) & 15;
                    float sc = orc_e4m3_decode(micro[(long)n * kblk + col / 16]) * ts;
                    float sm = (code & 8) ? -MAG[code & 7] : MAG[code & 7];
                    acc = fmaf(x[col], sm * sc, acc);
                }
            }
            lane[l] = acc;
        }
        for (int d = 16; d >= 1; d >>= 1)
            for (int l = 0; l < 32; l++) lane[l] = lane[l] + ((l + d < 32) ? lane[l + d] : lane[l]);
        y[n] = lane[0];
    }
}

/* One-query GQA attention over the cache with the online softmax of the fused device kernel:
 * m seeded -1e8, per position s = scale*dot(q,k_t), r = exp(m-mn), p = exp(s-mn),
 * acc = acc*r + p*v, l = l*r + p.  fused_decode_attn_kernel.hx:74-102. */
ORC_API void orc_decode_attn_online(const float* q, const float* kc, const float* vc, float* out, float scale,
                                    int NH, int T, int DH, long koff, int grp, long kvstride) {
    for (int h = 0; h < NH; h++) {
        long base = koff + (long)(h / grp) * kvstride;
        for (int d = 0; d < DH; d++) {
            float m = -100000000.0f, l = 0.0f, acc = 0.0f;
            for (int t = 0; t < T; t++) {
                float s = 0.0f;
                for (int e = 0; e < DH; e++) s = s + q[h * DH + e] * kc[base + (long)t * DH + e];
                s = s * scale;
                float mn = s > m ? s : m;
                float r = expf(m - mn), p = expf(s - mn);
                acc = acc * r + p * vc[base + (long)t * DH + d];
                l = l * r + p;
                m = mn;
            }
            out[h * DH + d] = acc / l;
        }
    }
}

/* ------------------------------------------------------------------------------------------------
 * HXGW v3 container.  Header and descriptors: gpt2_pack.c:581-582, 653-663; validation:
 * gpt2_infer.c:581-603; tensor order: build_order_llama(qwen3=1), gpt2_pack.c:255-281.
 * ---------------------------------------------------------------------------------------------- */
typedef struct { uint32_t packed, rows, K, Kpad; uint64_t data_off, scale_off; } OrcDesc;

typedef struct {
    int NL, DM, NH, NKV, DH, QD, KVD, DFF, NV, NC, ntens;
    float theta, eps_file, eps_used, attn_scale;
    const uint8_t* map; size_t maplen; int fd;
    const OrcDesc* desc;
    float *kc, *vc; int kv_cap, kv_len;
    float *cosT, *sinT;
    /* work buffers */
    float *x, *xn, *q, *k, *v, *ctx, *pj, *g, *u, *m, *mo, *sc, *pr;
} OrcModel;

enum { T_INLN = 0, T_Q, T_QN, T_K, T_KN, T_V, T_O, T_POSTLN, T_GATE, T_UP, T_DOWN, T_PER_LAYER };

static uint32_t rd32(const uint8_t* p) { uint32_t v; memcpy(&v, p, 4); return v; }
static float rdf32(const uint8_t* p) { float v; memcpy(&v, p, 4); return v; }

/* Validate that the descriptors tile the file exactly (gpt2_infer.c:587-599).  Returns 0 if ok. */
ORC_API int orc_v3_validate(const uint8_t* file, size_t len) {
    if (len < 64) return 1;
    if (rd32(file) != 0x48584757u) return 2;         /* MAGIC: reads "HXGW" as a hex word */
    if (rd32(file + 4) != 3u) return 3;
    uint32_t nt = rd32(file + 60);
    uint64_t cur = 64 + (uint64_t)nt * 32;
    if (cur > len) return 4;
    const OrcDesc* d = (const OrcDesc*)(file + 64);
    for (uint32_t i = 0; i < nt; i++) {
        if (d[i].data_off != cur) return 5;
        if (d[i].packed) {
            uint64_t wb = (uint64_t)d[i].rows * (d[i].Kpad / 7) * 4;
            if (d[i].scale_off != cur + wb) return 6;
            cur += wb + (uint64_t)d[i].rows * (d[i].Kpad / 16) + 4;
        } else cur += (uint64_t)d[i].rows * d[i].K * 4;
    }
    return cur == len ? 0 : 7;
}

ORC_API void orc_model_close(OrcModel* m);

/* Build the model over an HXGW v3 image already in memory (fd < 0: the caller keeps the bytes alive
 * and owns them).  use_file_eps = 0 uses 1e-5, which is what the reference computes whatever the
 * header says (gpt2_infer.c:661-664); 1 uses the header's rms_norm_eps. */
static OrcModel* model_from_image(const uint8_t* hb, size_t len, int fd, int kv_cap, int use_file_eps) {
    if (orc_v3_validate(hb, len)) return NULL;
    OrcModel* m = (OrcModel*)calloc(1, sizeof(OrcModel));
    m->map = hb; m->maplen = len; m->fd = fd;
    m->NL = (int)rd32(hb + 8); m->DM = (int)rd32(hb + 12); m->NH = (int)rd32(hb + 16); m->NV = (int)rd32(hb + 20);
    m->NC = (int)rd32(hb + 24); m->DFF = (int)rd32(hb + 28); m->NKV = (int)rd32(hb + 44);
    m->theta = rdf32(hb + 48); m->eps_file = rdf32(hb + 52);
    int hd = (int)rd32(hb + 56); m->ntens = (int)rd32(hb + 60);
    m->DH = hd > 0 ? hd : m->DM / m->NH; m->QD = m->NH * m->DH; m->KVD = m->NKV * m->DH;
    m->attn_scale = 1.0f / sqrtf((float)m->DH);
    m->eps_used = use_file_eps ? m->eps_file : 1e-5f;
    m->desc = (const OrcDesc*)(hb + 64);
    if (m->ntens != m->NL * T_PER_LAYER + 3 || m->NKV <= 0 || m->NH % m->NKV) { free(m); return NULL; }
    m->kv_cap = kv_cap; m->kv_len = 0;
    size_t kvn = (size_t)m->NL * m->NKV * kv_cap * m->DH;
    m->kc = (float*)calloc(kvn, 4); m->vc = (float*)calloc(kvn, 4);
    int half = m->DH / 2;
    m->cosT = (float*)malloc((size_t)kv_cap * half * 4); m->sinT = (float*)malloc((size_t)kv_cap * half * 4);
    orc_rope_tables(m->cosT, m->sinT, kv_cap, m->DH, (double)m->theta);
    int kp_dm = orc_kpad(m->DM), kp_qd = orc_kpad(m->QD), kp_df = orc_kpad(m->DFF);
    m->x = (float*)calloc(m->DM, 4); m->xn = (float*)calloc(kp_dm, 4);
    m->q = (float*)calloc(m->QD, 4); m->k = (float*)calloc(m->KVD, 4); m->v = (float*)calloc(m->KVD, 4);
    m->ctx = (float*)calloc(kp_qd, 4); m->pj = (float*)calloc(m->DM, 4);
    m->g = (float*)calloc(m->DFF, 4); m->u = (float*)calloc(m->DFF, 4); m->m = (float*)calloc(kp_df, 4);
    m->mo = (float*)calloc(m->DM, 4); m->sc = (float*)calloc(kv_cap, 4); m->pr = (float*)calloc(kv_cap, 4);
    return m;
}

ORC_API OrcModel* orc_model_open_image(const uint8_t* image, size_t len, int kv_cap, int use_file_eps) {
    return model_from_image(image, len, -1, kv_cap, use_file_eps);
}

/* Open an HXGW v3 file (mapped read-only, as load_gpt2_weights does, gpt2_infer.c:564-603). */
ORC_API OrcModel* orc_model_open(const char* path, int kv_cap, int use_file_eps) {
    int fd = open(path, O_RDONLY);
    if (fd < 0) return NULL;
    struct stat st; if (fstat(fd, &st)) { close(fd); return NULL; }
    void* mp = mmap(NULL, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (mp == MAP_FAILED) { close(fd); return NULL; }
    OrcModel* m = model_from_image((const uint8_t*)mp, (size_t)st.st_size, fd, kv_cap, use_file_eps);
    if (!m) { munmap(mp, (size_t)st.st_size); close(fd); }
    return m;
}

ORC_API void orc_model_close(OrcModel* m) {
    if (!m) return;
    free(m->kc); free(m->vc); free(m->cosT); free(m->sinT);
    free(m->x); free(m->xn); free(m->q); free(m->k); free(m->v); free(m->ctx); free(m->pj);
    free(m->g); free(m->u); free(m->m); free(m->mo); free(m->sc); free(m->pr);
    if (m->map && m->fd >= 0) { munmap((void*)m->map, m->maplen); close(m->fd); }
    free(m);
}

ORC_API void orc_model_dims(const OrcModel* m, int* out /* NL DM NH NKV DH DFF NV QD KVD */) {
    out[0]=m->NL; out[1]=m->DM; out[2]=m->NH; out[3]=m->NKV; out[4]=m->DH; out[5]=m->DFF; out[6]=m->NV; out[7]=m->QD; out[8]=m->KVD;
}
ORC_API void orc_model_reset(OrcModel* m) { m->kv_len = 0; }
/* Place n cached positions [pos0, pos0 + n) of (layer, kv head) into the cache: lets a test mirror a cache that
 * was not produced by this model's own prefill.  Layout as gpt2_infer.c:709-721. */
ORC_API int orc_model_kv_set(OrcModel* m, int L, int kv, int pos0, int n, const float* k, const float* v) {
    if (L < 0 || L >= m->NL || kv < 0 || kv >= m->NKV || pos0 < 0 || n < 0 || pos0 + n > m->kv_cap) return 1;
    size_t off = ((((size_t)L * m->NKV + kv) * m->kv_cap) + pos0) * m->DH;
    memcpy(m->kc + off, k, (size_t)n * m->DH * 4);
    memcpy(m->vc + off, v, (size_t)n * m->DH * 4);
    if (pos0 + n > m->kv_len) m->kv_len = pos0 + n;
    return 0;
}

static const float* dense_ptr(const OrcModel* m, int idx) { return (const float*)(m->map + m->desc[idx].data_off); }

/* y[0..rows) = packed tensor idx applied to xpad (Kpad long, zero tail). */
static void packed_gemv(const OrcModel* m, int idx, const float* xpad, float* y) {
    const OrcDesc* d = &m->desc[idx];
    const int32_t* W = (const int32_t*)(m->map + d->data_off);
    const uint8_t* mic = m->map + d->scale_off;
    float ts = rdf32(m->map + d->scale_off + (size_t)d->rows * (d->Kpad / 16));
    orc_gemv_packed(xpad, W, mic, ts, y, (int)d->rows, (int)d->Kpad);
}

static size_t kvoff(const OrcModel* m, int L, int kv) { return (((size_t)L * m->NKV + kv) * m->kv_cap) * m->DH; }

/* One decode step at position pos (= the number of cached positions).  Sequencing restates
 * decode_step_llama, gpt2_infer.c:1341-1613, with the per-head attention of :1531-1544 (scores by
 * gemv_abt, scale, three-pass softmax, probabilities times V by gemv_ab).  hidden_out (DM floats,
 * optional) receives the residual stream after the last layer. */
ORC_API int orc_model_decode(OrcModel* m, int id, int pos, float* logits, float* hidden_out) {
    if (pos >= m->kv_cap || id < 0 || id >= m->NV) return 1;
    int NL = m->NL, DM = m->DM, NH = m->NH, NKV = m->NKV, DH = m->DH, DFF = m->DFF, grp = NH / NKV, T = pos + 1;
    int half = DH / 2;
    memcpy(m->x, dense_ptr(m, NL * T_PER_LAYER + 0) + (size_t)id * DM, (size_t)DM * 4);   /* :1347-1350 */
    for (int L = 0; L < NL; L++) {
        int b = L * T_PER_LAYER;
        orc_rmsnorm(m->x, m->xn, dense_ptr(m, b + T_INLN), 1, DM, m->eps_used);
        packed_gemv(m, b + T_Q, m->xn, m->q);
        packed_gemv(m, b + T_K, m->xn, m->k);
        packed_gemv(m, b + T_V, m->xn, m->v);
        orc_rmsnorm(m->q, m->q, dense_ptr(m, b + T_QN), NH, DH, m->eps_used);     /* per-head QK-norm, :1500-1501 */
        orc_rmsnorm(m->k, m->k, dense_ptr(m, b + T_KN), NKV, DH, m->eps_used);
        for (int h = 0; h < NH; h++) orc_rope_rot(m->q + h * DH, m->cosT + (size_t)pos * half, m->sinT + (size_t)pos * half, 1, half);
        for (int kv = 0; kv < NKV; kv++) {
            orc_rope_rot(m->k + kv * DH, m->cosT + (size_t)pos * half, m->sinT + (size_t)pos * half, 1, half);
            memcpy(m->kc + kvoff(m, L, kv) + (size_t)pos * DH, m->k + kv * DH, (size_t)DH * 4);
            memcpy(m->vc + kvoff(m, L, kv) + (size_t)pos * DH, m->v + kv * DH, (size_t)DH * 4);
        }
        #pragma omp parallel for schedule(static)
        for (int h = 0; h < NH; h++) {
            int kv = h / grp;
            float* sc = (float*)malloc((size_t)T * 8); float* pr = sc + T;
            const float* kb = m->kc + kvoff(m, L, kv); const float* vb = m->vc + kvoff(m, L, kv);
            for (int t = 0; t < T; t++) {
                float acc = 0.0f;
                for (int e = 0; e < DH; e++) acc = fmaf(m->q[h * DH + e], kb[(size_t)t * DH + e], acc);
                sc[t] = acc * m->attn_scale;
            }
            orc_softmax_row(sc, pr, 1, T);
            for (int d = 0; d < DH; d++) {
                float acc = 0.0f;
                for (int t = 0; t < T; t++) acc = fmaf(pr[t], vb[(size_t)t * DH + d], acc);
                m->ctx[h * DH + d] = acc;
            }
            free(sc);
        }
        packed_gemv(m, b + T_O, m->ctx, m->pj);
        for (int i = 0; i < DM; i++) m->x[i] = m->x[i] + m->pj[i];
        orc_rmsnorm(m->x, m->xn, dense_ptr(m, b + T_POSTLN), 1, DM, m->eps_used);
        packed_gemv(m, b + T_GATE, m->xn, m->g);
        packed_gemv(m, b + T_UP, m->xn, m->u);
        orc_silu_mul(m->g, m->u, m->m, DFF);
        packed_gemv(m, b + T_DOWN, m->m, m->mo);
        for (int i = 0; i < DM; i++) m->x[i] = m->x[i] + m->mo[i];
    }
    if (hidden_out) memcpy(hidden_out, m->x, (size_t)DM * 4);
    if (logits) {
        orc_rmsnorm(m->x, m->xn, dense_ptr(m, NL * T_PER_LAYER + 1), 1, DM, m->eps_used);
        packed_gemv(m, NL * T_PER_LAYER + 2, m->xn, logits);
    }
    m->kv_len = T;
    return 0;
}

/* Prefill = the same arithmetic per position with causality carried by what is cached (the
 * reference states the two are identical by construction, gpt2_infer.c:1336-1340); returns the
 * logits of the last prompt position. */
ORC_API int orc_model_prefill(OrcModel* m, const int* ids, int T, float* last_logits) {
    m->kv_len = 0;
    for (int s = 0; s < T; s++)
        if (orc_model_decode(m, ids[s], s, s == T - 1 ? last_logits : NULL, NULL)) return 1;
    return 0;
}

/* Greedy generation: prefill, then n_new steps each feeding the arg-max back.
 * run_generate, gpt2_infer.c:3123-3195. */
ORC_API int orc_model_generate(OrcModel* m, const int* ids, int T, int n_new, int* out_ids, float* last_logits) {
    float* lg = (float*)malloc((size_t)m->NV * 4);
    if (orc_model_prefill(m, ids, T, lg)) { free(lg); return 1; }
    for (int i = 0; i < n_new; i++) {
        int nx = orc_argmax(lg, m->NV);
        out_ids[i] = nx;
        if (i == n_new - 1) break;
        if (orc_model_decode(m, nx, T + i, lg, NULL)) { free(lg); return 1; }
    }
    if (last_logits) memcpy(last_logits, lg, (size_t)m->NV * 4);
    free(lg);
    return 0;
}

/* Prompt-lookup drafter: pld_draft, gpt2_infer.c:2972-2994.  For k = k_max (capped to T-1) down to k_min the
 * last k tokens are searched for backwards from candidate start T-k-1; the first candidate that is followed by
 * at least one token before T gives the draft (those tokens, at most m, cap 16).  Returns the draft length. */
ORC_API int orc_pld_draft(const int* ids, int T, int k_min, int k_max, int m, int* draft) {
    if (T < k_min + 1) return 0;
    if (m > 16) m = 16;
    if (m < 1) return 0;
    int k = k_max > T - 1 ? T - 1 : k_max;
    while (k >= k_min) {
        int j = T - k - 1;
        while (j >= 0) {
            int same = 1, t = 0;
            while (t < k && same) { same = ids[j + t] == ids[T - k + t]; t++; }
            if (same) {
                int n = 0, src = j + k;
                while (n < m && src < T) draft[n++] = ids[src++];
                if (n > 0) return n;
            }
            j--;
        }
        k--;
    }
    return 0;
}

/* One speculative generation at the level of tokens: spec_step + run_generate's HX_SPEC loop, gpt2_infer.c:3076-3118,
 * 3150-3161, with the verify forward replaced by what it is defined to equal -- the plain greedy continuation
 * `greedy` (n_new tokens after the T prompt tokens).  Produces the counters of the reference's [specprof] line for
 * that sequence: stats = {steps, hits, drafted, accepted, emitted, forwards}.  kv_cap clamps a draft like :3084. */
ORC_API void orc_spec_counters(const int* prompt, int T, const int* greedy, int n_new, int k_min, int k_max, int m,
                               int kv_cap, long* stats) {
    int* ids = (int*)malloc((size_t)(T + n_new) * sizeof(int));
    memcpy(ids, prompt, (size_t)T * sizeof(int));
    for (int i = 0; i < 6; i++) stats[i] = 0;
    int len = T, step = 0;
    ids[len++] = greedy[0]; step = 1;                      /* step 0 is the prefill forward */
    while (step < n_new) {
        int draft[16];
        int pos = len - 1;
        int dn = orc_pld_draft(ids, len, k_min, k_max, m, draft);
        if (len >= k_min + 1) stats[0]++;
        if (dn > 0) { stats[1]++; stats[2] += dn; }
        if (pos + dn >= kv_cap) { dn = kv_cap - 1 - pos; if (dn < 0) dn = 0; }
        if (dn == 0) { ids[len] = greedy[len - T]; len++; step++; continue; }
        /* the verify rows' arg-maxes are the greedy tokens that follow (t, d_1..d_i) while the drafts are right */
        int commit = 1;
        for (int i = 1; i <= dn; i++) { if (draft[i - 1] == greedy[len - T + i - 1]) commit = i + 1; else break; }
        if (commit > n_new - step) commit = n_new - step;
        for (int i = 0; i < commit; i++) { ids[len] = greedy[len - T]; len++; }
        stats[3] += commit - 1; stats[4] += commit; stats[5]++;
        step += commit;
    }
    free(ids);
}

/* Seeded sampler: sample_next, gpt2_infer.c:1660-1711, with its PCG32 (:1632-1644).  Double precision throughout:
 * penalties on the raw logits of tokens seen before, temperature, candidates sorted by (-value, id), soft-max over
 * the top-k, top-p keeping the crossing token, min-p relative to the best, renormalise, one draw u in [0,1), first
 * index whose running sum exceeds u. */
static uint64_t orc_pcg_state, orc_pcg_inc;
ORC_API void orc_pcg_seed(uint64_t seed) {
    orc_pcg_state = 0u; orc_pcg_inc = (54u << 1) | 1u;
    orc_pcg_state = orc_pcg_state * 6364136223846793005ULL + orc_pcg_inc;
    orc_pcg_state += seed;
    orc_pcg_state = orc_pcg_state * 6364136223846793005ULL + orc_pcg_inc;
}
ORC_API uint32_t orc_pcg_next(void) {
    uint64_t old = orc_pcg_state;
    orc_pcg_state = old * 6364136223846793005ULL + orc_pcg_inc;
    uint32_t xs = (uint32_t)(((old >> 18) ^ old) >> 27), rot = (uint32_t)(old >> 59);
    return (xs >> rot) | (xs << ((32 - rot) & 31));
}
typedef struct { int id; double v; } OrcCand;
static int orc_cand_cmp(const void* a, const void* b) {
    const OrcCand* x = (const OrcCand*)a; const OrcCand* y = (const OrcCand*)b;
    if (x->v > y->v) return -1;
    if (x->v < y->v) return 1;
    return (x->id < y->id) ? -1 : (x->id > y->id) ? 1 : 0;
}
ORC_API int orc_sample_next(const float* logits, int nv, const unsigned short* counts, double temp, double top_p, double min_p,
                            double rep_pen, double freq_pen, double pres_pen, int top_k) {
    OrcCand* cand = (OrcCand*)malloc((size_t)nv * sizeof(OrcCand));
    double invt = 1.0 / temp;
    for (int i = 0; i < nv; i++) {
        double x = (double)logits[i];
        int c = counts ? (int)counts[i] : 0;
        if (c > 0 && rep_pen != 1.0) x = (x > 0.0) ? x / rep_pen : x * rep_pen;
        if (c > 0) x -= freq_pen * (double)c + pres_pen;
        cand[i].id = i; cand[i].v = x * invt;
    }
    qsort(cand, (size_t)nv, sizeof(OrcCand), orc_cand_cmp);
    int n = (top_k > 0 && top_k < nv) ? top_k : nv;
    double mx = cand[0].v, sum = 0.0;
    for (int i = 0; i < n; i++) { cand[i].v = exp(cand[i].v - mx); sum += cand[i].v; }
    for (int i = 0; i < n; i++) cand[i].v /= sum;
    if (top_p < 1.0) {
        double cum = 0.0; int keep = n;
        for (int i = 0; i < n; i++) { cum += cand[i].v; if (cum >= top_p) { keep = i + 1; break; } }
        n = keep;
    }
    if (min_p > 0.0) {
        double floor_p = min_p * cand[0].v; int keep = n;
        for (int i = 0; i < n; i++) if (cand[i].v < floor_p) { keep = i; break; }
        n = keep > 0 ? keep : 1;
    }
    double rsum = 0.0;
    for (int i = 0; i < n; i++) rsum += cand[i].v;
    double u = (double)orc_pcg_next() / 4294967296.0, cum2 = 0.0;
    int pick = cand[n - 1].id;
    for (int i = 0; i < n; i++) { cum2 += cand[i].v / rsum; if (cum2 > u) { pick = cand[i].id; break; } }
    free(cand);
    return pick;
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---------------------------------------------------------------------------------------------------
 * GPT-2 block with a KV cache (the GPT-2-124M configuration).  Restates forward_layer_gpt2, gpt2_infer.c:1131-1193
 * (LayerNorm -> fused qkv + bias -> per-head softmax(q k^T * 1/sqrt(DH)) v -> proj + bias + residual ->
 * LayerNorm -> c_fc + bias -> gelu_new -> proj + bias + residual), embed_gather :1201-1223 (wte row + wpe
 * row), ln_f and the tied head.  The reference re-forwards the whole context every token; with causal
 * attention that equals one position at a time over cached k and v, which is what is done here.
 * Weights arrive as f32 (already dequantized by the caller), every linear [out][in]:
 *   t[0..4] = wte, wpe, lnf_g, lnf_b, head_w; per layer 12 more: ln1_g ln1_b w_qkv b_qkv w_proj b_proj
 *   ln2_g ln2_b w_fc b_fc w_proj2 b_proj2.  dims = NL DM NH DFF NV.  kc, vc: [NL][NH][cap][DH], caller-owned. */
ORC_API int orc_gpt2_decode(const int* dims, const float* const* t, float* kc, float* vc, int cap, int tok, int pos, float* logits) {
    const int NL = dims[0], DM = dims[1], NH = dims[2], DFF = dims[3], NV = dims[4], DH = DM / NH;
    if (pos < 0 || pos >= cap || tok < 0 || tok >= NV) return 1;
    float* x = (float*)malloc((size_t)DM * 4); float* h = (float*)malloc((size_t)DM * 4);
    float* qkv = (float*)malloc((size_t)3 * DM * 4); float* ctx = (float*)malloc((size_t)DM * 4);
    float* f = (float*)malloc((size_t)DFF * 4); float* g = (float*)malloc((size_t)DFF * 4); float* y = (float*)malloc((size_t)DM * 4);
    float* sc = (float*)malloc((size_t)(pos + 1) * 4); float* pr = (float*)malloc((size_t)(pos + 1) * 4);
    const float scale = 1.0f / sqrtf((float)DH);
    for (int j = 0; j < DM; j++) x[j] = t[0][(long)tok * DM + j] + t[1][(long)pos * DM + j];
    for (int L = 0; L < NL; L++) {
        const float* const* w = t + 5 + 12 * L;
        orc_layernorm(x, h, w[0], w[1], 1, DM, 1e-5f);
        orc_gemv_abt(h, w[2], qkv, 3 * DM, DM);
        for (int j = 0; j < 3 * DM; j++) qkv[j] = qkv[j] + w[3][j];
        for (int hh = 0; hh < NH; hh++) {
            float* kr = kc + (((long)L * NH + hh) * cap + pos) * DH; float* vr = vc + (((long)L * NH + hh) * cap + pos) * DH;
            for (int d = 0; d < DH; d++) { kr[d] = qkv[DM + hh * DH + d]; vr[d] = qkv[2 * DM + hh * DH + d]; }
            const float* q = qkv + hh * DH;
            const float* kb = kc + ((long)L * NH + hh) * cap * DH; const float* vb = vc + ((long)L * NH + hh) * cap * DH;
            for (int s = 0; s <= pos; s++) { float a = 0.0f; for (int d = 0; d < DH; d++) a = fmaf(q[d], kb[(long)s * DH + d], a); sc[s] = a * scale; }
            orc_softmax_row(sc, pr, 1, pos + 1);
            for (int d = 0; d < DH; d++) { float a = 0.0f; for (int s = 0; s <= pos; s++) a = fmaf(pr[s], vb[(long)s * DH + d], a); ctx[hh * DH + d] = a; }
        }
        orc_gemv_abt(ctx, w[4], y, DM, DM);
        for (int j = 0; j < DM; j++) x[j] = x[j] + (y[j] + w[5][j]);
        orc_layernorm(x, h, w[6], w[7], 1, DM, 1e-5f);
        orc_gemv_abt(h, w[8], f, DFF, DM);
        for (int j = 0; j < DFF; j++) f[j] = f[j] + w[9][j];
        orc_gelu(f, g, DFF);
        orc_gemv_abt(g, w[10], y, DM, DFF);
        for (int j = 0; j < DM; j++) x[j] = x[j] + (y[j] + w[11][j]);
    }
    orc_layernorm(x, h, t[2], t[3], 1, DM, 1e-5f);
    orc_gemv_abt(h, t[4], logits, NV, DM);
    free(x); free(h); free(qkv); free(ctx); free(f); free(g); free(y); free(sc); free(pr);
    return 0;
}
