// hx_host.cu -- host-side pieces of the C ABI: error state, device-memory helpers, scalar codecs,
// SHA-256 and the HELIX_V16_RECEIPT writer / verifier.
//
// Reference: sha256* helixc/runtime/gpt2_infer.c:137-213; run_v3_receipt_from_logits :2827-2871;
// run_v3_receipt_check :2876-2912; calib_tau :2765-2769; argmax_row :1735-1739.
#include "hx_common.cuh"
#include <stdarg.h>
#include <stdlib.h>
#include <string>
#include <vector>

static thread_local char g_err[512] = "";

void hx_set_error(const char* fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_err, sizeof(g_err), fmt, ap); va_end(ap);
}
int hx_fail(int code, const char* fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_err, sizeof(g_err), fmt, ap); va_end(ap);
    return code;
}
HX_API const char* hx_last_error(void) { return g_err; }
HX_API const char* hx_version(void) { return "helix_b200 0.1 (sm_100a)"; }

// ---- device helpers ------------------------------------------------------------------------------
HX_API int hx_device_count(int* n) { HX_CHECK_ARG(n); HX_CUDA(cudaGetDeviceCount(n)); return HX_OK; }
HX_API int hx_set_device(int dev) { HX_CUDA(cudaSetDevice(dev)); return HX_OK; }
HX_API int hx_malloc(void** dptr, size_t bytes) { HX_CHECK_ARG(dptr); HX_CUDA(cudaMalloc(dptr, bytes ? bytes : 1)); return HX_OK; }
HX_API int hx_free(void* dptr) { HX_CUDA(cudaFree(dptr)); return HX_OK; }
HX_API int hx_memcpy_h2d(void* dst, const void* src, size_t bytes) { HX_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice)); return HX_OK; }
HX_API int hx_memcpy_d2h(void* dst, const void* src, size_t bytes) { HX_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost)); return HX_OK; }
HX_API int hx_memset(void* dptr, int value, size_t bytes) { HX_CUDA(cudaMemset(dptr, value, bytes)); return HX_OK; }
HX_API int hx_sync(void) { HX_CUDA(cudaDeviceSynchronize()); return HX_OK; }
HX_API int hx_host_alloc(void** hptr, size_t bytes) { HX_CHECK_ARG(hptr); HX_CUDA(cudaMallocHost(hptr, bytes ? bytes : 1)); return HX_OK; }
HX_API int hx_host_free(void* hptr) { HX_CUDA(cudaFreeHost(hptr)); return HX_OK; }
HX_API unsigned long long hx_launch_count(void) { return g_hx_launches; }

// ---- scalar codecs -------------------------------------------------------------------------------
HX_API float hx_e2m1_decode(int code) { return hx_e2m1_dec(code); }
HX_API int   hx_e2m1_encode(float v) { return hx_e2m1_enc(v); }
HX_API float hx_e4m3_decode(int code) { return hx_e4m3_dec(code); }
HX_API int   hx_e4m3_encode(float v) { return hx_e4m3_enc(v); }

// ---- SHA-256 (FIPS 180-4) ------------------------------------------------------------------------
namespace {
struct Sha {
    uint32_t h[8]; uint64_t len; uint8_t buf[64]; size_t fill;
    Sha() { static const uint32_t H0[8] = {0x6a09e667u,0xbb67ae85u,0x3c6ef372u,0xa54ff53au,0x510e527fu,0x9b05688cu,0x1f83d9abu,0x5be0cd19u};
            memcpy(h, H0, sizeof(h)); len = 0; fill = 0; }
    static uint32_t ror(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
    void block(const uint8_t* p) {
        static const uint32_t K[64] = {
            0x428a2f98,0x71374491,0xb5c0fbcf,0xe9b5dba5,0x3956c25b,0x59f111f1,0x923f82a4,0xab1c5ed5,0xd807aa98,0x12835b01,0x243185be,0x550c7dc3,
            0x72be5d74,0x80deb1fe,0x9bdc06a7,0xc19bf174,0xe49b69c1,0xefbe4786,0x0fc19dc6,0x240ca1cc,0x2de92c6f,0x4a7484aa,0x5cb0a9dc,0x76f988da,
            0x983e5152,0xa831c66d,0xb00327c8,0xbf597fc7,0xc6e00bf3,0xd5a79147,0x06ca6351,0x14292967,0x27b70a85,0x2e1b2138,0x4d2c6dfc,0x53380d13,
            0x650a7354,0x766a0abb,0x81c2c92e,0x92722c85,0xa2bfe8a1,0xa81a664b,0xc24b8b70,0xc76c51a3,0xd192e819,0xd6990624,0xf40e3585,0x106aa070,
            0x19a4c116,0x1e376c08,0x2748774c,0x34b0bcb5,0x391c0cb3,0x4ed8aa4a,0x5b9cca4f,0x682e6ff3,0x748f82ee,0x78a5636f,0x84c87814,0x8cc70208,
            0x90befffa,0xa4506ceb,0xbef9a3f7,0xc67178f2};
        uint32_t w[64];
        for (int i = 0; i < 16; i++) w[i] = (uint32_t)p[4*i] << 24 | (uint32_t)p[4*i+1] << 16 | (uint32_t)p[4*i+2] << 8 | p[4*i+3];
        for (int i = 16; i < 64; i++) {
            const uint32_t a = ror(w[i-15], 7) ^ ror(w[i-15], 18) ^ (w[i-15] >> 3);
            const uint32_t b = ror(w[i-2], 17) ^ ror(w[i-2], 19) ^ (w[i-2] >> 10);
            w[i] = w[i-16] + a + w[i-7] + b;
        }
        uint32_t s[8]; memcpy(s, h, sizeof(s));
        for (int i = 0; i < 64; i++) {
            const uint32_t t1 = s[7] + (ror(s[4], 6) ^ ror(s[4], 11) ^ ror(s[4], 25)) + ((s[4] & s[5]) ^ (~s[4] & s[6])) + K[i] + w[i];
            const uint32_t t2 = (ror(s[0], 2) ^ ror(s[0], 13) ^ ror(s[0], 22)) + ((s[0] & s[1]) ^ (s[0] & s[2]) ^ (s[1] & s[2]));
            s[7] = s[6]; s[6] = s[5]; s[5] = s[4]; s[4] = s[3] + t1; s[3] = s[2]; s[2] = s[1]; s[1] = s[0]; s[0] = t1 + t2;
        }
        for (int i = 0; i < 8; i++) h[i] += s[i];
    }
    void update(const uint8_t* p, size_t n) {
        len += n;
        if (fill) {
            size_t take = 64 - fill; if (take > n) take = n;
            memcpy(buf + fill, p, take); fill += take; p += take; n -= take;
            if (fill == 64) { block(buf); fill = 0; }
        }
        while (n >= 64) { block(p); p += 64; n -= 64; }
        if (n) { memcpy(buf, p, n); fill = n; }
    }
    void final(uint8_t out[32]) {
        const uint64_t bits = len * 8;
        uint8_t pad[72] = {0x80};
        size_t padn = (fill < 56) ? 56 - fill : 120 - fill;
        update(pad, padn);
        uint8_t lb[8]; for (int i = 0; i < 8; i++) lb[i] = (uint8_t)(bits >> (56 - 8 * i));
        update(lb, 8);
        for (int i = 0; i < 8; i++) { out[4*i] = h[i] >> 24; out[4*i+1] = h[i] >> 16; out[4*i+2] = h[i] >> 8; out[4*i+3] = h[i]; }
    }
};
void to_hex(const uint8_t d[32], char hex[65]) {
    static const char* X = "0123456789abcdef";
    for (int i = 0; i < 32; i++) { hex[2*i] = X[d[i] >> 4]; hex[2*i+1] = X[d[i] & 15]; }
    hex[64] = 0;
}
}  // namespace

HX_API int hx_sha256(const void* data, size_t n, uint8_t out[32]) {
    HX_CHECK_ARG((data || n == 0) && out);
    Sha s; s.update((const uint8_t*)data, n); s.final(out);
    return HX_OK;
}
HX_API int hx_sha256_hex(const void* data, size_t n, char hex[65]) {
    uint8_t d[32]; int rc = hx_sha256(data, n, d); if (rc) return rc;
    to_hex(d, hex); return HX_OK;
}
HX_API int hx_sha256_file(const char* path, char hex[65]) {
    HX_CHECK_ARG(path && hex);
    FILE* f = fopen(path, "rb");
    if (!f) return hx_fail(HX_ERR_IO, "cannot open %s", path);
    std::vector<uint8_t> buf(1 << 20);
    Sha s; size_t got;
    while ((got = fread(buf.data(), 1, buf.size(), f)) > 0) s.update(buf.data(), got);
    fclose(f);
    uint8_t d[32]; s.final(d); to_hex(d, hex);
    return HX_OK;
}

// ---- receipt -------------------------------------------------------------------------------------
static int argmax_first(const float* v, int n) {
    int a = 0; float best = v[0];
    for (int i = 1; i < n; i++) if (v[i] > best) { best = v[i]; a = i; }
    return a;
}

HX_API int hx_receipt_emit(const char* out_path, const char* weights_path, const int* ids, int n_ids,
                           const float* logits, int n_logits, const float* oracle_logits, double tau,
                           const char* tau_prov) {
    HX_CHECK_ARG(out_path && weights_path && ids && n_ids > 0 && logits && n_logits > 0);
    std::string lpath = std::string(out_path) + ".logits";
    FILE* lf = fopen(lpath.c_str(), "wb");
    if (!lf) return hx_fail(HX_ERR_IO, "cannot write %s", lpath.c_str());
    const bool okw = fwrite(logits, sizeof(float), (size_t)n_logits, lf) == (size_t)n_logits;
    fclose(lf);
    if (!okw) return hx_fail(HX_ERR_IO, "short write %s", lpath.c_str());
    char model_hex[65], logits_hex[65];
    int rc = hx_sha256_file(weights_path, model_hex); if (rc) return rc;
    rc = hx_sha256_hex(logits, (size_t)n_logits * sizeof(float), logits_hex); if (rc) return rc;
    const int am = argmax_first(logits, n_logits);
    double max_abs = -1.0; int argmatch = -1;
    if (oracle_logits) {
        double m = 0;
        for (int i = 0; i < n_logits; i++) { const double e = fabs((double)logits[i] - (double)oracle_logits[i]); if (e > m) m = e; }
        max_abs = m; argmatch = (am == argmax_first(oracle_logits, n_logits)) ? 1 : 0;
    }
    FILE* rf = fopen(out_path, "wb");
    if (!rf) return hx_fail(HX_ERR_IO, "cannot write %s", out_path);
    fprintf(rf, "HELIX_V16_RECEIPT\n");
    fprintf(rf, "model_sha256 %s\n", model_hex);
    fprintf(rf, "ids"); for (int i = 0; i < n_ids; i++) fprintf(rf, " %d", ids[i]); fprintf(rf, "\n");
    fprintf(rf, "n_logits %d\n", n_logits);
    fprintf(rf, "logits_sha256 %s\n", logits_hex);
    fprintf(rf, "argmax %d\n", am);
    fprintf(rf, "tier3_tau %.17g\n", tau > 0.0 ? tau : max_abs);
    fprintf(rf, "tier3_max_abs %.17g\n", max_abs);
    fprintf(rf, "tier3_argmax_match %d\n", argmatch);
    if (tau_prov && *tau_prov) fprintf(rf, "tier3_tau_prov %s\n", tau_prov);
    fprintf(rf, "note emitted by helix_b200 (sm_100a path); Tier-2=reproducibility (re-derive from the committed weights); "
                "Tier-3=empirical envelope vs a trusted f32 oracle.\n");
    fclose(rf);
    return HX_OK;
}

static std::vector<float> read_floats(const char* path, size_t n, bool* ok) {
    std::vector<float> v(n);
    FILE* f = fopen(path, "rb");
    *ok = false;
    if (!f) return v;
    *ok = fread(v.data(), sizeof(float), n, f) == n;
    fclose(f);
    return v;
}

HX_API int hx_receipt_check(const char* receipt, const char* weights_path, const char* logits_path,
                            const char* oracle_path) {
    HX_CHECK_ARG(receipt && weights_path && logits_path && oracle_path);
    FILE* rf = fopen(receipt, "rb");
    if (!rf) return hx_fail(HX_ERR_FORMAT, "REJECT=OPEN");
    char line[1024], r_model[80] = {0}, r_logits[80] = {0};
    int hdr = 0, r_argmax = -1, r_nlog = 0, r_argmatch = -1; double r_tau = -1;
    while (fgets(line, sizeof(line), rf)) {
        if (strncmp(line, "HELIX_V16_RECEIPT", 17) == 0) hdr = 1;
        else if (sscanf(line, "model_sha256 %79s", r_model) == 1) continue;
        else if (sscanf(line, "logits_sha256 %79s", r_logits) == 1) continue;
        else if (sscanf(line, "n_logits %d", &r_nlog) == 1) continue;
        else if (sscanf(line, "argmax %d", &r_argmax) == 1) continue;
        else if (sscanf(line, "tier3_tau %lf", &r_tau) == 1) continue;
        else if (sscanf(line, "tier3_argmax_match %d", &r_argmatch) == 1) continue;
    }
    fclose(rf);
    if (!hdr || !r_model[0] || !r_logits[0] || r_argmax < 0 || r_tau < 0 || r_nlog <= 0) return hx_fail(HX_ERR_FORMAT, "REJECT=VACUITY");
    char h[65];
    if (hx_sha256_file(weights_path, h)) return hx_fail(HX_ERR_FORMAT, "REJECT=MODEL_HASH (weights unreadable)");
    if (strcmp(h, r_model) != 0) return hx_fail(HX_ERR_FORMAT, "REJECT=MODEL_HASH");
    if (hx_sha256_file(logits_path, h)) return hx_fail(HX_ERR_FORMAT, "REJECT=LOGITS_HASH (logits unreadable)");
    if (strcmp(h, r_logits) != 0) return hx_fail(HX_ERR_FORMAT, "REJECT=LOGITS_HASH");
    bool ok;
    std::vector<float> L = read_floats(logits_path, (size_t)r_nlog, &ok);
    if (!ok) return hx_fail(HX_ERR_FORMAT, "REJECT=LOGITS_SIZE");
    const int am = argmax_first(L.data(), r_nlog);
    if (am != r_argmax) return hx_fail(HX_ERR_FORMAT, "REJECT=ARGMAX (logits %d != receipt %d)", am, r_argmax);
    std::vector<float> O = read_floats(oracle_path, (size_t)r_nlog, &ok);
    if (!ok) return hx_fail(HX_ERR_FORMAT, "REJECT=ORACLE_SIZE");
    double m = 0;
    for (int i = 0; i < r_nlog; i++) { const double e = fabs((double)L[i] - (double)O[i]); if (e > m) m = e; }
    if (m > r_tau) return hx_fail(HX_ERR_FORMAT, "REJECT=TIER3_ENVELOPE (max_abs=%.6f > tau=%.6f)", m, r_tau);
    if (am != argmax_first(O.data(), r_nlog)) return hx_fail(HX_ERR_FORMAT, "REJECT=TIER3_ARGMAX");
    hx_set_error("RECEIPT_CHECK_PASS");
    return HX_OK;
}

// ---- kernel-image launcher ---------------------------------------------------------------------------
// Loads a module image (fatbin, cubin or PTX text) and launches entries by name exactly the way the
// reference's host programs do: cuModuleLoadData + cuModuleGetFunction + cuLaunchKernel with the
// caller's grid/block, zero dynamic shared memory, the NULL stream
// (helixc/runtime/gpt2_infer.c:373-375, 1944-1964; helixc/runtime/cuda_launch.c:1058-1088).
// The driver library is bound at run time so that the shared object loads on machines without one.
#include <dlfcn.h>
namespace {
typedef int (*cuModuleLoadData_t)(void**, const void*);
typedef int (*cuModuleGetFunction_t)(void**, void*, const char*);
typedef int (*cuLaunchKernel_t)(void*, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, void*, void**, void**);
typedef int (*cuModuleUnload_t)(void*);
typedef int (*cuCtxSynchronize_t)(void);
typedef int (*cuGetErrorString_t)(int, const char**);
struct Drv {
    void* so = nullptr; cuModuleLoadData_t load; cuModuleGetFunction_t getf; cuLaunchKernel_t launch;
    cuModuleUnload_t unload; cuCtxSynchronize_t sync; cuGetErrorString_t errstr;
};
Drv* drv() {
    static Drv d; static bool tried = false;
    if (tried) return d.so ? &d : nullptr;
    tried = true;
    void* so = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!so) return nullptr;
    d.load = (cuModuleLoadData_t)dlsym(so, "cuModuleLoadData");
    d.getf = (cuModuleGetFunction_t)dlsym(so, "cuModuleGetFunction");
    d.launch = (cuLaunchKernel_t)dlsym(so, "cuLaunchKernel");
    d.unload = (cuModuleUnload_t)dlsym(so, "cuModuleUnload");
    d.sync = (cuCtxSynchronize_t)dlsym(so, "cuCtxSynchronize");
    d.errstr = (cuGetErrorString_t)dlsym(so, "cuGetErrorString");
    if (!d.load || !d.getf || !d.launch || !d.unload || !d.sync) return nullptr;
    d.so = so;
    return &d;
}
int drv_fail(Drv* d, int rc, const char* what) {
    const char* s = nullptr;
    if (d->errstr) d->errstr(rc, &s);
    return hx_fail(HX_ERR_CUDA, "%s failed: %s (CUresult %d)", what, s ? s : "?", rc);
}
}  // namespace

HX_API int hx_image_open(void** module, const char* path) {
    HX_CHECK_ARG(module && path);
    Drv* d = drv();
    if (!d) return hx_fail(HX_ERR_CUDA, "libcuda.so.1 is not available");
    HX_CUDA(cudaFree(0));                       // make the primary context current
    FILE* f = fopen(path, "rb");
    if (!f) return hx_fail(HX_ERR_IO, "cannot open %s", path);
    std::vector<char> buf;
    char tmp[65536]; size_t got;
    while ((got = fread(tmp, 1, sizeof(tmp), f)) > 0) buf.insert(buf.end(), tmp, tmp + got);
    fclose(f);
    buf.push_back(0);                           // the reference appends a NUL (PTX is text)
    int rc = d->load(module, buf.data());
    if (rc) return drv_fail(d, rc, "cuModuleLoadData");
    return HX_OK;
}
HX_API int hx_image_launch(void* module, const char* entry, unsigned gx, unsigned gy, unsigned gz,
                           unsigned bx, unsigned by, unsigned bz, void** args) {
    HX_CHECK_ARG(module && entry && args);
    Drv* d = drv();
    if (!d) return hx_fail(HX_ERR_CUDA, "libcuda.so.1 is not available");
    void* fn = nullptr;
    int rc = d->getf(&fn, module, entry);
    if (rc) return drv_fail(d, rc, "cuModuleGetFunction");
    rc = d->launch(fn, gx, gy, gz, bx, by, bz, 0, nullptr, args, nullptr);
    if (rc) return drv_fail(d, rc, "cuLaunchKernel");
    rc = d->sync();
    if (rc) return drv_fail(d, rc, "cuCtxSynchronize");
    g_hx_launches += 1;
    return HX_OK;
}
HX_API int hx_image_close(void* module) {
    Drv* d = drv();
    if (d && module) d->unload(module);
    return HX_OK;
}
