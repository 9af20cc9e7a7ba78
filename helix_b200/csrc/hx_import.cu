// hx_import.cu -- safetensors checkpoint (single file or sharded, F32 or BF16) -> HXGW v3 NVFP4 file, on the GPU.
//
// Replaces pack_qwen3, helixc/runtime/gpt2_pack.c:587-733, with the same file bytes out: header (:648-658),
// 32-byte descriptors (:622-644), data in the order of build_order_llama(qwen3=1) (:255-281), the packed
// tensors quantized by the forward quantizer (hx_quant.cu, bit-exact with nvfp4_quantize_tensor), the dense ones
// (norm gains, embedding) widened to f32.  Then the reference's verify step (:692-732): the written file is read
// back, every packed tensor is dequantized from the file's bytes and compared with the source (worst relative
// RMS error must stay below 0.15), every dense tensor must be bit-exact.
//
// Data flow: shard files are mapped; a tensor's bytes go to the device through two pinned staging buffers
// (copy of chunk i+1 from the page cache overlaps the transfer of chunk i), are widened there if BF16,
// quantized there, and the results come back through the same staging buffers straight into fwrite.
#include "hx_common.cuh"
#include <errno.h>
#include <fcntl.h>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

namespace {

struct SrcTensor { std::string name; std::vector<long> shape; bool bf16 = false; const unsigned char* data = nullptr; size_t nbytes = 0; };
struct Shard { int fd = -1; size_t len = 0; unsigned char* base = nullptr; };

long numel(const std::vector<long>& s) { long p = 1; for (long v : s) p *= v; return p; }

bool read_text(const std::string& path, std::string& out) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return false;
    char buf[65536]; size_t n;
    out.clear();
    while ((n = fread(buf, 1, sizeof(buf), f)) > 0) out.append(buf, n);
    fclose(f);
    return true;
}

// ---- a JSON reader for the two shapes of text met here: flat config objects and the safetensors header ----
struct Json {
    const char* p; const char* end;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
    bool lit(char c) { ws(); if (p < end && *p == c) { p++; return true; } return false; }
    bool str(std::string& s) {
        ws(); if (p >= end || *p != '"') return false;
        p++; s.clear();
        while (p < end && *p != '"') { if (*p == '\\' && p + 1 < end) { p++; } s.push_back(*p++); }
        if (p >= end) return false;
        p++; return true;
    }
    bool num(double& v) {
        ws(); char* e = nullptr; v = strtod(p, &e);
        if (e == p) return false;
        p = e; return true;
    }
    // skips any value
    bool skip() {
        ws(); if (p >= end) return false;
        if (*p == '"') { std::string s; return str(s); }
        if (*p == '{' || *p == '[') {
            const char open = *p, close = open == '{' ? '}' : ']';
            p++;
            if (lit(close)) return true;
            for (;;) {
                if (open == '{') { std::string k; if (!str(k) || !lit(':')) return false; }
                if (!skip()) return false;
                if (lit(',')) continue;
                return lit(close);
            }
        }
        while (p < end && *p != ',' && *p != '}' && *p != ']') p++;      // number, true, false, null
        return true;
    }
};

// top-level "key": number of a flat JSON object
bool json_number(const std::string& text, const char* key, double& out) {
    Json j{text.data(), text.data() + text.size()};
    if (!j.lit('{')) return false;
    if (j.lit('}')) return false;
    for (;;) {
        std::string k;
        if (!j.str(k) || !j.lit(':')) return false;
        if (k == key) return j.num(out);
        if (!j.skip()) return false;
        if (!j.lit(',')) return false;
    }
}

// the header of one safetensors file: {"name": {"dtype": "F32"|"BF16", "shape": [...], "data_offsets": [a, b]}, ...}
int parse_header(const char* js, size_t n, const unsigned char* blob, size_t blob_len, std::vector<SrcTensor>& out) {
    Json j{js, js + n};
    if (!j.lit('{')) return hx_fail(HX_ERR_FORMAT, "safetensors header: not an object");
    if (j.lit('}')) return HX_OK;
    for (;;) {
        std::string name;
        if (!j.str(name) || !j.lit(':')) return hx_fail(HX_ERR_FORMAT, "safetensors header: bad key");
        if (name == "__metadata__") { if (!j.skip()) return hx_fail(HX_ERR_FORMAT, "safetensors header: bad metadata"); }
        else {
            SrcTensor t; t.name = name;
            std::string dtype; double a = -1, b = -1;
            if (!j.lit('{')) return hx_fail(HX_ERR_FORMAT, "safetensors header: tensor %s is not an object", name.c_str());
            for (;;) {
                std::string f;
                if (!j.str(f) || !j.lit(':')) return hx_fail(HX_ERR_FORMAT, "safetensors header: bad field in %s", name.c_str());
                if (f == "dtype") { if (!j.str(dtype)) return hx_fail(HX_ERR_FORMAT, "safetensors header: dtype of %s", name.c_str()); }
                else if (f == "shape") {
                    if (!j.lit('[')) return hx_fail(HX_ERR_FORMAT, "safetensors header: shape of %s", name.c_str());
                    if (!j.lit(']')) for (;;) { double v; if (!j.num(v)) return hx_fail(HX_ERR_FORMAT, "safetensors header: shape of %s", name.c_str());
                                               t.shape.push_back((long)v); if (j.lit(',')) continue; if (j.lit(']')) break; return hx_fail(HX_ERR_FORMAT, "safetensors header: shape of %s", name.c_str()); }
                } else if (f == "data_offsets") {
                    if (!j.lit('[') || !j.num(a) || !j.lit(',') || !j.num(b) || !j.lit(']')) return hx_fail(HX_ERR_FORMAT, "safetensors header: offsets of %s", name.c_str());
                } else if (!j.skip()) return hx_fail(HX_ERR_FORMAT, "safetensors header: field %s of %s", f.c_str(), name.c_str());
                if (j.lit(',')) continue;
                if (j.lit('}')) break;
                return hx_fail(HX_ERR_FORMAT, "safetensors header: tensor %s", name.c_str());
            }
            if (dtype == "F32") t.bf16 = false; else if (dtype == "BF16") t.bf16 = true;
            else return hx_fail(HX_ERR_FORMAT, "tensor %s has dtype %s, not F32 or BF16", name.c_str(), dtype.c_str());
            const size_t want = (size_t)numel(t.shape) * (t.bf16 ? 2 : 4);
            if (a < 0 || b < a || (size_t)b > blob_len || (size_t)(b - a) != want)
                return hx_fail(HX_ERR_FORMAT, "tensor %s: data_offsets [%.0f, %.0f) do not hold its %zu bytes", name.c_str(), a, b, want);
            t.data = blob + (size_t)a; t.nbytes = want;
            out.push_back(std::move(t));
        }
        if (j.lit(',')) continue;
        if (j.lit('}')) return HX_OK;
        return hx_fail(HX_ERR_FORMAT, "safetensors header: truncated");
    }
}

// the unique shard file names an index.json mentions, in order of first appearance (index_shards, gpt2_pack.c:511-531)
std::vector<std::string> shard_names(const std::string& index_json) {
    std::vector<std::string> names;
    const std::string needle = ".safetensors\"";
    size_t at = 0;
    while ((at = index_json.find(needle, at)) != std::string::npos) {
        size_t q = index_json.rfind('"', at);
        if (q != std::string::npos) {
            std::string nm = index_json.substr(q + 1, at + needle.size() - 1 - (q + 1));
            bool seen = false;
            for (auto& s : names) if (s == nm) seen = true;
            if (!seen && !nm.empty()) names.push_back(nm);
        }
        at += needle.size();
    }
    return names;
}

struct OrderEntry { std::string name; std::vector<long> shape; bool packed; };

__global__ void k_widen_bf16(const uint16_t* __restrict__ src, float* __restrict__ dst, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = __uint_as_float((uint32_t)src[i] << 16);
}
// sums of squared error and squared source over the [rows][K] part of a [rows][Kpad] reconstruction
__global__ void k_rms_err(const float* __restrict__ w, const float* __restrict__ rec, int rows, int K, int Kpad, double* __restrict__ acc) {
    double se = 0.0, sw = 0.0;
    const size_t n = (size_t)rows * K;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / K, k = i - r * K;
        const float o = w[i], g = rec[r * Kpad + k];
        const double d = (double)g - (double)o;
        se += d * d; sw += (double)o * (double)o;
    }
    for (int off = 16; off >= 1; off >>= 1) { se += __shfl_xor_sync(0xffffffffu, se, off); sw += __shfl_xor_sync(0xffffffffu, sw, off); }
    if ((threadIdx.x & 31) == 0) { atomicAdd(acc, se); atomicAdd(acc + 1, sw); }
}
__global__ void k_count_diff(const uint32_t* __restrict__ a, const uint32_t* __restrict__ b, size_t n, unsigned long long* __restrict__ cnt) {
    unsigned long long c = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) c += a[i] != b[i];
    if (c) atomicAdd(cnt, c);
}

// Host <-> device streaming through two pinned staging buffers.
struct Stager {
    static constexpr size_t CHUNK = (size_t)32 << 20;
    unsigned char* pin[2] = {nullptr, nullptr};
    cudaEvent_t ev[2] = {nullptr, nullptr};
    cudaStream_t st = nullptr;
    int init() {
        HX_CUDA(cudaStreamCreate(&st));
        for (int i = 0; i < 2; i++) { HX_CUDA(cudaMallocHost((void**)&pin[i], CHUNK)); HX_CUDA(cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming)); }
        return HX_OK;
    }
    ~Stager() { for (int i = 0; i < 2; i++) { if (pin[i]) cudaFreeHost(pin[i]); if (ev[i]) cudaEventDestroy(ev[i]); } if (st) cudaStreamDestroy(st); }
    // host memory (a mapped file) -> device
    int up(void* dst, const unsigned char* src, size_t n) {
        int k = 0;
        for (size_t o = 0; o < n; o += CHUNK, k ^= 1) {
            const size_t m = n - o < CHUNK ? n - o : CHUNK;
            HX_CUDA(cudaEventSynchronize(ev[k]));                 // the transfer that last used this buffer is done
            memcpy(pin[k], src + o, m);
            HX_CUDA(cudaMemcpyAsync((unsigned char*)dst + o, pin[k], m, cudaMemcpyHostToDevice, st));
            HX_CUDA(cudaEventRecord(ev[k], st));
        }
        return HX_OK;
    }
    // device -> file: chunks alternate between the two buffers, so writing chunk i overlaps the transfer of chunk i+1
    int down(FILE* f, const void* src, size_t n) {
        size_t held[2] = {0, 0};
        size_t o = 0;
        for (int k = 0; o < n || held[0] || held[1]; k ^= 1) {
            if (held[k]) {
                HX_CUDA(cudaEventSynchronize(ev[k]));
                if (fwrite(pin[k], 1, held[k], f) != held[k]) return hx_fail(HX_ERR_IO, "write failed: %s", strerror(errno));
                held[k] = 0;
            }
            if (o < n) {
                const size_t m = n - o < CHUNK ? n - o : CHUNK;
                HX_CUDA(cudaMemcpyAsync(pin[k], (const unsigned char*)src + o, m, cudaMemcpyDeviceToHost, st));
                HX_CUDA(cudaEventRecord(ev[k], st));
                held[k] = m; o += m;
            }
        }
        return HX_OK;
    }
};

struct DevBuf {
    void* p = nullptr; size_t cap = 0;
    ~DevBuf() { if (p) cudaFree(p); }
    int need(size_t n) {
        if (n <= cap) return HX_OK;
        if (p) { cudaFree(p); p = nullptr; cap = 0; }
        if (cudaMalloc(&p, n) != cudaSuccess) return hx_fail(HX_ERR_NOMEM, "device allocation of %zu bytes failed", n);
        cap = n; return HX_OK;
    }
};

struct Importer {
    std::vector<Shard> shards; std::vector<SrcTensor> src;
    Stager sg; DevBuf raw, f32, words, micro, rec, misc;
    ~Importer() { for (auto& s : shards) { if (s.base) munmap(s.base, s.len); if (s.fd >= 0) close(s.fd); } }
    const SrcTensor* find(const std::string& n) const { for (auto& t : src) if (t.name == n) return &t; return nullptr; }

    int open_shard(const std::string& path) {
        Shard s;
        s.fd = open(path.c_str(), O_RDONLY);
        if (s.fd < 0) return hx_fail(HX_ERR_IO, "open %s: %s", path.c_str(), strerror(errno));
        struct stat st;
        if (fstat(s.fd, &st) != 0 || st.st_size < 8) { close(s.fd); return hx_fail(HX_ERR_FORMAT, "%s is too short for a safetensors file", path.c_str()); }
        s.len = (size_t)st.st_size;
        s.base = (unsigned char*)mmap(nullptr, s.len, PROT_READ, MAP_PRIVATE, s.fd, 0);
        if (s.base == MAP_FAILED) { close(s.fd); return hx_fail(HX_ERR_IO, "mmap %s: %s", path.c_str(), strerror(errno)); }
        shards.push_back(s);
        uint64_t hlen; memcpy(&hlen, s.base, 8);
        if (hlen > s.len - 8) return hx_fail(HX_ERR_FORMAT, "%s: header length %llu exceeds the file", path.c_str(), (unsigned long long)hlen);
        return parse_header((const char*)s.base + 8, (size_t)hlen, s.base + 8 + hlen, s.len - 8 - (size_t)hlen, src);
    }

    // the tensor as f32 on the device (in `f32`)
    int materialize(const SrcTensor& t) {
        const size_t n = (size_t)numel(t.shape);
        int rc;
        if ((rc = f32.need(n * 4))) return rc;
        if (!t.bf16) return sg.up(f32.p, t.data, n * 4);
        if ((rc = raw.need(n * 2))) return rc;
        if ((rc = sg.up(raw.p, t.data, n * 2))) return rc;
        int g = (int)((n + 255) / 256); if (g > 148 * 16) g = 148 * 16;
        k_widen_bf16<<<g, 256, 0, sg.st>>>((const uint16_t*)raw.p, (float*)f32.p, n);
        HX_COUNT_LAUNCH(1);
        HX_CUDA(cudaGetLastError());
        return HX_OK;
    }
};

}  // namespace

HX_API int hx_pack_qwen3(const char* model_dir, const char* out_path, int verify, hx_pack_report* rep) {
    HX_CHECK_ARG(model_dir && out_path);
    if (rep) memset(rep, 0, sizeof(*rep));
    const std::string dir = model_dir;
    // ---- config.json (:588-607): six required integers, defaults for the rest ----
    std::string cfg;
    if (!read_text(dir + "/config.json", cfg)) return hx_fail(HX_ERR_IO, "open %s/config.json: %s", model_dir, strerror(errno));
    double NL, DM, NH, NKV, DF, NV, NC, HD, theta, eps;
    if (!json_number(cfg, "num_hidden_layers", NL) || !json_number(cfg, "hidden_size", DM) || !json_number(cfg, "num_attention_heads", NH) ||
        !json_number(cfg, "num_key_value_heads", NKV) || !json_number(cfg, "intermediate_size", DF) || !json_number(cfg, "vocab_size", NV))
        return hx_fail(HX_ERR_FORMAT, "config.json lacks a required integer field");
    if (!json_number(cfg, "head_dim", HD)) HD = (double)((long)DM / (long)NH);
    if (!json_number(cfg, "max_position_embeddings", NC)) NC = 40960;
    if (!json_number(cfg, "rope_theta", theta)) theta = 1000000.0;
    if (!json_number(cfg, "rms_norm_eps", eps)) eps = 1e-6;
    if (NL < 1 || DM < 1 || NH < 1 || NKV < 1 || DF < 1 || NV < 1 || HD < 1) return hx_fail(HX_ERR_FORMAT, "config.json: non-positive dimension");
    const long nl = (long)NL, dm = (long)DM, nh = (long)NH, nkv = (long)NKV, df = (long)DF, nv = (long)NV, hd = (long)HD;
    const long qd = nh * hd, kvd = nkv * hd;

    Importer im;
    int rc = im.sg.init(); if (rc) return rc;
    // ---- shards (:533-571): the index names them, a lone model.safetensors otherwise ----
    {
        std::string idx;
        std::vector<std::string> names;
        if (read_text(dir + "/model.safetensors.index.json", idx)) {
            names = shard_names(idx);
            if (names.empty()) return hx_fail(HX_ERR_FORMAT, "model.safetensors.index.json names no shard file");
        } else names.push_back("model.safetensors");
        for (auto& n : names) if ((rc = im.open_shard(dir + "/" + n))) return rc;
    }
    // ---- order (:255-281) ----
    std::vector<OrderEntry> ord;
    for (long L = 0; L < nl; L++) {
        const std::string p = "model.layers." + std::to_string(L) + ".";
        ord.push_back({p + "input_layernorm.weight", {dm}, false});
        ord.push_back({p + "self_attn.q_proj.weight", {qd, dm}, true});
        ord.push_back({p + "self_attn.q_norm.weight", {hd}, false});
        ord.push_back({p + "self_attn.k_proj.weight", {kvd, dm}, true});
        ord.push_back({p + "self_attn.k_norm.weight", {hd}, false});
        ord.push_back({p + "self_attn.v_proj.weight", {kvd, dm}, true});
        ord.push_back({p + "self_attn.o_proj.weight", {dm, qd}, true});
        ord.push_back({p + "post_attention_layernorm.weight", {dm}, false});
        ord.push_back({p + "mlp.gate_proj.weight", {df, dm}, true});
        ord.push_back({p + "mlp.up_proj.weight", {df, dm}, true});
        ord.push_back({p + "mlp.down_proj.weight", {dm, df}, true});
    }
    ord.push_back({"model.embed_tokens.weight", {nv, dm}, false});
    ord.push_back({"model.norm.weight", {dm}, false});
    ord.push_back({"lm_head.weight", {nv, dm}, true});

    // ---- descriptors (:622-644) ----
    struct Desc { uint32_t packed, rows, K, Kpad; uint64_t data_off, scale_off; };
    static_assert(sizeof(Desc) == 32, "descriptor is 32 bytes");
    const int no = (int)ord.size();
    std::vector<Desc> desc(no);
    std::vector<const SrcTensor*> from(no);
    uint64_t cur = 64 + (uint64_t)no * 32;
    int n_packed = 0;
    for (int e = 0; e < no; e++) {
        const SrcTensor* t = im.find(ord[e].name);
        if (!t) return hx_fail(HX_ERR_FORMAT, "checkpoint lacks tensor %s", ord[e].name.c_str());
        const long want = numel(ord[e].shape), have = numel(t->shape);
        if (want != have) return hx_fail(HX_ERR_FORMAT, "%s holds %ld elements, expected %ld", ord[e].name.c_str(), have, want);
        from[e] = t;
        Desc& d = desc[e];
        if (ord[e].packed) {
            if (t->shape.size() != 2) return hx_fail(HX_ERR_FORMAT, "%s is not a matrix", ord[e].name.c_str());
            const int rows = (int)t->shape[0], K = (int)t->shape[1], Kpad = hx_kpad(K);
            d.packed = 1; d.rows = (uint32_t)rows; d.K = (uint32_t)K; d.Kpad = (uint32_t)Kpad;
            d.data_off = cur;
            const uint64_t wbytes = (uint64_t)rows * (Kpad / 7) * 4;
            d.scale_off = cur + wbytes;
            cur += wbytes + (uint64_t)rows * (Kpad / 16) + 4;
            n_packed++;
        } else {
            d.packed = 0; d.rows = 1; d.K = (uint32_t)have; d.Kpad = (uint32_t)have; d.data_off = cur; d.scale_off = 0;
            cur += (uint64_t)have * 4;
        }
    }
    const uint64_t total = cur;

    cudaEvent_t e0, e1, e2;
    HX_CUDA(cudaEventCreate(&e0)); HX_CUDA(cudaEventCreate(&e1)); HX_CUDA(cudaEventCreate(&e2));
    struct EvGuard { cudaEvent_t a, b, c; ~EvGuard() { cudaEventDestroy(a); cudaEventDestroy(b); cudaEventDestroy(c); } } evg{e0, e1, e2};
    cudaEventRecord(e0, im.sg.st);

    // ---- write ----
    FILE* of = fopen(out_path, "wb");
    if (!of) return hx_fail(HX_ERR_IO, "open %s: %s", out_path, strerror(errno));
    struct FileGuard { FILE* f; ~FileGuard() { if (f) fclose(f); } } fg{of};
    {
        unsigned char hdr[64]; memset(hdr, 0, sizeof(hdr));
        const uint32_t h32[8] = {0x48584757u, 3u, (uint32_t)nl, (uint32_t)dm, (uint32_t)nh, (uint32_t)nv, (uint32_t)(long)NC, (uint32_t)df};
        memcpy(hdr, h32, 32);
        const uint32_t arch = 1u, nkv32 = (uint32_t)nkv, hd32 = (uint32_t)hd, nt32 = (uint32_t)no;
        const float th = (float)theta, ep = (float)eps;
        memcpy(hdr + 40, &arch, 4); memcpy(hdr + 44, &nkv32, 4); memcpy(hdr + 48, &th, 4); memcpy(hdr + 52, &ep, 4);
        memcpy(hdr + 56, &hd32, 4); memcpy(hdr + 60, &nt32, 4);
        if (fwrite(hdr, 1, 64, of) != 64 || fwrite(desc.data(), 32, (size_t)no, of) != (size_t)no) return hx_fail(HX_ERR_IO, "write %s: %s", out_path, strerror(errno));
    }
    for (int e = 0; e < no; e++) {
        const SrcTensor& t = *from[e];
        const Desc& d = desc[e];
        if ((uint64_t)ftell(of) != d.data_off) return hx_fail(HX_ERR_IO, "offset drift at %s", t.name.c_str());
        if ((rc = im.materialize(t))) return rc;
        if (d.packed) {
            const size_t nw = (size_t)d.rows * (d.Kpad / 7) * 4, nm = (size_t)d.rows * (d.Kpad / 16);
            if ((rc = im.words.need(nw)) || (rc = im.micro.need(nm + 4 + 16))) return rc;
            // micro bytes and, right behind them (4-byte aligned), the tensor scale: the file wants them adjacent
            const size_t ts_off = (nm + 3) & ~(size_t)3;
            float* ts_dev = (float*)((unsigned char*)im.micro.p + ts_off);
            if ((rc = hx_quantize_nvfp4((const float*)im.f32.p, (int)d.rows, (int)d.K, (int32_t*)im.words.p, (uint8_t*)im.micro.p, nullptr, ts_dev, im.sg.st))) return rc;
            if ((rc = im.sg.down(of, im.words.p, nw))) return rc;
            if ((rc = im.sg.down(of, im.micro.p, nm))) return rc;
            if ((rc = im.sg.down(of, ts_dev, 4))) return rc;
        } else if ((rc = im.sg.down(of, im.f32.p, (size_t)d.K * 4))) return rc;
    }
    if ((uint64_t)ftell(of) != total) return hx_fail(HX_ERR_IO, "wrote %ld bytes, expected %llu", ftell(of), (unsigned long long)total);
    fg.f = nullptr;
    if (fclose(of) != 0) return hx_fail(HX_ERR_IO, "close %s: %s", out_path, strerror(errno));
    cudaEventRecord(e1, im.sg.st);

    // ---- verify (:692-732): from the bytes of the written file ----
    double worst = 0.0; int worst_e = -1; bool f32_exact = true;
    if (verify) {
        Shard v;
        v.fd = open(out_path, O_RDONLY);
        if (v.fd < 0) return hx_fail(HX_ERR_IO, "reopen %s: %s", out_path, strerror(errno));
        struct stat st; fstat(v.fd, &st);
        v.len = (size_t)st.st_size;
        v.base = (unsigned char*)mmap(nullptr, v.len, PROT_READ, MAP_PRIVATE, v.fd, 0);
        if (v.base == MAP_FAILED) { close(v.fd); return hx_fail(HX_ERR_IO, "mmap %s: %s", out_path, strerror(errno)); }
        im.shards.push_back(v);                                   // unmapped with the others
        if (v.len != total) return hx_fail(HX_ERR_IO, "%s has %zu bytes, expected %llu", out_path, v.len, (unsigned long long)total);
        const Desc* vd = (const Desc*)(v.base + 64);
        if ((rc = im.misc.need(64))) return rc;
        for (int e = 0; e < no && !rc; e++) {
            const SrcTensor& t = *from[e];
            if ((rc = im.materialize(t))) break;
            if (vd[e].packed) {
                const int rows = (int)vd[e].rows, K = (int)vd[e].K, Kpad = (int)vd[e].Kpad;
                const size_t nw = (size_t)rows * (Kpad / 7) * 4, nm = (size_t)rows * (Kpad / 16);
                const size_t ts_off = (nm + 3) & ~(size_t)3;
                if ((rc = im.words.need(nw)) || (rc = im.micro.need(ts_off + 4)) || (rc = im.rec.need((size_t)rows * Kpad * 4))) break;
                if ((rc = im.sg.up(im.words.p, v.base + vd[e].data_off, nw))) break;
                if ((rc = im.sg.up(im.micro.p, v.base + vd[e].scale_off, nm))) break;
                if ((rc = im.sg.up((unsigned char*)im.micro.p + ts_off, v.base + vd[e].scale_off + nm, 4))) break;
                if ((rc = hx_dequant_nvfp4((const int32_t*)im.words.p, (const uint8_t*)im.micro.p, (const float*)((unsigned char*)im.micro.p + ts_off), nullptr,
                                           (float*)im.rec.p, rows, Kpad, im.sg.st))) break;
                cudaMemsetAsync(im.misc.p, 0, 16, im.sg.st);
                k_rms_err<<<148 * 4, 256, 0, im.sg.st>>>((const float*)im.f32.p, (const float*)im.rec.p, rows, K, Kpad, (double*)im.misc.p);
                HX_COUNT_LAUNCH(1);
                double acc[2];
                HX_CUDA(cudaMemcpyAsync(acc, im.misc.p, 16, cudaMemcpyDeviceToHost, im.sg.st));
                HX_CUDA(cudaStreamSynchronize(im.sg.st));
                const double cnt = (double)rows * K, rmse = sqrt(acc[0] / cnt), rms_w = sqrt(acc[1] / cnt);
                const double rel = rms_w > 0 ? rmse / rms_w : 0.0;
                if (rel > worst) { worst = rel; worst_e = e; }
            } else {
                const size_t n = (size_t)vd[e].K;
                if ((rc = im.rec.need(n * 4))) break;
                if ((rc = im.sg.up(im.rec.p, v.base + vd[e].data_off, n * 4))) break;
                cudaMemsetAsync(im.misc.p, 0, 16, im.sg.st);
                int g = (int)((n + 255) / 256); if (g > 148 * 8) g = 148 * 8;
                k_count_diff<<<g, 256, 0, im.sg.st>>>((const uint32_t*)im.f32.p, (const uint32_t*)im.rec.p, n, (unsigned long long*)im.misc.p);
                HX_COUNT_LAUNCH(1);
                unsigned long long bad = 0;
                HX_CUDA(cudaMemcpyAsync(&bad, im.misc.p, 8, cudaMemcpyDeviceToHost, im.sg.st));
                HX_CUDA(cudaStreamSynchronize(im.sg.st));
                if (bad) f32_exact = false;
            }
        }
        if (rc) return rc;
    }
    cudaEventRecord(e2, im.sg.st);
    HX_CUDA(cudaStreamSynchronize(im.sg.st));
    if (rep) {
        rep->tensors = no; rep->packed = n_packed; rep->bytes = total; rep->worst_rms = worst; rep->f32_exact = f32_exact ? 1 : 0; rep->verified = verify ? 1 : 0;
        if (worst_e >= 0) snprintf(rep->worst_name, sizeof(rep->worst_name), "%s", ord[worst_e].name.c_str());
        cudaEventElapsedTime(&rep->ms_pack, e0, e1); cudaEventElapsedTime(&rep->ms_verify, e1, e2);
    }
    if (verify && !(worst < 0.15 && f32_exact))
        return hx_fail(HX_ERR_FORMAT, "verify failed: worst relative RMS error %.4f (%s), dense tensors %s", worst,
                       worst_e >= 0 ? ord[worst_e].name.c_str() : "-", f32_exact ? "exact" : "NOT exact");
    return HX_OK;
}
