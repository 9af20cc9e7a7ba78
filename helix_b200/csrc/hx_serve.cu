// hx_serve.cu -- the worker protocol of the reference's --serve mode on top of this library, and its seeded sampler.
//
// Replaces run_serve, helixc/runtime/gpt2_infer.c:3284-3400: one request frame per input line
//   {"ids":[..],"n_gen":N,"request_id":"..", sampling fields}   or   {"cmd":"quit"}
// and newline-delimited JSON events on the output: hello, tokenize, then per generated token forward_begin and
// token, then done (event formats :845-1121).  The per-op / per-layer telemetry of the reference (op, layer_begin,
// layer_end, head, the logit lens) describes its own launch sequence and has no counterpart in a one-kernel token;
// the stream emitted here is the one the reference emits for "detail":"token" requests.  No tokenizer is linked:
// a frame must carry "ids"; a "prompt" frame gets the reference's own error for that case.
//
// The sampler is sample_next, :1660-1711, operation for operation in double precision: repetition penalty,
// frequency / presence penalties, temperature, top-k, soft-max, sort by (-p, id), top-p (crossing token kept),
// min-p, renormalise, one PCG32 draw, first index whose running sum passes it.  temperature 0 is the arg-max.
// All of this is host code; the forward passes are hx_prefill / hx_decode_step.
#include "hx_common.cuh"
#include <algorithm>
#include <string>
#include <time.h>
#include <unistd.h>
#include <vector>

struct hx_sampler {
    int vocab = 0;
    hx_sample_config cfg = {0.0, 1.0, 0.0, 1.0, 0.0, 0.0, 0, 0};
    std::vector<unsigned short> count;
    bool counting = false;                            // the reference's count array exists only after its first sample_reset
    uint64_t state = 0, inc = 0;                      // unseeded, like the reference's zero-initialised generator
    std::vector<std::pair<double, int>> cand;         // (value, id)
};

namespace {

void pcg_seed(hx_sampler* s, uint64_t seed) {          // pcg32_seed, :1632-1637
    s->state = 0u; s->inc = (54u << 1) | 1u;
    s->state = s->state * 6364136223846793005ULL + s->inc;
    s->state += seed;
    s->state = s->state * 6364136223846793005ULL + s->inc;
}
uint32_t pcg_next(hx_sampler* s) {                     // pcg32_next, :1638-1644
    const uint64_t old = s->state;
    s->state = old * 6364136223846793005ULL + s->inc;
    const uint32_t x = (uint32_t)(((old >> 18) ^ old) >> 27), rot = (uint32_t)(old >> 59);
    return (x >> rot) | (x << ((32 - rot) & 31));
}

}  // namespace

HX_API int hx_sampler_create(hx_sampler** out, int vocab) {
    HX_CHECK_ARG(out && vocab > 0);
    hx_sampler* s = new hx_sampler();
    s->vocab = vocab; s->count.assign((size_t)vocab, 0);
    *out = s;
    return HX_OK;
}
HX_API int hx_sampler_free(hx_sampler* s) { delete s; return HX_OK; }

// The parameters alone, with the limits of sample_cfg_from_json, :1729-1732.
HX_API int hx_sampler_configure(hx_sampler* s, const hx_sample_config* cfg) {
    HX_CHECK_ARG(s && cfg);
    s->cfg = *cfg;
    if (s->cfg.temperature < 0.0) s->cfg.temperature = 0.0;
    if (s->cfg.temperature > 4.0) s->cfg.temperature = 4.0;
    if (s->cfg.top_p <= 0.0 || s->cfg.top_p > 1.0) s->cfg.top_p = 1.0;
    if (s->cfg.rep_penalty <= 0.0) s->cfg.rep_penalty = 1.0;
    return HX_OK;
}
// sample_reset, :1651-1657: the prompt counted, the generator seeded.
HX_API int hx_sampler_reset(hx_sampler* s, const hx_sample_config* cfg, const int32_t* prompt, int n_prompt) {
    HX_CHECK_ARG(s && cfg && (prompt || n_prompt == 0));
    hx_sampler_configure(s, cfg);
    s->counting = true;
    std::fill(s->count.begin(), s->count.end(), (unsigned short)0);
    for (int i = 0; i < n_prompt; i++)
        if (prompt[i] >= 0 && prompt[i] < s->vocab && s->count[prompt[i]] < 65535) s->count[prompt[i]]++;
    pcg_seed(s, s->cfg.seed);
    return HX_OK;
}
HX_API int hx_sampler_count(hx_sampler* s, int32_t id) {          // sample_count, :1658-1660
    HX_CHECK_ARG(s);
    if (s->counting && id >= 0 && id < s->vocab && s->count[id] < 65535) s->count[id]++;
    return HX_OK;
}

HX_API int hx_sampler_next(hx_sampler* s, const float* logits, int32_t* id) {
    HX_CHECK_ARG(s && logits && id);
    const int nv = s->vocab;
    const hx_sample_config& c = s->cfg;
    if (!(c.temperature > 0.0)) {                                   // argmax_row, :1735-1739: first maximum
        int a = 0; float best = logits[0];
        for (int i = 1; i < nv; i++) if (logits[i] > best) { best = logits[i]; a = i; }
        *id = a;
        return HX_OK;
    }
    s->cand.resize((size_t)nv);
    const double invt = 1.0 / c.temperature;
    for (int i = 0; i < nv; i++) {
        double x = (double)logits[i];
        const int n = (int)s->count[i];
        if (n > 0 && c.rep_penalty != 1.0) x = (x > 0.0) ? x / c.rep_penalty : x * c.rep_penalty;
        if (n > 0) x -= c.freq_penalty * (double)n + c.pres_penalty;
        s->cand[i] = std::make_pair(x * invt, i);
    }
    std::sort(s->cand.begin(), s->cand.end(), [](const std::pair<double, int>& a, const std::pair<double, int>& b) {
        if (a.first > b.first) return true;
        if (a.first < b.first) return false;
        return a.second < b.second;
    });
    int n = (c.top_k > 0 && c.top_k < nv) ? c.top_k : nv;
    const double mx = s->cand[0].first;
    double sum = 0.0;
    for (int i = 0; i < n; i++) { s->cand[i].first = exp(s->cand[i].first - mx); sum += s->cand[i].first; }
    for (int i = 0; i < n; i++) s->cand[i].first /= sum;
    if (c.top_p < 1.0) {
        double cum = 0.0; int keep = n;
        for (int i = 0; i < n; i++) { cum += s->cand[i].first; if (cum >= c.top_p) { keep = i + 1; break; } }
        n = keep;
    }
    if (c.min_p > 0.0) {
        const double floor_p = c.min_p * s->cand[0].first;
        int keep = n;
        for (int i = 0; i < n; i++) if (s->cand[i].first < floor_p) { keep = i; break; }
        n = keep > 0 ? keep : 1;
    }
    double rsum = 0.0;
    for (int i = 0; i < n; i++) rsum += s->cand[i].first;
    const double u = (double)pcg_next(s) / 4294967296.0;
    double cum = 0.0; int pick = s->cand[n - 1].second;
    for (int i = 0; i < n; i++) { cum += s->cand[i].first / rsum; if (cum > u) { pick = s->cand[i].second; break; } }
    *id = pick;
    return HX_OK;
}

// ---- the request loop -------------------------------------------------------------------------------------
namespace {

struct Emitter {
    int fd; long seq = 0;
    void raw(const std::string& s) {
        size_t off = 0;
        while (off < s.size()) { const ssize_t w = write(fd, s.data() + off, s.size() - off); if (w <= 0) break; off += (size_t)w; }
    }
    void error(const char* where, const char* msg, bool fatal) {
        char b[768];
        snprintf(b, sizeof b, "{\"_ev\":\"error\",\"seq\":%ld,\"where\":\"%s\",\"message\":\"%s\",\"fatal\":%s}\n", seq++, where, msg, fatal ? "true" : "false");
        raw(b);
    }
};

// the value that follows the first "key": in the line (json_find_key, :3214-3225), or nullptr
const char* find_key(const char* s, const char* key) {
    char pat[64]; snprintf(pat, sizeof pat, "\"%s\"", key);
    const char* p = strstr(s, pat);
    if (!p) return nullptr;
    p += strlen(pat);
    while (*p == ' ' || *p == '\t') p++;
    if (*p != ':') return nullptr;
    p++;
    while (*p == ' ' || *p == '\t') p++;
    return p;
}

// JSON string escaping of a byte string (jesc, :822-843): quotes, backslashes, \n \r \t, other control bytes as
// \u00XX, everything else verbatim
std::string jesc(const std::string& in) {
    static const char* H = "0123456789abcdef";
    std::string out;
    for (unsigned char c : in) {
        switch (c) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\r': out += "\\r"; break;
            case '\t': out += "\\t"; break;
            default:
                if (c < 0x20) { out += "\\u00"; out.push_back(H[(c >> 4) & 0xF]); out.push_back(H[c & 0xF]); }
                else out.push_back((char)c);
        }
    }
    return out;
}

// the JSON string that starts at p (after its opening quote): escapes \n \t \r \" \\ \/ and \uXXXX (as UTF-8)
// undone (parse_req_json, :3238-3266)
std::string json_unescape(const char* p) {
    std::string out;
    while (*p && *p != '"') {
        if (*p == '\\' && p[1]) {
            p++;
            switch (*p) {
                case 'n': out.push_back('\n'); break; case 't': out.push_back('\t'); break; case 'r': out.push_back('\r'); break;
                case '"': out.push_back('"'); break; case '\\': out.push_back('\\'); break; case '/': out.push_back('/'); break;
                case 'u': {
                    unsigned v = 0;
                    for (int i = 0; i < 4 && p[1]; i++) {
                        p++; const char h = *p; v <<= 4;
                        if (h >= '0' && h <= '9') v |= (unsigned)(h - '0'); else if (h >= 'a' && h <= 'f') v |= (unsigned)(h - 'a' + 10);
                        else if (h >= 'A' && h <= 'F') v |= (unsigned)(h - 'A' + 10);
                    }
                    if (v < 0x80) out.push_back((char)v);
                    else if (v < 0x800) { out.push_back((char)(0xC0 | (v >> 6))); out.push_back((char)(0x80 | (v & 0x3F))); }
                    else { out.push_back((char)(0xE0 | (v >> 12))); out.push_back((char)(0x80 | ((v >> 6) & 0x3F))); out.push_back((char)(0x80 | (v & 0x3F))); }
                    break;
                }
                default: out.push_back(*p); break;
            }
            p++;
        } else out.push_back(*p++);
    }
    return out;
}

std::string decode_ids(const hx_tokenizer* tok, const int32_t* ids, int n) {
    if (!tok || n <= 0) return std::string();
    size_t len = 0;
    hx_tokenizer_decode(tok, ids, n, nullptr, 0, &len);           // sizes the text (the call reports the short buffer)
    std::string out(len, '\0');
    if (len) hx_tokenizer_decode(tok, ids, n, &out[0], len, &len);
    return out;
}

double now_s() { struct timespec ts; clock_gettime(CLOCK_MONOTONIC, &ts); return (double)ts.tv_sec + (double)ts.tv_nsec * 1e-9; }

}  // namespace

HX_API int hx_serve(hx_model* m, int in_fd, int out_fd, int max_ctx) { return hx_serve_text(m, nullptr, 0, -1, in_fd, out_fd, max_ctx); }

HX_API int hx_serve_text(hx_model* m, const hx_tokenizer* tok, int with_specials, int eos_id, int in_fd, int out_fd, int max_ctx) {
    HX_CHECK_ARG(m && in_fd >= 0 && out_fd >= 0);
    hx_config cfg;
    int rc = hx_model_config(m, &cfg); if (rc) return rc;
    Emitter em{out_fd};
    int smax = ((max_ctx + 63) / 64) * 64; if (smax < 64) smax = 64;
    hx_sampler* smp = nullptr;
    if ((rc = hx_sampler_create(&smp, cfg.vocab))) return rc;
    std::vector<float> logits((size_t)cfg.vocab);
    hx_sample_config prev = {0.0, 1.0, 0.0, 1.0, 0.0, 0.0, 0, 0};        // sampling configuration left by the previous frame
    char dev_name[256] = "";
    { int dev = 0; cudaDeviceProp pr; if (cudaGetDevice(&dev) == cudaSuccess && cudaGetDeviceProperties(&pr, dev) == cudaSuccess) snprintf(dev_name, sizeof dev_name, "%s", pr.name); }
    FILE* in = fdopen(dup(in_fd), "r");
    if (!in) { hx_sampler_free(smp); return hx_fail(HX_ERR_IO, "serve: cannot read the request stream"); }
    char* line = nullptr; size_t cap = 0;
    while (getline(&line, &cap, in) > 0) {
        const char* p;
        if ((p = find_key(line, "cmd")) && *p == '"' && strncmp(p + 1, "quit", 4) == 0) break;
        int n_gen = 20;
        if ((p = find_key(line, "n_gen"))) n_gen = atoi(p);
        const bool has_prompt = (p = find_key(line, "prompt")) && *p == '"';
        std::vector<int32_t> ids;
        if (!has_prompt && (p = find_key(line, "ids")) && *p == '[') {
            p++;
            while (*p && *p != ']' && ids.size() < 1024) {
                while (*p == ' ' || *p == ',') p++;
                if (*p == ']' || !*p) break;
                ids.push_back(atoi(p));
                while (*p && *p != ',' && *p != ']') p++;
            }
        }
        if (!has_prompt && ids.empty()) { em.error("load", "bad request json", false); continue; }
        if (has_prompt && !tok) { em.error("tokenize", "no in-process tokenizer and no pre-tokenized ids", false); continue; }
        if (has_prompt) {
            const std::string text = json_unescape(find_key(line, "prompt") + 1);
            ids.resize(text.size() + 8);
            int nid = 0;
            if (hx_tokenizer_encode(tok, text.data(), text.size(), with_specials, ids.data(), (int)ids.size(), &nid) != HX_OK || nid <= 0) {
                em.error("tokenize", "empty/failed tokenization", false); continue;
            }
            ids.resize((size_t)nid);
        }
        bool bad_id = false;
        for (int32_t t : ids) if (t < 0 || t >= cfg.vocab) bad_id = true;
        if (bad_id) { em.error("tokenize", "token id outside the vocabulary", false); continue; }
        const int T0 = (int)ids.size();
        int Ngen = n_gen < 1 ? 1 : (n_gen > 256 ? 256 : n_gen);
        if (((T0 + Ngen + 63) / 64) * 64 > smax) { em.error("forward", "context exceeds --max-ctx; raise --max-ctx", false); continue; }

        char b[1400];
        snprintf(b, sizeof b,
                 "{\"_ev\":\"hello\",\"seq\":%ld,\"schema_version\":1,\"model\":\"hxgw-v3\",\"n_layer\":%d,\"n_head\":%d,\"d_model\":%d,\"d_ff\":%d,"
                 "\"n_vocab\":%d,\"device\":\"%s\",\"sm\":\"sm_100a\",\"precision\":\"nvfp4 weights, fp32 activations\",\"build\":\"forward-only\","
                 "\"mode\":\"serve\",\"engine\":\"%s\"}\n",
                 em.seq++, cfg.n_layers, cfg.n_heads, cfg.d_model, cfg.d_ff, cfg.vocab, dev_name, hx_model_engine(m));
        em.raw(b);
        {
            std::string s = "{\"_ev\":\"tokenize\",\"seq\":" + std::to_string(em.seq++) + ",\"ids\":[";
            for (int i = 0; i < T0; i++) { if (i) s += ","; s += std::to_string(ids[i]); }
            s += "],\"strings\":[";
            if (tok) for (int i = 0; i < T0; i++) { if (i) s += ","; s += "\"" + jesc(decode_ids(tok, &ids[i], 1)) + "\""; }
            s += "],\"n_prompt\":" + std::to_string(T0) + ",\"s_pad\":" + std::to_string(((T0 + 63) / 64) * 64) + "}\n";
            em.raw(s);
        }
        hx_sample_config sc = {0.0, 1.0, 0.0, 1.0, 0.0, 0.0, 0, 0};
        if ((p = find_key(line, "temperature"))) sc.temperature = atof(p);
        if ((p = find_key(line, "top_p"))) sc.top_p = atof(p);
        if ((p = find_key(line, "top_k"))) sc.top_k = atoi(p);
        if ((p = find_key(line, "min_p"))) sc.min_p = atof(p);
        if ((p = find_key(line, "rep_penalty"))) sc.rep_penalty = atof(p);
        if ((p = find_key(line, "freq_penalty"))) sc.freq_penalty = atof(p);
        if ((p = find_key(line, "pres_penalty"))) sc.pres_penalty = atof(p);
        if ((p = find_key(line, "seed"))) sc.seed = (uint64_t)strtoull(p, nullptr, 10);
        // The reference resets its sampler state (counts of the prompt, generator seed) BEFORE it reads the frame's own
        // sampling fields (:3338 against :3349): the reset happens only if the configuration left by the previous frame
        // samples, and with that frame's seed.  A first sampling request after a greedy one therefore draws from an
        // unseeded generator (every draw 0: the most probable candidate) with no counts.  Reproduced as is, so that the
        // stream equals the reference's frame for frame.
        if (prev.temperature > 0.0) hx_sampler_reset(smp, &prev, ids.data(), T0);
        hx_sampler_configure(smp, &sc);
        prev = sc;
        if (prev.temperature < 0.0) prev.temperature = 0.0;

        // stop sequences: up to four of up to 31 bytes, matched against the tail of the decoded text (stops_parse /
        // stops_hit, :1043-1094); they need the tokenizer's pieces
        std::vector<std::string> stops;
        if (tok && (p = find_key(line, "stop")) && *p == '[') {
            p++;
            while (stops.size() < 4) {
                while (*p == ' ' || *p == ',') p++;
                if (*p != '"') break;
                p++;
                std::string st;
                while (*p && *p != '"' && st.size() < 31) {
                    if (*p == '\\' && p[1]) { p++; st.push_back(*p == 'n' ? '\n' : (*p == 't' ? '\t' : *p)); p++; }
                    else st.push_back(*p++);
                }
                while (*p && *p != '"') p++;
                if (*p == '"') p++;
                if (!st.empty()) stops.push_back(st);
                while (*p == ' ') p++;
                if (*p != ',') break;
            }
        }
        std::string tail;
        hx_model_reset(m);                                           // KV is per request: a fresh prefill fills it
        std::vector<int32_t> gen;
        int nonfinite = 0, T = T0;
        bool failed = false;
        const double t0 = now_s();
        for (int step = 0; step < Ngen; step++) {
            snprintf(b, sizeof b, "{\"_ev\":\"forward_begin\",\"seq\":%ld,\"step\":%d,\"context_len\":%d,\"s_pad\":%d,\"n_layers\":%d}\n",
                     em.seq++, step, T, ((T + 63) / 64) * 64, cfg.n_layers);
            em.raw(b);
            int32_t dummy = 0;
            if (step == 0) rc = hx_prefill(m, ids.data(), T0, &dummy, logits.data());
            else { const int32_t tok = ids[T - 1]; rc = hx_decode_step(m, &tok, T - 1, &dummy, logits.data()); }
            if (rc) { em.error("forward", hx_last_error(), false); failed = true; break; }
            for (int i = 0; i < cfg.vocab; i++) if (!isfinite(logits[i])) { nonfinite = 1; break; }
            int32_t nxt = 0;
            hx_sampler_next(smp, logits.data(), &nxt);
            const std::string piece = decode_ids(tok, &nxt, 1);
            {
                std::string esc = jesc(piece);
                if (esc.size() > 255) esc.resize(255);               // the reference escapes a piece into 256 bytes
                std::string ev = "{\"_ev\":\"token\",\"seq\":" + std::to_string(em.seq++) + ",\"step\":" + std::to_string(step) + ",\"id\":" +
                                 std::to_string(nxt) + ",\"string\":\"" + esc + "\"";
                snprintf(b, sizeof b, ",\"logit\":%.5f,\"context_len\":%d}\n", (double)logits[nxt], T + 1);
                em.raw(ev + b);
            }
            gen.push_back(nxt); ids.push_back(nxt); T++;
            if (sc.temperature > 0.0) hx_sampler_count(smp, nxt);
            bool stop_now = false;
            if (!stops.empty()) {
                tail += piece;
                if (tail.size() > 255) tail.erase(0, tail.size() - 255);
                for (auto& st : stops) if (tail.size() >= st.size() && tail.compare(tail.size() - st.size(), st.size(), st) == 0) stop_now = true;
            }
            if (stop_now || (eos_id >= 0 && nxt == eos_id)) break;
        }
        if (failed) continue;
        const double secs = now_s() - t0;
        std::string s = "{\"_ev\":\"done\",\"seq\":" + std::to_string(em.seq++) + ",\"n_prompt\":" + std::to_string(T0) + ",\"n_gen\":" +
                        std::to_string((int)gen.size()) + ",\"n_total\":" + std::to_string(T);
        snprintf(b, sizeof b, ",\"seconds\":%.3f,\"tok_per_s\":%.3f,\"text\":\"", secs, secs > 0 ? (double)gen.size() / secs : 0.0);
        s += b;
        s += jesc(decode_ids(tok, gen.data(), (int)gen.size()));
        s += "\",\"gen_ids\":[";
        for (size_t i = 0; i < gen.size(); i++) { if (i) s += ","; s += std::to_string(gen[i]); }
        s += "],\"nonfinite\":" + std::to_string(nonfinite) + "}\n";
        em.raw(s);
    }
    free(line);
    fclose(in);
    hx_sampler_free(smp);
    return HX_OK;
}
