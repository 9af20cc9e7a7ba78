// hx_tokenizer.cu -- GPT-2 byte-level BPE: text <-> token ids from a vocab.json and a merges.txt.
//
// Replaces helixc/runtime/gpt2_tok.c (what the reference's serve mode links for "prompt" frames and for the
// strings of its events).  Host code only.  Like the reference it works in BYTE space: the byte <-> unicode map of
// GPT-2 is a bijection, so a vocabulary key is decoded to the byte string it stands for once at load time, a merge
// rule is a pair of byte strings, and decoding concatenates the byte strings of the ids (gpt2_tok.c:22-28).
//   * byte <-> unicode map: build_byte_unicode, :104-125;
//   * vocabulary keys and merge fields decoded through that map, a character outside it kept as its own UTF-8
//     bytes: parse_json_string_to_bytes :195-248, field_to_bytes :337-353; a leading '#' line of the merges is
//     skipped, a line without two fields does not consume a rank (:355-386);
//   * pre-tokenizer: the GPT-2 pattern 's|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+
//     written out as a scanner over code points (:532-640);
//   * BPE of a chunk: the adjacent pair of lowest rank is merged at all its non-overlapping occurrences, left to
//     right, until no pair has a rank (:389-447);
//   * control tokens (vocabulary entries of the form <...>): split off first, earliest then longest (:483-530).
// \p{L} and \p{N} come from the Unicode database of the Python that generated hx_unicode_ranges.inc; the
// reference's tables come from another Unicode version, so code points assigned in between may classify differently.
#include "hx_common.cuh"
#include <string>
#include <unordered_map>
#include <vector>
#include "hx_unicode_ranges.inc"

namespace {

// the White_Space property (what \s means in the pattern)
const unsigned int HX_UNI_S[][2] = {{0x9, 0xD}, {0x20, 0x20}, {0x85, 0x85}, {0xA0, 0xA0}, {0x1680, 0x1680}, {0x2000, 0x200A},
                                    {0x2028, 0x2029}, {0x202F, 0x202F}, {0x205F, 0x205F}, {0x3000, 0x3000}};
const int HX_UNI_S_N = 10;

bool in_ranges(unsigned int cp, const unsigned int (*tbl)[2], int n) {
    int lo = 0, hi = n - 1;
    while (lo <= hi) {
        const int mid = (lo + hi) >> 1;
        if (cp < tbl[mid][0]) hi = mid - 1; else if (cp > tbl[mid][1]) lo = mid + 1; else return true;
    }
    return false;
}
bool is_l(unsigned int cp) { return in_ranges(cp, HX_UNI_L, HX_UNI_L_N); }
bool is_n(unsigned int cp) { return in_ranges(cp, HX_UNI_N, HX_UNI_N_N); }
bool is_s(unsigned int cp) { return in_ranges(cp, HX_UNI_S, HX_UNI_S_N); }

// one code point at s[i..); a malformed lead byte is taken as itself (utf8_next, :127-146)
unsigned int utf8_next(const unsigned char* s, size_t n, size_t* i) {
    const unsigned int b0 = s[*i];
    auto at = [&](size_t k) -> unsigned int { return *i + k < n ? s[*i + k] : 0u; };
    if (b0 < 0x80) { (*i)++; return b0; }
    if ((b0 & 0xE0) == 0xC0 && *i + 1 < n) { const unsigned int cp = ((b0 & 0x1F) << 6) | (at(1) & 0x3F); *i += 2; return cp; }
    if ((b0 & 0xF0) == 0xE0) { const unsigned int cp = ((b0 & 0x0F) << 12) | ((at(1) & 0x3F) << 6) | (at(2) & 0x3F); *i += 3; if (*i > n) *i = n; return cp; }
    if ((b0 & 0xF8) == 0xF0) { const unsigned int cp = ((b0 & 0x07) << 18) | ((at(1) & 0x3F) << 12) | ((at(2) & 0x3F) << 6) | (at(3) & 0x3F); *i += 4; if (*i > n) *i = n; return cp; }
    (*i)++; return b0;
}

}  // namespace

struct hx_tokenizer {
    int u2b[512];
    std::unordered_map<std::string, int> vocab;            // byte string -> id
    std::vector<std::string> id2bytes;                      // id -> byte string ("" = unused id)
    std::vector<char> id_used;
    std::unordered_map<std::string, int> rank;              // (2-byte length of left) + left + right -> rank
    struct Special { std::string bytes; int id; };
    std::vector<Special> specials;                          // longest first

    void append_mapped(unsigned int cp, std::string& out) const {
        const int b = cp < 512 ? u2b[cp] : -1;
        if (b >= 0) { out.push_back((char)b); return; }
        if (cp < 0x80) out.push_back((char)cp);
        else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
        else { out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
    }
    static std::string pair_key(const char* l, int ll, const char* r, int rl) {
        std::string k; k.reserve((size_t)ll + rl + 2);
        k.push_back((char)(ll & 0xFF)); k.push_back((char)((ll >> 8) & 0xFF));
        k.append(l, (size_t)ll); k.append(r, (size_t)rl);
        return k;
    }
    int merge_rank(const char* l, int ll, const char* r, int rl) const {
        auto it = rank.find(pair_key(l, ll, r, rl));
        return it == rank.end() ? -1 : it->second;
    }

    // BPE of one chunk; false if a final symbol is not in the vocabulary
    bool bpe(const unsigned char* w, int wlen, std::vector<int32_t>& out) const {
        if (wlen == 0) return true;
        std::vector<std::pair<int, int>> syms((size_t)wlen);         // (offset, length)
        for (int i = 0; i < wlen; i++) syms[i] = std::make_pair(i, 1);
        const char* wc = reinterpret_cast<const char*>(w);
        for (;;) {
            const int ns = (int)syms.size();
            if (ns < 2) break;
            int best = -1, best_i = -1;
            for (int i = 0; i + 1 < ns; i++) {
                const int r = merge_rank(wc + syms[i].first, syms[i].second, wc + syms[i + 1].first, syms[i + 1].second);
                if (r >= 0 && (best < 0 || r < best)) { best = r; best_i = i; }
            }
            if (best_i < 0) break;
            const int ll = syms[best_i].second, rl = syms[best_i + 1].second;
            const std::string L(wc + syms[best_i].first, (size_t)ll), R(wc + syms[best_i + 1].first, (size_t)rl);
            std::vector<std::pair<int, int>> next; next.reserve(syms.size());
            for (int i = 0; i < ns;) {
                if (i + 1 < ns && syms[i].second == ll && memcmp(wc + syms[i].first, L.data(), (size_t)ll) == 0 &&
                    syms[i + 1].second == rl && memcmp(wc + syms[i + 1].first, R.data(), (size_t)rl) == 0) {
                    next.push_back(std::make_pair(syms[i].first, ll + rl)); i += 2;
                } else next.push_back(syms[i++]);
            }
            syms.swap(next);
        }
        for (auto& sy : syms) {
            auto it = vocab.find(std::string(wc + sy.first, (size_t)sy.second));
            if (it == vocab.end()) return false;
            out.push_back(it->second);
        }
        return true;
    }

    bool encode_plain(const unsigned char* text, size_t n, std::vector<int32_t>& ids) const {
        std::vector<unsigned int> cp; std::vector<size_t> bs;
        for (size_t i = 0; i < n;) { bs.push_back(i); cp.push_back(utf8_next(text, n, &i)); }
        bs.push_back(n);
        const int ncp = (int)cp.size();
        auto other = [&](unsigned int c) { return !is_s(c) && !is_l(c) && !is_n(c); };
        int p = 0;
        while (p < ncp) {
            int end = -1;
            const unsigned int c = cp[p];
            if (c == '\'') {                                            // contractions
                const unsigned int c1 = p + 1 < ncp ? cp[p + 1] : 0, c2 = p + 2 < ncp ? cp[p + 2] : 0;
                if (c1 == 's' || c1 == 't' || c1 == 'm' || c1 == 'd') end = p + 2;
                else if ((c1 == 'r' && c2 == 'e') || (c1 == 'v' && c2 == 'e') || (c1 == 'l' && c2 == 'l')) end = p + 3;
            }
            if (end < 0) {                                              // one optional space, then letters / digits / the rest
                const int q = c == ' ' ? p + 1 : p;
                if (q < ncp) {
                    const unsigned int d = cp[q];
                    int r = q;
                    if (is_l(d)) { while (r < ncp && is_l(cp[r])) r++; end = r; }
                    else if (is_n(d)) { while (r < ncp && is_n(cp[r])) r++; end = r; }
                    else if (other(d)) { while (r < ncp && other(cp[r])) r++; end = r; }
                }
            }
            if (end < 0 && is_s(c)) {                                   // white space: all but the last before a word, else all
                int r = p;
                while (r < ncp && is_s(cp[r])) r++;
                const int end5 = r >= ncp ? r : r - 1;
                end = end5 > p ? end5 : r;
            }
            if (end < 0) end = p + 1;
            if (!bpe(text + bs[p], (int)(bs[end] - bs[p]), ids)) return false;
            p = end;
        }
        return true;
    }
};

namespace {

bool slurp(const char* path, std::string& out) {
    FILE* f = fopen(path, "rb");
    if (!f) return false;
    char buf[65536]; size_t n;
    out.clear();
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) out.append(buf, n);
    fclose(f);
    return true;
}

}  // namespace

HX_API int hx_tokenizer_load(hx_tokenizer** out, const char* vocab_json, const char* merges_txt) {
    HX_CHECK_ARG(out && vocab_json && merges_txt);
    std::string vs, ms;
    if (!slurp(vocab_json, vs)) return hx_fail(HX_ERR_IO, "cannot read %s", vocab_json);
    if (!slurp(merges_txt, ms)) return hx_fail(HX_ERR_IO, "cannot read %s", merges_txt);
    hx_tokenizer* t = new hx_tokenizer();
    {   // byte <-> unicode: printable bytes stand for themselves, the others for 256, 257, ... in byte order
        bool direct[256] = {false};
        for (int c = '!'; c <= '~'; c++) direct[c] = true;
        for (int c = 0xA1; c <= 0xAC; c++) direct[c] = true;
        for (int c = 0xAE; c <= 0xFF; c++) direct[c] = true;
        for (int i = 0; i < 512; i++) t->u2b[i] = -1;
        int k = 0;
        for (int b = 0; b < 256; b++) { if (direct[b]) t->u2b[b] = b; else t->u2b[256 + k++] = b; }
    }
    const unsigned char* s = reinterpret_cast<const unsigned char*>(vs.data());
    const size_t n = vs.size();
    size_t i = 0;
    while (i < n && s[i] != '{') i++;
    if (i < n) i++;
    for (;;) {
        while (i < n && (s[i] == ' ' || s[i] == '\n' || s[i] == '\r' || s[i] == '\t' || s[i] == ',')) i++;
        if (i >= n || s[i] == '}') break;
        if (s[i] != '"') { i++; continue; }
        std::string key;
        i++;
        while (i < n && s[i] != '"') {
            unsigned int cp;
            if (s[i] == '\\' && i + 1 < n) {
                const char e = (char)s[i + 1];
                i += 2;
                switch (e) {
                    case 'n': cp = '\n'; break; case 't': cp = '\t'; break; case 'r': cp = '\r'; break; case 'b': cp = '\b'; break;
                    case 'f': cp = '\f'; break; case '/': cp = '/'; break; case '\\': cp = '\\'; break; case '"': cp = '"'; break;
                    case 'u': {
                        unsigned int v = 0;
                        for (int k = 0; k < 4 && i < n; k++, i++) {
                            const char h = (char)s[i]; v <<= 4;
                            if (h >= '0' && h <= '9') v |= (unsigned)(h - '0'); else if (h >= 'a' && h <= 'f') v |= (unsigned)(h - 'a' + 10);
                            else if (h >= 'A' && h <= 'F') v |= (unsigned)(h - 'A' + 10);
                        }
                        cp = v; break;
                    }
                    default: cp = (unsigned char)e; break;
                }
            } else if (s[i] < 0x80) cp = s[i++];
            else cp = utf8_next(s, n, &i);
            t->append_mapped(cp, key);
        }
        if (i < n) i++;
        while (i < n && (s[i] == ' ' || s[i] == '\n' || s[i] == '\r' || s[i] == '\t' || s[i] == ':')) i++;
        bool neg = false, any = false; long id = 0;
        if (i < n && s[i] == '-') { neg = true; i++; }
        while (i < n && s[i] >= '0' && s[i] <= '9') { id = id * 10 + (s[i] - '0'); i++; any = true; }
        if (!any) continue;
        if (neg || id > 16 * 1024 * 1024) { delete t; return hx_fail(HX_ERR_FORMAT, "%s: token id %ld out of range", vocab_json, neg ? -id : id); }
        t->vocab[key] = (int)id;
        if ((size_t)id >= t->id2bytes.size()) { t->id2bytes.resize((size_t)id + 1); t->id_used.resize((size_t)id + 1, 0); }
        t->id2bytes[(size_t)id] = key; t->id_used[(size_t)id] = 1;
    }
    if (t->vocab.empty()) { delete t; return hx_fail(HX_ERR_FORMAT, "%s holds no vocabulary entries", vocab_json); }
    const unsigned char* m = reinterpret_cast<const unsigned char*>(ms.data());
    const size_t mn = ms.size();
    i = 0;
    if (i < mn && m[i] == '#') { while (i < mn && m[i] != '\n') i++; if (i < mn) i++; }
    int rk = 0;
    auto field = [&](std::string& f) {
        f.clear();
        while (i < mn) {
            const unsigned char c = m[i];
            if (c == ' ' || c == '\n' || c == '\r' || c == '\t') break;
            unsigned int cp;
            if (c < 0x80) { cp = c; i++; } else cp = utf8_next(m, mn, &i);
            t->append_mapped(cp, f);
        }
    };
    std::string l, r;
    while (i < mn) {
        while (i < mn && (m[i] == '\n' || m[i] == '\r')) i++;
        if (i >= mn) break;
        field(l);
        while (i < mn && (m[i] == ' ' || m[i] == '\t')) i++;
        field(r);
        while (i < mn && m[i] != '\n') i++;
        if (i < mn) i++;
        if (l.empty() || r.empty()) continue;
        const std::string k = hx_tokenizer::pair_key(l.data(), (int)l.size(), r.data(), (int)r.size());
        if (t->rank.find(k) == t->rank.end()) t->rank[k] = rk;         // a repeated rule keeps its first rank
        rk++;
    }
    // control tokens: vocabulary entries of the form <...>, at most 64, in id order, then longest first (stable)
    for (size_t id = 0; id < t->id2bytes.size() && t->specials.size() < 64; id++) {
        const std::string& b = t->id2bytes[id];
        if (t->id_used[id] && b.size() >= 3 && b.front() == '<' && b.back() == '>') t->specials.push_back({b, (int)id});
    }
    for (size_t a = 0; a < t->specials.size(); a++)
        for (size_t b = a + 1; b < t->specials.size(); b++)
            if (t->specials[b].bytes.size() > t->specials[a].bytes.size()) std::swap(t->specials[a], t->specials[b]);
    *out = t;
    return HX_OK;
}

HX_API int hx_tokenizer_free(hx_tokenizer* t) { delete t; return HX_OK; }
HX_API int hx_tokenizer_vocab_size(const hx_tokenizer* t) { return t ? (int)t->id2bytes.size() : 0; }

// text -> ids.  with_specials != 0: control tokens are split off first (encode_bytes_special).  *n_ids is the number
// of ids the text has; HX_ERR_ARG if it exceeds max_ids (ids then holds the first max_ids).
HX_API int hx_tokenizer_encode(const hx_tokenizer* t, const char* text, size_t n, int with_specials, int32_t* ids, int max_ids, int* n_ids) {
    HX_CHECK_ARG(t && (text || n == 0) && n_ids && (ids || max_ids == 0));
    const unsigned char* s = reinterpret_cast<const unsigned char*>(text);
    std::vector<int32_t> out;
    bool ok = true;
    if (!with_specials || t->specials.empty()) ok = t->encode_plain(s, n, out);
    else {
        size_t i = 0;
        while (i < n && ok) {
            size_t best_pos = n; int best = -1;
            for (size_t k = 0; k < t->specials.size(); k++) {
                const std::string& sp = t->specials[k].bytes;
                for (size_t j = i; j + sp.size() <= n && j <= best_pos; j++)
                    if (s[j] == (unsigned char)sp[0] && memcmp(s + j, sp.data(), sp.size()) == 0) { if (j < best_pos) { best_pos = j; best = (int)k; } break; }
            }
            const size_t seg_end = best >= 0 ? best_pos : n;
            if (seg_end > i) ok = t->encode_plain(s + i, seg_end - i, out);
            if (best < 0) break;
            out.push_back(t->specials[(size_t)best].id);
            i = best_pos + t->specials[(size_t)best].bytes.size();
        }
    }
    if (!ok) return hx_fail(HX_ERR_FORMAT, "a byte sequence of the text has no vocabulary entry (vocabulary and merges do not belong together)");
    *n_ids = (int)out.size();
    const int ncopy = (int)out.size() < max_ids ? (int)out.size() : max_ids;
    if (ncopy > 0) memcpy(ids, out.data(), (size_t)ncopy * sizeof(int32_t));
    if ((int)out.size() > max_ids) return hx_fail(HX_ERR_ARG, "the text has %d tokens, the buffer holds %d", (int)out.size(), max_ids);
    return HX_OK;
}

// ids -> the bytes they stand for (decode_range, :660-671); unknown ids contribute nothing.  *len is the length the
// text has; HX_ERR_ARG if it exceeds cap (out then holds the first cap bytes).  No terminator is written.
HX_API int hx_tokenizer_decode(const hx_tokenizer* t, const int32_t* ids, int n, char* out, size_t cap, size_t* len) {
    HX_CHECK_ARG(t && (ids || n == 0) && len && (out || cap == 0));
    size_t k = 0;
    for (int i = 0; i < n; i++) {
        if (ids[i] < 0 || (size_t)ids[i] >= t->id2bytes.size()) continue;
        const std::string& b = t->id2bytes[(size_t)ids[i]];
        for (size_t j = 0; j < b.size(); j++, k++) if (k < cap) out[k] = b[j];
    }
    *len = k;
    if (k > cap) return hx_fail(HX_ERR_ARG, "the text has %zu bytes, the buffer holds %zu", k, cap);
    return HX_OK;
}
