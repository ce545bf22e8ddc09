// Reading side of the path's files.
//
//  * Frozen base from a Hugging Face model directory: config.json + safetensors shards, the roles of
//    parser::ModelConfig (src/parser/config.cpp:43-110), parser::WeightMap::open
//    (src/parser/weight_map.cpp:26-68), parser::SafeTensors (src/parser/safetensors.cpp:60-250) and
//    base::BaseLoader::load (src/base/base_loader.cpp:80-170).  Shards are mmap'ed and copied straight
//    into the weight arena (BF16 as is; F32 staged on the device and rounded there, RNE like the
//    reference's host loop); nothing is staged per tensor on the heap.
//  * Resume: optimizer.safetensors (FP32 masters, AdamW m / v, step, centroid sums) written next to
//    the reference-format checkpoint files and read back into the flat LoRA arrays.  The reference
//    only documents this file (README "Mid-run checkpoint layout"); its code never writes or reads it.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "trainer.h"

namespace fs = std::filesystem;

namespace ta {
namespace {

// ── minimal JSON reader (objects, arrays, strings, numbers, true/false/null) ──────────────────────
struct Json {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0;
    bool is_int = false;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;   // document order

    const Json* get(const std::string& k) const {
        if (kind != Obj) return nullptr;
        for (auto& kv : obj) if (kv.first == k) return &kv.second;
        return nullptr;
    }
};

struct JsonParser {
    const char* p;
    const char* end;
    std::string err;

    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
    bool fail_(const std::string& m) { if (err.empty()) err = m; return false; }

    static void utf8(std::string& o, unsigned cp) {
        if (cp < 0x80) o += char(cp);
        else if (cp < 0x800) { o += char(0xC0 | (cp >> 6)); o += char(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { o += char(0xE0 | (cp >> 12)); o += char(0x80 | ((cp >> 6) & 0x3F)); o += char(0x80 | (cp & 0x3F)); }
        else { o += char(0xF0 | (cp >> 18)); o += char(0x80 | ((cp >> 12) & 0x3F)); o += char(0x80 | ((cp >> 6) & 0x3F)); o += char(0x80 | (cp & 0x3F)); }
    }
    bool hex4(unsigned* v) {
        if (end - p < 4) return fail_("short \\u escape");
        unsigned x = 0;
        for (int i = 0; i < 4; i++) {
            const char c = *p++;
            x <<= 4;
            if (c >= '0' && c <= '9') x |= unsigned(c - '0');
            else if (c >= 'a' && c <= 'f') x |= unsigned(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') x |= unsigned(c - 'A' + 10);
            else return fail_("bad \\u escape");
        }
        *v = x;
        return true;
    }
    bool string(std::string& o) {
        if (p >= end || *p != '"') return fail_("expected string");
        p++;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return fail_("dangling escape");
                const char c = *p++;
                switch (c) {
                    case '"': o += '"'; break;   case '\\': o += '\\'; break; case '/': o += '/'; break;
                    case 'b': o += '\b'; break;  case 'f': o += '\f'; break;  case 'n': o += '\n'; break;
                    case 'r': o += '\r'; break;  case 't': o += '\t'; break;
                    case 'u': {
                        unsigned cp;
                        if (!hex4(&cp)) return false;
                        if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
                            p += 2;
                            unsigned lo;
                            if (!hex4(&lo)) return false;
                            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                        }
                        utf8(o, cp);
                        break;
                    }
                    default: return fail_("bad escape");
                }
            } else {
                o += *p++;
            }
        }
        if (p >= end) return fail_("unterminated string");
        p++;
        return true;
    }
    bool value(Json& v, int depth = 0) {
        if (depth > 64) return fail_("nesting too deep");
        ws();
        if (p >= end) return fail_("unexpected end");
        if (*p == '{') {
            v.kind = Json::Obj; p++; ws();
            if (p < end && *p == '}') { p++; return true; }
            for (;;) {
                ws();
                std::string k;
                if (!string(k)) return false;
                ws();
                if (p >= end || *p != ':') return fail_("expected ':'");
                p++;
                Json c;
                if (!value(c, depth + 1)) return false;
                v.obj.emplace_back(std::move(k), std::move(c));
                ws();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == '}') { p++; return true; }
                return fail_("expected ',' or '}'");
            }
        }
        if (*p == '[') {
            v.kind = Json::Arr; p++; ws();
            if (p < end && *p == ']') { p++; return true; }
            for (;;) {
                Json c;
                if (!value(c, depth + 1)) return false;
                v.arr.push_back(std::move(c));
                ws();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == ']') { p++; return true; }
                return fail_("expected ',' or ']'");
            }
        }
        if (*p == '"') { v.kind = Json::Str; return string(v.str); }
        if (end - p >= 4 && !std::strncmp(p, "true", 4)) { v.kind = Json::Bool; v.b = true; p += 4; return true; }
        if (end - p >= 5 && !std::strncmp(p, "false", 5)) { v.kind = Json::Bool; v.b = false; p += 5; return true; }
        if (end - p >= 4 && !std::strncmp(p, "null", 4)) { v.kind = Json::Null; p += 4; return true; }
        const char* s = p;
        if (p < end && *p == '-') p++;
        bool integral = true;
        while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '+' || *p == '-')) {
            if (*p == '.' || *p == 'e' || *p == 'E') integral = false;
            p++;
        }
        if (p == s) return fail_("unexpected character");
        v.kind = Json::Num;
        v.is_int = integral;
        v.num = std::strtod(std::string(s, p).c_str(), nullptr);
        return true;
    }
};

bool parse_json(const char* text, size_t n, Json* out, std::string* err) {
    JsonParser jp{text, text + n, {}};
    if (!jp.value(*out)) { *err = jp.err; return false; }
    jp.ws();
    if (jp.p != jp.end) { *err = "trailing characters"; return false; }
    return true;
}

// ── SHA-256 (FIPS 180-4), for BaseConfig::base_sha (src/base/base_loader.cpp:30-52) ───────────────
struct Sha256 {
    uint32_t h[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au, 0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
    static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
    struct RoundConstants {
        uint32_t k[64];
        RoundConstants() {   // fractional parts of the cube roots of the first 64 primes
            int n = 0;
            for (int c = 2; n < 64; c++) {
                bool prime = true;
                for (int d = 2; d * d <= c; d++) if (c % d == 0) { prime = false; break; }
                if (!prime) continue;
                const long double r = cbrtl((long double)c);
                k[n++] = uint32_t((r - floorl(r)) * 4294967296.0L);
            }
        }
    };
    static const uint32_t* K() {
        static const RoundConstants rc;   // initialised once, thread-safe
        return rc.k;
    }
    void block(const unsigned char* b) {
        const uint32_t* k = K();
        uint32_t w[64];
        for (int i = 0; i < 16; i++) w[i] = uint32_t(b[4 * i]) << 24 | uint32_t(b[4 * i + 1]) << 16 | uint32_t(b[4 * i + 2]) << 8 | b[4 * i + 3];
        for (int i = 16; i < 64; i++) {
            const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
            const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
            w[i] = w[i - 16] + s0 + w[i - 7] + s1;
        }
        uint32_t a = h[0], bb = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
        for (int i = 0; i < 64; i++) {
            const uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25), ch = (e & f) ^ (~e & g);
            const uint32_t t1 = hh + S1 + ch + k[i] + w[i];
            const uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22), mj = (a & bb) ^ (a & c) ^ (bb & c);
            const uint32_t t2 = S0 + mj;
            hh = g; g = f; f = e; e = d + t1; d = c; c = bb; bb = a; a = t1 + t2;
        }
        h[0] += a; h[1] += bb; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
    }
    static std::string hex(const std::string& msg) {
        Sha256 s;
        std::string m = msg;
        const uint64_t bits = uint64_t(msg.size()) * 8;
        m += char(0x80);
        while (m.size() % 64 != 56) m += char(0);
        for (int i = 7; i >= 0; i--) m += char((bits >> (8 * i)) & 0xFF);
        for (size_t o = 0; o < m.size(); o += 64) s.block(reinterpret_cast<const unsigned char*>(m.data()) + o);
        char buf[65];
        for (int i = 0; i < 8; i++) std::snprintf(buf + 8 * i, 9, "%08x", s.h[i]);
        return std::string(buf, 64);
    }
};

// ── safetensors shards ───────────────────────────────────────────────────────────────────────────
struct StEntry {
    int dtype = -1;   // 0 F32, 1 BF16, 2 F16, 3 other
    std::vector<long> shape;
    const unsigned char* data = nullptr;
    size_t bytes = 0;
    long numel() const { long n = 1; for (long d : shape) n *= d; return n; }
};

struct Shard {
    void* map = nullptr;
    size_t size = 0;
    ~Shard() { if (map) munmap(map, size); }
};

struct WeightFiles {
    std::vector<std::unique_ptr<Shard>> shards;
    std::map<std::string, StEntry> entries;
};

int dtype_code(const std::string& s) {
    if (s == "F32") return 0;
    if (s == "BF16") return 1;
    if (s == "F16") return 2;
    return 3;
}
size_t dtype_size(int code, const std::string& s) {
    if (code == 0) return 4;
    if (code == 1 || code == 2) return 2;
    if (s == "F64" || s == "I64" || s == "U64") return 8;
    if (s == "I32" || s == "U32") return 4;
    if (s == "I16" || s == "U16") return 2;
    return 1;
}

// One shard: 8-byte little-endian header length, JSON header, data section; every descriptor is
// validated like src/parser/safetensors.cpp:150-226 (object with string dtype, unsigned shape,
// two data_offsets with end >= begin inside the file, no duplicate names across shards).
bool add_shard(const std::string& path, WeightFiles* wf, std::string* err) {
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) { *err = "cannot open " + path; return false; }
    struct stat st{};
    if (fstat(fd, &st) != 0 || st.st_size < 8) { ::close(fd); *err = "file too small to be safetensors: " + path; return false; }
    auto sh = std::make_unique<Shard>();
    sh->size = size_t(st.st_size);
    sh->map = mmap(nullptr, sh->size, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (sh->map == MAP_FAILED) { sh->map = nullptr; *err = "mmap failed: " + path; return false; }
    const unsigned char* base = static_cast<const unsigned char*>(sh->map);
    uint64_t hlen = 0;
    std::memcpy(&hlen, base, 8);
    if (hlen == 0) { *err = "safetensors header length is zero: " + path; return false; }
    if (hlen > sh->size - 8) { *err = "safetensors header length exceeds file size: " + path; return false; }
    const size_t data_start = 8 + size_t(hlen);
    Json root;
    std::string jerr;
    if (!parse_json(reinterpret_cast<const char*>(base + 8), size_t(hlen), &root, &jerr)) {
        *err = "JSON parse error in safetensors header: " + jerr + " in: " + path;
        return false;
    }
    if (root.kind != Json::Obj) { *err = "safetensors header is not a JSON object: " + path; return false; }
    for (auto& kv : root.obj) {
        const std::string& name = kv.first;
        const Json& d = kv.second;
        if (name == "__metadata__") {
            if (d.kind != Json::Obj) { *err = "__metadata__ is not a JSON object in: " + path; return false; }
            continue;
        }
        if (d.kind != Json::Obj) { *err = "tensor descriptor for \"" + name + "\" is not a JSON object in: " + path; return false; }
        const Json *dt = d.get("dtype"), *shp = d.get("shape"), *off = d.get("data_offsets");
        if (!dt || dt->kind != Json::Str) { *err = "missing or non-string dtype for tensor \"" + name + "\" in: " + path; return false; }
        if (!shp || shp->kind != Json::Arr) { *err = "missing or non-array shape for tensor \"" + name + "\" in: " + path; return false; }
        StEntry e;
        e.dtype = dtype_code(dt->str);
        for (auto& dim : shp->arr) {
            if (dim.kind != Json::Num || !dim.is_int || dim.num < 0) { *err = "non-integer shape dimension for tensor \"" + name + "\" in: " + path; return false; }
            e.shape.push_back(long(dim.num));
        }
        if (!off || off->kind != Json::Arr || off->arr.size() != 2 || off->arr[0].kind != Json::Num || off->arr[1].kind != Json::Num) {
            *err = "missing or invalid data_offsets for tensor \"" + name + "\" in: " + path;
            return false;
        }
        const uint64_t b = uint64_t(off->arr[0].num), en = uint64_t(off->arr[1].num);
        if (en < b) { *err = "data_offsets end < begin for tensor \"" + name + "\" in: " + path; return false; }
        if (data_start + en > sh->size) { *err = "tensor \"" + name + "\" data range exceeds file size in: " + path; return false; }
        if (size_t(e.numel()) * dtype_size(e.dtype, dt->str) != en - b) {
            *err = "tensor \"" + name + "\": shape and data_offsets disagree in: " + path;
            return false;
        }
        if (wf->entries.count(name)) { *err = "duplicate tensor name \"" + name + "\" found in: " + path; return false; }
        e.data = base + data_start + b;
        e.bytes = size_t(en - b);
        wf->entries[name] = std::move(e);
    }
    wf->shards.push_back(std::move(sh));
    return true;
}

std::vector<fs::path> list_safetensors(const fs::path& d) {
    std::vector<fs::path> v;
    std::error_code ec;
    for (const auto& e : fs::directory_iterator(d, ec))
        if (e.is_regular_file() && e.path().extension() == ".safetensors") v.push_back(e.path());
    std::sort(v.begin(), v.end(), [](const fs::path& a, const fs::path& b) { return a.filename() < b.filename(); });
    return v;
}

// WeightMap::open: a .safetensors file, else <dir>/model.safetensors alone, else every shard by name.
bool open_weights(const std::string& dir, WeightFiles* wf, std::string* err) {
    fs::path d(dir);
    std::error_code ec;
    if (!fs::exists(d, ec)) { *err = "path does not exist: " + dir; return false; }
    if (fs::is_regular_file(d, ec) && d.extension() == ".safetensors") return add_shard(dir, wf, err);
    if (!fs::is_directory(d, ec)) { *err = "not a file or directory: " + dir; return false; }
    if (fs::exists(d / "model.safetensors", ec)) return add_shard((d / "model.safetensors").string(), wf, err);
    auto shards = list_safetensors(d);
    if (shards.empty()) { *err = "no .safetensors files found in: " + dir; return false; }
    for (auto& s : shards) if (!add_shard(s.string(), wf, err)) return false;
    return true;
}

bool read_text(const std::string& path, std::string* out) {
    std::ifstream f(path, std::ios::binary);
    if (!f) return false;
    out->assign(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>());
    return true;
}

struct BaseInfo {
    ta_model_config mc{};
    std::string arch_name, sha;
    bool known_arch = false;
};

// ModelConfig accessors with the reference's defaults (src/parser/config.cpp:100-110) and
// BaseLoader's derived fields (head_dim = hidden / heads; tie = no lm_head.weight in the shards).
bool read_base_info(const std::string& dir, const char* arch_hint, const WeightFiles* wf, BaseInfo* bi, std::string* err) {
    std::string txt;
    const std::string cpath = (fs::path(dir) / "config.json").string();
    if (!read_text(cpath, &txt)) { *err = "cannot open " + cpath; return false; }
    Json root;
    std::string jerr;
    if (!parse_json(txt.data(), txt.size(), &root, &jerr) || root.kind != Json::Obj) {
        *err = "JSON parse error in " + cpath + ": " + jerr;
        return false;
    }
    auto num = [&](const char* k, double def) { const Json* v = root.get(k); return v && v->kind == Json::Num ? v->num : def; };
    const Json* mt = root.get("model_type");
    bi->arch_name = mt && mt->kind == Json::Str ? mt->str : "";
    const std::string s = arch_hint && *arch_hint ? std::string(arch_hint) : bi->arch_name;
    bi->known_arch = s.find("qwen") != std::string::npos || s.find("llama") != std::string::npos;
    ta_model_config& m = bi->mc;
    m.vocab = int(num("vocab_size", 32000));
    m.hidden = int(num("hidden_size", 4096));
    m.layers = int(num("num_hidden_layers", 32));
    m.q_heads = int(num("num_attention_heads", 32));
    m.kv_heads = int(num("num_key_value_heads", double(m.q_heads)));
    m.head_dim = m.q_heads > 0 ? m.hidden / m.q_heads : 0;
    m.intermediate = int(num("intermediate_size", 11008));
    m.rms_eps = float(num("rms_norm_eps", 1e-5));
    m.rope_theta = float(num("rope_theta", 10000.0));
    m.tie_embeddings = wf ? (wf->entries.count("lm_head.weight") ? 0 : 1) : 0;
    std::string listing;
    for (auto& f : list_safetensors(fs::path(dir))) {
        std::error_code ec;
        listing += f.filename().string() + ":" + std::to_string(fs::file_size(f, ec)) + ";";
    }
    bi->sha = Sha256::hex(listing);
    return true;
}

__global__ void f32_to_bf16_rn_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long n) {
    for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < n; i += long(gridDim.x) * blockDim.x)
        out[i] = __float2bfloat16_rn(in[i]);
}

// Copy one tensor of the shards into its place in the weight arena.
int upload_weight(ta_trainer* t, const WeightFiles& wf, const std::string& name, __nv_bfloat16* dst, long numel,
                  float* stage, long stage_elems) {
    auto it = wf.entries.find(name);
    if (it == wf.entries.end()) return fail(t->ctx, TA_ERR_INVALID, "tensor not found: " + name);
    const StEntry& e = it->second;
    if (e.numel() != numel)
        return fail(t->ctx, TA_ERR_INVALID, "tensor " + name + " has " + std::to_string(e.numel()) + " elements, the model config needs " +
                                                std::to_string(numel));
    if (e.dtype == 1) {
        TA_CUDA(t->ctx, cudaMemcpyAsync(dst, e.data, size_t(numel) * 2, cudaMemcpyHostToDevice, t->stream));
        return TA_OK;
    }
    if (e.dtype == 0) {
        const float* src = reinterpret_cast<const float*>(e.data);
        for (long o = 0; o < numel; o += stage_elems) {
            const long n = std::min(stage_elems, numel - o);
            TA_CUDA(t->ctx, cudaMemcpyAsync(stage, src + o, size_t(n) * 4, cudaMemcpyHostToDevice, t->stream));
            f32_to_bf16_rn_kernel<<<unsigned(std::min<long>((n + 255) / 256, 4096)), 256, 0, t->stream>>>(stage, dst + o, n);
            TA_LAUNCH_CHECK(t->ctx, "f32_to_bf16_rn_kernel");
        }
        return TA_OK;
    }
    return fail(t->ctx, TA_ERR_UNSUPPORTED, "unsupported weight dtype for " + name);   // as BaseLoader: BF16 or F32 only
}

void copy_cstr(char* dst, int cap, const std::string& s) {
    if (!dst || cap <= 0) return;
    const size_t n = std::min(size_t(cap - 1), s.size());
    std::memcpy(dst, s.data(), n);
    dst[n] = 0;
}

std::string st_header(const std::vector<std::pair<std::string, std::pair<std::string, std::vector<long>>>>& tensors,
                      std::vector<size_t>* begins) {
    // key-sorted compact header, data in the order given; F32 / I64 entries
    std::map<std::string, std::string> m;
    size_t off = 0;
    for (auto& tn : tensors) {
        size_t numel = 1;
        std::string shp;
        for (size_t i = 0; i < tn.second.second.size(); i++) { numel *= size_t(tn.second.second[i]); shp += (i ? "," : "") + std::to_string(tn.second.second[i]); }
        const size_t bytes = numel * (tn.second.first == "I64" ? 8 : 4);
        begins->push_back(off);
        m[tn.first] = "{\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + bytes) + "],\"dtype\":\"" + tn.second.first +
                      "\",\"shape\":[" + shp + "]}";
        off += bytes;
    }
    std::string h = "{";
    bool first = true;
    for (auto& kv : m) { h += (first ? "\"" : ",\"") + kv.first + "\":" + kv.second; first = false; }
    h += "}";
    while (h.size() % 8) h += ' ';
    return h;
}

}  // namespace
}  // namespace ta

using namespace ta;

extern "C" {

int ta_base_probe(const char* dir, const char* arch_hint, ta_model_config* mc, char* arch_name, int arch_cap, char* sha_hex,
                  int sha_cap, char* err_text, int err_cap) {
    if (!dir || !mc) return TA_ERR_INVALID;
    WeightFiles wf;
    std::string err;
    BaseInfo bi;
    if (!open_weights(dir, &wf, &err) || !read_base_info(dir, arch_hint, &wf, &bi, &err)) {
        copy_cstr(err_text, err_cap, err);
        return TA_ERR_IO;
    }
    *mc = bi.mc;
    copy_cstr(arch_name, arch_cap, bi.arch_name);
    copy_cstr(sha_hex, sha_cap, bi.sha);
    if (!bi.known_arch) {
        copy_cstr(err_text, err_cap, "unknown architecture: " + bi.arch_name);
        return TA_ERR_UNSUPPORTED;
    }
    return TA_OK;
}

int ta_trainer_load_base(ta_trainer* t, const char* dir, const char* arch_hint) {
    if (!t || !dir) return TA_ERR_INVALID;
    WeightFiles wf;
    std::string err;
    BaseInfo bi;
    if (!open_weights(dir, &wf, &err) || !read_base_info(dir, arch_hint, &wf, &bi, &err)) return fail(t->ctx, TA_ERR_IO, err);
    if (!bi.known_arch) return fail(t->ctx, TA_ERR_UNSUPPORTED, "unknown architecture: " + bi.arch_name);
    const ta_model_config &a = bi.mc, &b = t->mc;
    if (a.vocab != b.vocab || a.hidden != b.hidden || a.layers != b.layers || a.q_heads != b.q_heads || a.kv_heads != b.kv_heads ||
        a.head_dim != b.head_dim || a.intermediate != b.intermediate || a.tie_embeddings != b.tie_embeddings)
        return fail(t->ctx, TA_ERR_INVALID, "config.json of " + std::string(dir) + " does not match the model config the trainer was created with");
    const long H = b.hidden, I = b.intermediate, V = b.vocab, qd = long(b.q_heads) * b.head_dim, kv = long(b.kv_heads) * b.head_dim;
    const long stage_elems = 8l << 20;   // 32 MB FP32 staging block, only touched for F32 checkpoints
    DeviceBuffer stage_buf;
    bool any_f32 = false;
    for (auto& kv2 : wf.entries) any_f32 |= kv2.second.dtype == 0;
    if (any_f32) TA_CUDA(t->ctx, stage_buf.alloc(size_t(stage_elems) * 4));
    float* stage = stage_buf.as<float>();
    int rc = upload_weight(t, wf, "model.embed_tokens.weight", t->embed, V * H, stage, stage_elems);
    for (int l = 0; l < b.layers && rc == TA_OK; l++) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        LayerW& w = t->L[size_t(l)];
        const struct { const char* name; __nv_bfloat16* dst; long n; } items[] = {
            {"input_layernorm.weight", w.input_norm, H},
            {"self_attn.q_proj.weight", w.q_w, qd * H}, {"self_attn.q_proj.bias", w.q_b, qd},
            {"self_attn.k_proj.weight", w.k_w, kv * H}, {"self_attn.k_proj.bias", w.k_b, kv},
            {"self_attn.v_proj.weight", w.v_w, kv * H}, {"self_attn.v_proj.bias", w.v_b, kv},
            {"self_attn.o_proj.weight", w.o_w, H * qd},
            {"post_attention_layernorm.weight", w.post_norm, H},
            {"mlp.gate_proj.weight", w.gate_w, I * H}, {"mlp.up_proj.weight", w.up_w, I * H}, {"mlp.down_proj.weight", w.down_w, H * I}};
        for (auto& it : items) {
            rc = upload_weight(t, wf, p + it.name, it.dst, it.n, stage, stage_elems);
            if (rc) break;
        }
    }
    if (rc == TA_OK) rc = upload_weight(t, wf, "model.norm.weight", t->final_norm, H, stage, stage_elems);
    if (rc == TA_OK && !b.tie_embeddings) rc = upload_weight(t, wf, "lm_head.weight", t->lm_head, V * H, stage, stage_elems);
    cudaStreamSynchronize(t->stream);   // the shards are unmapped on return
    if (rc) return rc;
    t->arch_name = bi.arch_name;
    t->base_sha = bi.sha;
    int st = 0;
    return ta_device_status(t->ctx, &st);
}

int ta_trainer_counters(ta_trainer* t, long* step, long* tokens_consumed) {
    if (!t) return TA_ERR_INVALID;
    if (step) *step = t->step_count;
    if (tokens_consumed) *tokens_consumed = t->tokens_seen;
    return TA_OK;
}

// optimizer.safetensors: "lora.master" / "lora.m" / "lora.v" (F32, the flat arrays with their padding),
// "centroid.acc" / "centroid.weight" (+ as-built pair), "step", "tokens_consumed" and "targets" (I64; the
// TA_TARGET_* mask the flat arrays were laid out for).
int ta_trainer_save_optimizer(ta_trainer* t, const char* dir) {
    if (!t || !dir) return TA_ERR_INVALID;
    TA_CUDA(t->ctx, cudaStreamSynchronize(t->stream));
    std::error_code ec;
    fs::create_directories(dir, ec);
    const long n = t->lora_n, D = t->mc.hidden;
    std::vector<std::pair<std::string, std::pair<std::string, std::vector<long>>>> tensors = {
        {"lora.master", {"F32", {n}}}, {"lora.m", {"F32", {n}}}, {"lora.v", {"F32", {n}}},
        {"centroid.acc", {"F32", {D}}}, {"centroid.weight", {"F32", {1}}},
        {"centroid_asbuilt.acc", {"F32", {D}}}, {"centroid_asbuilt.weight", {"F32", {1}}},
        {"step", {"I64", {1}}}, {"tokens_consumed", {"I64", {1}}}, {"targets", {"I64", {1}}}};
    std::vector<size_t> begins;
    const std::string hdr = st_header(tensors, &begins);
    const size_t total = begins.back() + 8;
    std::vector<char> data(total);
    const float* srcs[] = {t->master, t->m, t->v, t->cen_acc, t->cen_w, t->cen_acc_ab, t->cen_w_ab};
    const long lens[] = {n, n, n, D, 1, D, 1};
    for (int i = 0; i < 7; i++)
        TA_CUDA(t->ctx, cudaMemcpy(data.data() + begins[size_t(i)], srcs[i], size_t(lens[i]) * 4, cudaMemcpyDeviceToHost));
    const int64_t step = t->step_count, tok = t->tokens_seen, tgs = t->ac.targets;
    std::memcpy(data.data() + begins[7], &step, 8);
    std::memcpy(data.data() + begins[8], &tok, 8);
    std::memcpy(data.data() + begins[9], &tgs, 8);
    const std::string path = std::string(dir) + "/optimizer.safetensors";
    std::ofstream f(path, std::ios::binary);
    if (!f) return fail(t->ctx, TA_ERR_IO, "cannot write " + path);
    const uint64_t hlen = hdr.size();
    f.write(reinterpret_cast<const char*>(&hlen), 8);
    f.write(hdr.data(), std::streamsize(hlen));
    f.write(data.data(), std::streamsize(data.size()));
    return f ? TA_OK : fail(t->ctx, TA_ERR_IO, "short write to " + path);
}

// Resume from a checkpoint directory.  With optimizer.safetensors the FP32 state comes back exactly;
// without it (a reference-written checkpoint) the masters are the BF16 values of adapter.safetensors,
// moments start at zero and step / tokens come from train_state.json.  adapter.json is validated
// first: rank, alpha and base_sha must match this trainer.
int ta_trainer_resume(ta_trainer* t, const char* dir) {
    if (!t || !dir) return TA_ERR_INVALID;
    const fs::path d(dir);
    std::string txt, jerr;
    if (read_text((d / "adapter.json").string(), &txt)) {
        Json j;
        if (!parse_json(txt.data(), txt.size(), &j, &jerr) || j.kind != Json::Obj)
            return fail(t->ctx, TA_ERR_IO, "JSON parse error in adapter.json: " + jerr);
        const Json *rk = j.get("rank"), *al = j.get("alpha"), *sha = j.get("base_sha");
        if (rk && rk->kind == Json::Num && int(rk->num) != t->ac.rank)
            return fail(t->ctx, TA_ERR_INVALID, "checkpoint rank " + std::to_string(int(rk->num)) + " != adapter config rank " + std::to_string(t->ac.rank));
        if (al && al->kind == Json::Num && float(al->num) != t->ac.alpha)
            return fail(t->ctx, TA_ERR_INVALID, "checkpoint alpha does not match the adapter config");
        if (sha && sha->kind == Json::Str && !t->base_sha.empty() && !sha->str.empty() && sha->str != t->base_sha)
            return fail(t->ctx, TA_ERR_INVALID, "checkpoint was trained on another base (base_sha mismatch)");
        // the set of adapted projections decides the layout of the flat arrays: it must be the same
        static const struct { const char* key; int bit; } inj[] = {
            {"inject_q", TA_TARGET_Q}, {"inject_k", TA_TARGET_K}, {"inject_v", TA_TARGET_V}, {"inject_o", TA_TARGET_O},
            {"inject_gate", TA_TARGET_GATE}, {"inject_up", TA_TARGET_UP}, {"inject_down", TA_TARGET_DOWN}};
        for (const auto& i : inj) {
            const Json* v = j.get(i.key);
            if (!v) continue;
            if (v->kind != Json::Bool) continue;
            if (v->b != ((t->ac.targets & i.bit) != 0))
                return fail(t->ctx, TA_ERR_INVALID, std::string("checkpoint and adapter config disagree on ") + i.key);
        }
    } else {
        return fail(t->ctx, TA_ERR_IO, "cannot open " + (d / "adapter.json").string());
    }
    WeightFiles wf;
    std::string err;
    std::error_code ec;
    const long n = t->lora_n, D = t->mc.hidden;
    if (fs::exists(d / "optimizer.safetensors", ec)) {
        if (!add_shard((d / "optimizer.safetensors").string(), &wf, &err)) return fail(t->ctx, TA_ERR_IO, err);
        const struct { const char* name; float* dst; long len; } items[] = {
            {"lora.master", t->master, n}, {"lora.m", t->m, n}, {"lora.v", t->v, n}, {"centroid.acc", t->cen_acc, D},
            {"centroid.weight", t->cen_w, 1}, {"centroid_asbuilt.acc", t->cen_acc_ab, D}, {"centroid_asbuilt.weight", t->cen_w_ab, 1}};
        for (auto& it : items) {
            auto e = wf.entries.find(it.name);
            if (e == wf.entries.end() || e->second.dtype != 0 || e->second.numel() != it.len)
                return fail(t->ctx, TA_ERR_INVALID, std::string("optimizer.safetensors: missing or mis-sized ") + it.name +
                                                        " (another rank, target set or model?)");
            TA_CUDA(t->ctx, cudaMemcpyAsync(it.dst, e->second.data, size_t(it.len) * 4, cudaMemcpyHostToDevice, t->stream));
        }
        auto s = wf.entries.find("step"), k = wf.entries.find("tokens_consumed");
        if (s == wf.entries.end() || k == wf.entries.end() || s->second.bytes != 8 || k->second.bytes != 8)
            return fail(t->ctx, TA_ERR_INVALID, "optimizer.safetensors: missing step / tokens_consumed");
        auto tg = wf.entries.find("targets");
        if (tg != wf.entries.end() && tg->second.bytes == 8) {
            int64_t tv;
            std::memcpy(&tv, tg->second.data, 8);
            if (int(tv) != t->ac.targets)
                return fail(t->ctx, TA_ERR_INVALID, "optimizer.safetensors was written for another set of adapted projections");
        }
        int64_t sv, kv;
        std::memcpy(&sv, s->second.data, 8);
        std::memcpy(&kv, k->second.data, 8);
        t->step_count = long(sv);
        t->tokens_seen = long(kv);
    } else {
        if (!add_shard((d / "adapter.safetensors").string(), &wf, &err)) return fail(t->ctx, TA_ERR_IO, err);
        std::vector<float> master(static_cast<size_t>(n), 0.f);
        static const char* const proj[T_COUNT] = {"self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                                                  "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"};
        auto widen = [](uint16_t b) { uint32_t u = uint32_t(b) << 16; float f; std::memcpy(&f, &u, 4); return f; };
        for (int l = 0; l < t->mc.layers; l++)
            for (int tg = 0; tg < T_COUNT; tg++) {
                LoraSlot& sl = t->slot(l, tg);
                if (!sl.on) continue;
                const std::string base = "layers." + std::to_string(l) + "." + proj[tg];
                auto ea = wf.entries.find(base + ".lora_A"), eb = wf.entries.find(base + ".lora_B");
                const long na = long(t->ac.rank) * sl.in, nb = long(sl.out) * t->ac.rank;
                if (ea == wf.entries.end() || eb == wf.entries.end() || ea->second.dtype != 1 || eb->second.dtype != 1 ||
                    ea->second.numel() != na || eb->second.numel() != nb)
                    return fail(t->ctx, TA_ERR_INVALID, "adapter.safetensors: missing or mis-sized " + base);
                const uint16_t* pa = reinterpret_cast<const uint16_t*>(ea->second.data);
                const uint16_t* pb = reinterpret_cast<const uint16_t*>(eb->second.data);
                for (long i = 0; i < na; i++) master[size_t(sl.offA + i)] = widen(pa[i]);
                for (long o = 0; o < sl.out; o++)
                    for (int r = 0; r < t->ac.rank; r++) master[size_t(sl.offB + o * t->r_pad + r)] = widen(pb[o * t->ac.rank + r]);
            }
        TA_CUDA(t->ctx, cudaMemcpy(t->master, master.data(), size_t(n) * 4, cudaMemcpyHostToDevice));
        TA_CUDA(t->ctx, cudaMemsetAsync(t->m, 0, size_t(n) * 4, t->stream));
        TA_CUDA(t->ctx, cudaMemsetAsync(t->v, 0, size_t(n) * 4, t->stream));
        t->step_count = 0;
        t->tokens_seen = 0;
        if (read_text((d / "train_state.json").string(), &txt)) {
            Json j;
            if (parse_json(txt.data(), txt.size(), &j, &jerr) && j.kind == Json::Obj) {
                if (const Json* s = j.get("step")) if (s->kind == Json::Num) t->step_count = long(s->num);
                if (const Json* k = j.get("tokens_consumed")) if (k->kind == Json::Num) t->tokens_seen = long(k->num);
            }
        }
    }
    TA_CUDA(t->ctx, cudaStreamSynchronize(t->stream));   // the mapping goes away on return
    // Snapshots the interrupted run already wrote (<run>/centroids/step-N.centroid beside <run>/step-N) come back
    // into the in-memory list in step order, so that the final merge sees the whole run - the reference's
    // merge_and_write reads the directory when its list is empty (src/centroid/centroid_accumulator.cpp:93-107).
    t->snapshots.clear();
    const fs::path cdir = d.parent_path() / "centroids";
    if (fs::is_directory(cdir, ec)) {
        std::vector<std::pair<long, fs::path>> files;
        for (const auto& e : fs::directory_iterator(cdir, ec)) {
            const std::string name = e.path().filename().string();
            long sn = -1;
            if (e.path().extension() == ".centroid" && std::sscanf(name.c_str(), "step-%ld", &sn) == 1 && sn >= 0 && sn <= t->step_count)
                files.emplace_back(sn, e.path());
        }
        std::sort(files.begin(), files.end());
        for (const auto& f : files) {
            std::ifstream in(f.second, std::ios::binary);
            int dd = 0;
            in.read(reinterpret_cast<char*>(&dd), 4);
            if (!in || dd != t->mc.hidden) continue;
            std::vector<float> c(static_cast<size_t>(dd), 0.f);
            in.read(reinterpret_cast<char*>(c.data()), std::streamsize(size_t(dd) * 4));
            if (in) t->snapshots.push_back(std::move(c));
        }
    }
    return ta_trainer_sync_working(t);
}

}  // extern "C"
