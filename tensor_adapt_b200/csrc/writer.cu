// Files of the path: adapter.safetensors / adapter.json / train_state.json (byte-compatible with
// src/checkpoint/adapter_writer.cpp:30-159, which serialises through nlohmann::json: keys sorted,
// `dump()` compact for the safetensors header, `dump(2)` for the JSON files), centroid snapshots and
// the merged centroid file (src/centroid/centroid_accumulator.cpp:72-91,160-165).
#include <sys/stat.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <map>
#include <string>
#include <vector>

#include "trainer.h"

namespace fs = std::filesystem;

namespace ta {
namespace {

std::string json_string(const std::string& s) {
    std::string o = "\"";
    for (unsigned char ch : s) {
        switch (ch) {
            case '"': o += "\\\""; break;
            case '\\': o += "\\\\"; break;
            case '\b': o += "\\b"; break;
            case '\f': o += "\\f"; break;
            case '\n': o += "\\n"; break;
            case '\r': o += "\\r"; break;
            case '\t': o += "\\t"; break;
            default:
                if (ch < 0x20) { char b[8]; std::snprintf(b, sizeof(b), "\\u%04x", ch); o += b; }
                else o += char(ch);
        }
    }
    return o + "\"";
}

// Text of a double as nlohmann::json prints it: shortest digits that round-trip, fixed notation for
// decimal exponents in (-4, 15], otherwise d.ddde+XX; integers get a trailing ".0".
std::string json_double(double v) {
    if (!std::isfinite(v)) return "null";
    if (v == 0) return std::signbit(v) ? "-0.0" : "0.0";
    char buf[40];
    int prec = 1;
    for (; prec <= 17; prec++) {
        std::snprintf(buf, sizeof(buf), "%.*e", prec - 1, v);
        if (std::strtod(buf, nullptr) == v) break;
    }
    std::string t(buf);
    const bool neg = t[0] == '-';
    if (neg) t.erase(0, 1);
    const size_t e = t.find('e');
    std::string digits = t.substr(0, e);
    const int exp10 = std::atoi(t.c_str() + e + 1);
    digits.erase(std::remove(digits.begin(), digits.end(), '.'), digits.end());
    while (digits.size() > 1 && digits.back() == '0') digits.pop_back();
    const int k = int(digits.size()), n = exp10 + 1;   // value = 0.digits * 10^n
    std::string o;
    if (k <= n && n <= 15) o = digits + std::string(size_t(n - k), '0') + ".0";
    else if (0 < n && n <= 15) o = digits.substr(0, size_t(n)) + "." + digits.substr(size_t(n));
    else if (-4 < n && n <= 0) o = "0." + std::string(size_t(-n), '0') + digits;
    else {
        o = digits.substr(0, 1);
        if (k > 1) o += "." + digits.substr(1);
        const int ex = n - 1;
        char eb[16];
        std::snprintf(eb, sizeof(eb), "e%c%02d", ex < 0 ? '-' : '+', std::abs(ex));
        o += eb;
    }
    return (neg ? "-" : "") + o;
}

uint16_t bf16_rne(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF;
    u += ((u >> 16) & 1u) + 0x7FFFu;
    return uint16_t(u >> 16);
}

const char* const kProjNames[T_COUNT] = {"self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                                         "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"};

bool write_file(const std::string& path, const void* data, size_t n) {
    std::ofstream f(path, std::ios::binary);
    if (!f) return false;
    f.write(static_cast<const char*>(data), std::streamsize(n));
    return bool(f);
}

}  // namespace
}  // namespace ta

using namespace ta;

extern "C" {

int ta_trainer_set_meta(ta_trainer* t, const char* arch_name, const char* base_sha) {
    if (!t) return TA_ERR_INVALID;
    t->arch_name = arch_name ? arch_name : "";
    t->base_sha = base_sha ? base_sha : "";
    return TA_OK;
}

int ta_trainer_save_checkpoint(ta_trainer* t, const char* dir, const char* domain, long step, long tokens, int final_) {
    if (!t || !dir) return TA_ERR_INVALID;
    TA_CUDA(t->ctx, cudaStreamSynchronize(t->stream));
    std::error_code ec;
    fs::create_directories(dir, ec);
    std::vector<float> master(size_t(t->lora_n));
    TA_CUDA(t->ctx, cudaMemcpy(master.data(), t->master, master.size() * 4, cudaMemcpyDeviceToHost));

    // data section in insertion order (layer, projection, A then B); header text key-sorted
    std::map<std::string, std::string> entries;
    std::vector<uint16_t> data;
    for (int l = 0; l < t->mc.layers; l++)
        for (int tg = 0; tg < T_COUNT; tg++) {
            LoraSlot& sl = t->slot(l, tg);
            if (!sl.on) continue;
            for (int ab = 0; ab < 2; ab++) {
                const size_t begin = data.size() * 2;
                size_t numel;
                if (ab == 0) {
                    numel = size_t(t->ac.rank) * sl.in;
                    for (size_t i = 0; i < numel; i++) data.push_back(bf16_rne(master[size_t(sl.offA) + i]));
                } else {
                    numel = size_t(sl.out) * t->ac.rank;
                    for (int o = 0; o < sl.out; o++)
                        for (int r = 0; r < t->ac.rank; r++)
                            data.push_back(bf16_rne(master[size_t(sl.offB) + size_t(o) * t->r_pad + r]));
                }
                const std::string name = "layers." + std::to_string(l) + "." + kProjNames[tg] + (ab ? ".lora_B" : ".lora_A");
                entries[name] = "{\"data_offsets\":[" + std::to_string(begin) + "," + std::to_string(begin + numel * 2) +
                                "],\"dtype\":\"BF16\",\"shape\":[" + std::to_string(numel) + "]}";
            }
        }
    std::string hdr = "{";
    bool first = true;
    for (auto& kv : entries) {
        if (!first) hdr += ",";
        first = false;
        hdr += json_string(kv.first) + ":" + kv.second;
    }
    hdr += "}";
    while (hdr.size() % 8) hdr += ' ';
    const uint64_t hlen = hdr.size();
    {
        std::ofstream f(std::string(dir) + "/adapter.safetensors", std::ios::binary);
        if (!f) return fail(t->ctx, TA_ERR_IO, std::string("cannot write into ") + dir);
        f.write(reinterpret_cast<const char*>(&hlen), 8);
        f.write(hdr.data(), std::streamsize(hlen));
        f.write(reinterpret_cast<const char*>(data.data()), std::streamsize(data.size() * 2));
    }
    // adapter.json (src/checkpoint/adapter_writer.cpp:103-124), keys in sorted order
    const int tg = t->ac.targets;
    std::map<std::string, std::string> j;
    j["domain"] = json_string(domain ? domain : "");
    j["architecture"] = json_string(t->arch_name);
    j["base_model"] = json_string("unknown");
    j["base_sha"] = json_string(t->base_sha);
    j["rank"] = std::to_string(t->ac.rank);
    j["alpha"] = json_double(double(t->ac.alpha));
    j["target_begin"] = "0";
    j["target_end"] = std::to_string(t->mc.layers - 1);
    j["inject_q"] = (tg & TA_TARGET_Q) ? "true" : "false";
    j["inject_k"] = (tg & TA_TARGET_K) ? "true" : "false";
    j["inject_v"] = (tg & TA_TARGET_V) ? "true" : "false";
    j["inject_o"] = (tg & TA_TARGET_O) ? "true" : "false";
    j["inject_up"] = (tg & TA_TARGET_UP) ? "true" : "false";
    j["inject_down"] = (tg & TA_TARGET_DOWN) ? "true" : "false";
    if (tg & TA_TARGET_GATE) j["inject_gate"] = "true";   // extension: the reference has no such key
    j["tokens_trained"] = std::to_string(tokens);
    j["centroid_dim"] = std::to_string(t->mc.hidden);
    j["centroid_count"] = "16";
    j["step"] = std::to_string(step);
    j["tensor_adapt_version"] = json_string("0.1.0");
    std::string txt = "{\n";
    size_t i = 0;
    for (auto& kv : j) txt += "  " + json_string(kv.first) + ": " + kv.second + (++i < j.size() ? ",\n" : "\n");
    txt += "}";
    if (!write_file(std::string(dir) + "/adapter.json", txt.data(), txt.size()))
        return fail(t->ctx, TA_ERR_IO, "cannot write adapter.json");
    if (!final_) {
        const std::string st = "{\n  \"step\": " + std::to_string(step) + ",\n  \"tokens_consumed\": " + std::to_string(tokens) + "\n}";
        if (!write_file(std::string(dir) + "/train_state.json", st.data(), st.size()))
            return fail(t->ctx, TA_ERR_IO, "cannot write train_state.json");
    }
    return TA_OK;
}

int ta_trainer_write_snapshot(ta_trainer* t, int mode, const char* path, float* centroid_out, float* weight_out) {
    if (!t || (mode != 0 && mode != 1)) return TA_ERR_INVALID;
    const int D = t->mc.hidden;
    TA_CUDA(t->ctx, cudaStreamSynchronize(t->stream));
    std::vector<float> acc(static_cast<size_t>(D), 0.f);
    float w = 0.f;
    TA_CUDA(t->ctx, cudaMemcpy(acc.data(), mode == 0 ? t->cen_acc : t->cen_acc_ab, size_t(D) * 4, cudaMemcpyDeviceToHost));
    TA_CUDA(t->ctx, cudaMemcpy(&w, mode == 0 ? t->cen_w : t->cen_w_ab, 4, cudaMemcpyDeviceToHost));
    if (weight_out) *weight_out = w;
    if (w == 0.f) return TA_OK;
    for (int d = 0; d < D; d++) acc[size_t(d)] = acc[size_t(d)] / w;
    if (centroid_out) std::memcpy(centroid_out, acc.data(), size_t(D) * 4);
    if (path) {
        std::ofstream f(path, std::ios::binary);
        if (!f) return fail(t->ctx, TA_ERR_IO, std::string("cannot write ") + path);
        f.write(reinterpret_cast<const char*>(&D), 4);
        f.write(reinterpret_cast<const char*>(acc.data()), std::streamsize(size_t(D) * 4));
        f.write(reinterpret_cast<const char*>(&w), 4);
    }
    t->snapshots.push_back(acc);
    return TA_OK;
}

// One record of the reference's snapshot layout per layer, back to back (a "bank"): int32 D | D x f32 | f32 weight.
// Layers whose weight is still zero are left out, like the reference skips an empty accumulator.
extern "C" int ta_trainer_write_snapshot_bank(ta_trainer* t, const char* path, float* centroids_out, float* weights_out,
                                              int* n_records) {
    if (!t) return TA_ERR_INVALID;
    if (!(t->ac.centroid_modes & 4)) return fail(t->ctx, TA_ERR_INVALID, "snapshot bank: the trainer was created without centroid mode 4");
    const int D = t->mc.hidden, L = t->mc.layers;
    TA_CUDA(t->ctx, cudaStreamSynchronize(t->stream));
    std::vector<float> acc(size_t(L) * D), w(static_cast<size_t>(L));
    TA_CUDA(t->ctx, cudaMemcpy(acc.data(), t->cen_bank, acc.size() * 4, cudaMemcpyDeviceToHost));
    TA_CUDA(t->ctx, cudaMemcpy(w.data(), t->cen_bank_w, w.size() * 4, cudaMemcpyDeviceToHost));
    for (int l = 0; l < L; l++)
        if (w[size_t(l)] != 0.f)
            for (int d = 0; d < D; d++) acc[size_t(l) * D + d] = acc[size_t(l) * D + d] / w[size_t(l)];
    if (centroids_out) std::memcpy(centroids_out, acc.data(), acc.size() * 4);
    if (weights_out) std::memcpy(weights_out, w.data(), w.size() * 4);
    int n = 0;
    std::ofstream f;
    if (path) {
        f.open(path, std::ios::binary);
        if (!f) return fail(t->ctx, TA_ERR_IO, std::string("cannot write ") + path);
    }
    for (int l = 0; l < L; l++) {
        if (w[size_t(l)] == 0.f) continue;
        n++;
        if (!path) continue;
        f.write(reinterpret_cast<const char*>(&D), 4);
        f.write(reinterpret_cast<const char*>(acc.data() + size_t(l) * D), std::streamsize(size_t(D) * 4));
        f.write(reinterpret_cast<const char*>(&w[size_t(l)]), 4);
    }
    if (n_records) *n_records = n;
    return TA_OK;
}

struct MergeOptions {
    bool extended = false;           // seeded k-means++ / mass ranking instead of the reference's merge
    int init_mode = 0, rank = 0;
    unsigned long long seed = 0;
    const std::vector<float>* mass = nullptr;
};

static int merge_vectors(ta_ctx* ctx, const std::vector<std::vector<float>>& snaps, int D, int k, const char* out_path,
                         int* passes, const MergeOptions& mo = MergeOptions()) {
    const int N = int(snaps.size());
    std::vector<float> flat(size_t(N) * D);
    for (int n = 0; n < N; n++) std::memcpy(flat.data() + size_t(n) * D, snaps[size_t(n)].data(), size_t(D) * 4);
    const int kk = std::min(k, N);
    DeviceBuffer bv, bc, ba, bm;
    TA_CUDA(ctx, bv.alloc(flat.size() * 4));
    TA_CUDA(ctx, bc.alloc(size_t(kk) * D * 4));
    TA_CUDA(ctx, ba.alloc(size_t(N) * 4));
    float *dv = bv.as<float>(), *dc = bc.as<float>();
    int* da = ba.as<int>();
    TA_CUDA(ctx, cudaMemcpy(dv, flat.data(), flat.size() * 4, cudaMemcpyHostToDevice));
    int kout = 0;
    int rc;
    if (mo.extended) {
        if (mo.mass) {
            TA_CUDA(ctx, bm.alloc(size_t(N) * 4));
            TA_CUDA(ctx, cudaMemcpy(bm.p, mo.mass->data(), size_t(N) * 4, cudaMemcpyHostToDevice));
        }
        rc = ta_kmeans_merge_ex(ctx, dv, bm.as<float>(), N, D, k, 50, mo.init_mode, mo.seed, mo.rank, dc, da, nullptr, nullptr, &kout,
                                passes, nullptr);
    } else {
        rc = ta_kmeans_merge(ctx, dv, N, D, k, 50, dc, da, &kout, passes, nullptr);
    }
    if (rc) return rc;
    std::vector<float> centers(size_t(kk) * D);
    TA_CUDA(ctx, cudaStreamSynchronize(nullptr));
    TA_CUDA(ctx, cudaMemcpy(centers.data(), dc, centers.size() * 4, cudaMemcpyDeviceToHost));
    std::ofstream f(out_path, std::ios::binary);
    if (!f) return fail(ctx, TA_ERR_IO, std::string("cannot write ") + out_path);
    f.write(reinterpret_cast<const char*>(&kout), 4);
    f.write(reinterpret_cast<const char*>(&D), 4);
    f.write(reinterpret_cast<const char*>(centers.data()), std::streamsize(centers.size() * 4));
    return TA_OK;
}

static int merge_dir(ta_ctx* ctx, const char* dir, const char* out_path, int k, int* n_vectors, int* passes, MergeOptions mo) {
    if (!ctx || !dir || !out_path || k <= 0) return fail(ctx, TA_ERR_INVALID, "centroid_merge_dir: bad argument");
    std::error_code ec;
    int D = 0;
    for (const auto& e : fs::directory_iterator(dir, ec)) {
        if (e.path().extension() == ".centroid") {
            std::ifstream f(e.path(), std::ios::binary);
            f.read(reinterpret_cast<char*>(&D), 4);
            break;
        }
    }
    if (ec || D <= 0) return fail(ctx, TA_ERR_IO, std::string("No .centroid files in ") + dir);
    std::vector<std::vector<float>> snaps;
    std::vector<float> mass;
    for (const auto& e : fs::directory_iterator(dir, ec)) {
        if (e.path().extension() != ".centroid") continue;
        std::ifstream f(e.path(), std::ios::binary);
        int d = 0;
        f.read(reinterpret_cast<char*>(&d), 4);
        if (d != D) continue;
        std::vector<float> c(size_t(d), 0.f);
        f.read(reinterpret_cast<char*>(c.data()), std::streamsize(size_t(d) * 4));
        float w = 0.f;   // trailing accumulated gradient mass; the reference's merge never reads it
        f.read(reinterpret_cast<char*>(&w), 4);
        snaps.push_back(std::move(c));
        mass.push_back(w);
        // A bank file carries further records of the same layout.  The reference's reader stops after the first
        // (src/centroid/centroid_accumulator.cpp:96-106) and so does the reference-mode merge; the extended merge
        // clusters every vector of every file.
        while (mo.extended && f) {
            int d2 = 0;
            f.read(reinterpret_cast<char*>(&d2), 4);
            if (!f || d2 != D) break;
            std::vector<float> c2(size_t(D), 0.f);
            f.read(reinterpret_cast<char*>(c2.data()), std::streamsize(size_t(D) * 4));
            float w2 = 0.f;
            f.read(reinterpret_cast<char*>(&w2), 4);
            if (!f) break;
            snaps.push_back(std::move(c2));
            mass.push_back(w2);
        }
    }
    if (n_vectors) *n_vectors = int(snaps.size());
    if (snaps.empty()) return TA_OK;   // the reference logs "no snapshots to merge" and writes nothing
    if (mo.extended) mo.mass = &mass;
    return merge_vectors(ctx, snaps, D, k, out_path, passes, mo);
}

int ta_centroid_merge_dir(ta_ctx* ctx, const char* dir, const char* out_path, int k, int* n_vectors, int* passes) {
    return merge_dir(ctx, dir, out_path, k, n_vectors, passes, MergeOptions());
}

int ta_centroid_merge_dir_ex(ta_ctx* ctx, const char* dir, const char* out_path, int k, int init_mode, unsigned long long seed,
                             int rank_by_mass, int* n_vectors, int* passes) {
    MergeOptions mo;
    mo.extended = true; mo.init_mode = init_mode; mo.seed = seed; mo.rank = rank_by_mass;
    return merge_dir(ctx, dir, out_path, k, n_vectors, passes, mo);
}

int ta_trainer_merge_snapshots(ta_trainer* t, int k, const char* out_path, int* passes) {
    if (!t || !out_path || k <= 0) return TA_ERR_INVALID;
    if (t->snapshots.empty()) return TA_OK;
    return merge_vectors(t->ctx, t->snapshots, t->mc.hidden, k, out_path, passes);
}

}  // extern "C"
