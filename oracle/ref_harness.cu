// Test infrastructure, not product code.
//
// Driver that runs the UNMODIFIED reference (objects compiled by oracle/Makefile from the
// reference tree) on seeded inputs read from raw files, and dumps its results as raw files.
// The parity tests compare the package's CUDA path with these dumps; bench.py's reference
// arm uses the `bench` mode.  Nothing here is linked into the product library.
//
// Modes
//   ref_harness op      <case_dir> <out_dir>   one LoRA linear: y = x.W^T + s.B(A.x) and its
//                                              backward, through gemm_bf16 with the GemmParams of
//                                              src/base/arch/qwen2.cu:21-41 and
//                                              AdapterModel::apply_lora_fwd/bwd
//   ref_harness step    <case_dir> <out_dir>   Qwen2Base::forward -> ops::cross_entropy_fwd ->
//                                              Qwen2Base::backward -> centroid accumulate ->
//                                              grad-norm / clip -> AdamW::step_all, i.e. the body of
//                                              src/trainer/adapt_trainer.cu:190-253 with injected weights
//   ref_harness trainer <case_dir> <out_dir>   AdaptTrainer::create + step() through the public API
//   ref_harness bench   <case_dir>             timing of the `step` body on random weights; one JSON line
//
// Case directories hold `cfg.txt` ("key value" per line) and raw little-endian arrays.

#include <tensor/adapter/adapter_config.hpp>
#include <tensor/adapter/adapter_model.hpp>
#include <tensor/backend/cuda/device.hpp>
#include <tensor/backend/cuda/ops.hpp>
#include <tensor/backend/cuda/tensor.hpp>
#include <tensor/base/arch/qwen2.hpp>
#include <tensor/base/base_loader.hpp>
#include <tensor/base/frozen_base.hpp>
#include <tensor/centroid/centroid_accumulator.hpp>
#include <tensor/checkpoint/adapter_writer.hpp>
#include <tensor/data/dataset.hpp>
#include <tensor/trainer/adamw.hpp>
#include <tensor/trainer/adapt_trainer.hpp>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <iostream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

namespace fs = std::filesystem;
using namespace tensor;
using backend::cuda::Device;
using backend::cuda::GemmParams;
using backend::cuda::Tensor;
namespace ops = backend::cuda::ops;
using core::DType;

// ───────────────────────── small file helpers ─────────────────────────

static std::map<std::string, std::string> read_cfg(const std::string& dir) {
    std::map<std::string, std::string> m;
    std::ifstream f(dir + "/cfg.txt");
    if (!f) { std::cerr << "no cfg.txt in " << dir << "\n"; std::exit(2); }
    std::string k, v;
    while (f >> k >> v) m[k] = v;
    return m;
}
static long   geti(const std::map<std::string, std::string>& m, const char* k, long d) {
    auto it = m.find(k); return it == m.end() ? d : std::stol(it->second);
}
static double getf(const std::map<std::string, std::string>& m, const char* k, double d) {
    auto it = m.find(k); return it == m.end() ? d : std::stod(it->second);
}
static bool exists(const std::string& p) { return fs::exists(p); }

static std::vector<char> slurp(const std::string& p) {
    std::ifstream f(p, std::ios::binary | std::ios::ate);
    if (!f) { std::cerr << "cannot open " << p << "\n"; std::exit(2); }
    std::size_t n = f.tellg();
    std::vector<char> b(n);
    f.seekg(0);
    f.read(b.data(), n);
    return b;
}
static void dump(const std::string& p, const void* d, std::size_t n) {
    std::ofstream f(p, std::ios::binary);
    f.write(static_cast<const char*>(d), n);
}
static void dump_tensor(const std::string& p, const Tensor& t) {
    std::vector<char> h(t.nbytes());
    cudaMemcpy(h.data(), t.data(), t.nbytes(), cudaMemcpyDeviceToHost);
    dump(p, h.data(), h.size());
}

// Deterministic device fill, bit-identical to the package's ta_trainer_init_random (seed 0): approximately
// normal N(0, std) BF16 values as the centred sum of twelve 16-bit hash fields, scaled with single
// correctly-rounded operations so that this file's --use_fast_math build produces the same bits.  Lets both
// implementations start from identical multi-gigabyte weights without writing them to disk.
__device__ static unsigned long long k_mix64(unsigned long long z) {
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull; z ^= z >> 27; z *= 0x94D049BB133111EBull; z ^= z >> 31;
    return z;
}
__global__ void k_fill_normal(__nv_bfloat16* p, std::size_t n, float stdv, unsigned seed) {
    std::size_t i = blockIdx.x * (std::size_t)blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float c = __fmul_rn(stdv, 1.52587890625e-05f);
    const unsigned long long x = (unsigned long long)(i + 1) * 0x9E3779B97F4A7C15ull + (unsigned long long)seed * 0xD1B54A32D192ED03ull;
    const unsigned long long z[3] = {k_mix64(x), k_mix64(x ^ 0xA5A5A5A5A5A5A5A5ull), k_mix64(x + 0x632BE59BD9B4E019ull)};
    int sum = 0;
    for (int k = 0; k < 3; k++)
        sum += int(z[k] & 0xFFFF) + int((z[k] >> 16) & 0xFFFF) + int((z[k] >> 32) & 0xFFFF) + int(z[k] >> 48);
    p[i] = __float2bfloat16_rn(__fmul_rn(__int2float_rn(sum - 6 * 65535), c));
}
__global__ void k_fill_const(__nv_bfloat16* p, std::size_t n, float v) {
    std::size_t i = blockIdx.x * (std::size_t)blockDim.x + threadIdx.x;
    if (i < n) p[i] = __float2bfloat16(v);
}

static Tensor load_or_fill_bf16(const std::string& path, core::Shape shape, const Device& dev,
                                float stdv, unsigned seed, float constant = -1.f) {
    if (exists(path)) {
        auto b = slurp(path);
        core::TensorView v{b.data(), DType::BF16, shape};
        if (b.size() != v.nbytes()) { std::cerr << "size mismatch " << path << "\n"; std::exit(2); }
        return Tensor::from_host(v, dev);
    }
    Tensor t = Tensor::empty_bf16(shape, dev);
    std::size_t n = t.numel();
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (constant >= 0.f) k_fill_const<<<blocks, 256, 0, dev.stream()>>>(t.bf16(), n, constant);
    else                 k_fill_normal<<<blocks, 256, 0, dev.stream()>>>(t.bf16(), n, stdv, seed);
    return t;
}
static Tensor load_f32(const std::string& path, core::Shape shape, const Device& dev) {
    auto b = slurp(path);
    core::TensorView v{b.data(), DType::F32, shape};
    if (b.size() != v.nbytes()) { std::cerr << "size mismatch " << path << "\n"; std::exit(2); }
    return Tensor::from_host(v, dev);
}

// ───────────────────────── model construction ─────────────────────────

static base::FrozenBase make_base(const std::map<std::string, std::string>& c,
                                  const std::string& dir, const Device& dev) {
    base::FrozenBase b;
    base::BaseConfig& bc = b.config;
    bc.arch_name = "qwen2"; bc.arch = base::ArchType::Qwen2; bc.base_sha = "synthetic";
    bc.vocab_size = geti(c, "vocab", 0);   bc.hidden_size = geti(c, "hidden", 0);
    bc.num_layers = geti(c, "layers", 0);  bc.num_q_heads = geti(c, "hq", 0);
    bc.num_kv_heads = geti(c, "hkv", 0);   bc.head_dim = geti(c, "hd", 0);
    bc.intermediate_size = geti(c, "inter", 0);
    bc.rms_norm_eps = (float)getf(c, "eps", 1e-6); bc.rope_theta = (float)getf(c, "theta", 1e6);
    bc.tie_embeddings = geti(c, "tie", 1) != 0;
    std::size_t V = bc.vocab_size, H = bc.hidden_size, I = bc.intermediate_size;
    std::size_t qd = bc.num_q_heads * bc.head_dim, kv = bc.num_kv_heads * bc.head_dim;
    float sd = (float)getf(c, "init_std", 0.02);
    unsigned s = 1;
    b.embed_w      = load_or_fill_bf16(dir + "/embed.bin", {V, H}, dev, sd, s++);
    b.final_norm_w = load_or_fill_bf16(dir + "/final_norm.bin", {H}, dev, 0, 0, 1.f);
    if (!bc.tie_embeddings) b.lm_head_w = load_or_fill_bf16(dir + "/lm_head.bin", {V, H}, dev, sd, s++);
    b.layers.resize(bc.num_layers);
    for (std::size_t l = 0; l < bc.num_layers; l++) {
        auto& w = b.layers[l];
        std::string p = dir + "/l" + std::to_string(l) + "_";
        w.input_norm_w = load_or_fill_bf16(p + "input_norm.bin", {H}, dev, 0, 0, 1.f);
        w.post_norm_w  = load_or_fill_bf16(p + "post_norm.bin",  {H}, dev, 0, 0, 1.f);
        w.q_proj_w = load_or_fill_bf16(p + "q_w.bin", {qd, H}, dev, sd, s++);
        w.k_proj_w = load_or_fill_bf16(p + "k_w.bin", {kv, H}, dev, sd, s++);
        w.v_proj_w = load_or_fill_bf16(p + "v_w.bin", {kv, H}, dev, sd, s++);
        w.o_proj_w = load_or_fill_bf16(p + "o_w.bin", {H, qd}, dev, sd, s++);
        w.q_proj_b = load_or_fill_bf16(p + "q_b.bin", {qd}, dev, sd, s++);
        w.k_proj_b = load_or_fill_bf16(p + "k_b.bin", {kv}, dev, sd, s++);
        w.v_proj_b = load_or_fill_bf16(p + "v_b.bin", {kv}, dev, sd, s++);
        w.gate_proj_w = load_or_fill_bf16(p + "gate_w.bin", {I, H}, dev, sd, s++);
        w.up_proj_w   = load_or_fill_bf16(p + "up_w.bin",   {I, H}, dev, sd, s++);
        w.down_proj_w = load_or_fill_bf16(p + "down_w.bin", {H, I}, dev, sd, s++);
    }
    dev.sync();
    return b;
}

static adapter::AdapterConfig make_acfg(const std::map<std::string, std::string>& c) {
    adapter::AdapterConfig a;
    a.rank = (int)geti(c, "rank", 16);       a.alpha = (float)getf(c, "alpha", 32);
    a.lr = (float)getf(c, "lr", 2e-4);       a.grad_clip = (float)getf(c, "grad_clip", 1.0);
    a.warmup_steps = geti(c, "warmup", 1);   a.adam_beta1 = (float)getf(c, "beta1", 0.9);
    a.adam_beta2 = (float)getf(c, "beta2", 0.999); a.weight_decay = (float)getf(c, "wd", 0.01);
    a.batch_size = geti(c, "B", 1);          a.seq_len = geti(c, "T", 128);
    a.architecture = "qwen2";
    return a;
}

static const char* PN[4] = {"q", "k", "v", "o"};
static adapter::LoraPair* pair_of(adapter::LayerAdapter& la, int i) {
    return i == 0 ? &la.lora_q : i == 1 ? &la.lora_k : i == 2 ? &la.lora_v : &la.lora_o;
}

// Replace the hash-initialised A / zero B by the case's F32 masters; the BF16 working copy is
// the device-side RNE cast the optimiser itself uses (ops::cast_f32_to_bf16).
static void inject_lora(adapter::AdapterModel& m, const std::string& dir, const Device& dev) {
    for (std::size_t l = 0; l < m.layers.size(); l++)
        for (int i = 0; i < 4; i++) {
            adapter::LoraPair* lp = pair_of(m.layers[l], i);
            std::string p = dir + "/l" + std::to_string(l) + "_lora_" + PN[i];
            if (!exists(p + "_A.bin")) continue;
            lp->A_f32 = load_f32(p + "_A.bin", {(std::size_t)lp->rank, (std::size_t)lp->in_dim}, dev);
            lp->B_f32 = load_f32(p + "_B.bin", {(std::size_t)lp->out_dim, (std::size_t)lp->rank}, dev);
            ops::cast_f32_to_bf16(lp->A_f32.f32(), lp->A_bf16.bf16(), lp->rank * lp->in_dim, dev.stream());
            ops::cast_f32_to_bf16(lp->B_f32.f32(), lp->B_bf16.bf16(), lp->out_dim * lp->rank, dev.stream());
        }
    dev.sync();
}

__global__ static void k_scale(float* g, int N, float s) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < N) g[i] *= s;
}

// Same launches as compute_grad_norm / clip_gradients (src/trainer/adapt_trainer.cu:32-70), which
// are file-static there: ops::sum_sq_into per tensor into one scalar, sqrt on the host, and a
// scale of max/(norm+1e-6) when norm > max.
static float grad_norm_and_clip(adapter::AdapterModel& m, float max_norm, const Device& dev) {
    Tensor acc = Tensor::zeros_f32({1}, dev);
    for (auto& la : m.layers)
        for (int i = 0; i < 4; i++) {
            adapter::LoraPair* lp = pair_of(la, i);
            ops::sum_sq_into(lp->gA.f32(), acc.f32(), lp->rank * lp->in_dim, dev.stream());
            ops::sum_sq_into(lp->gB.f32(), acc.f32(), lp->out_dim * lp->rank, dev.stream());
        }
    dev.sync();
    float norm = std::sqrt(acc.to_host_f32()[0]);
    if (norm > max_norm) {
        float s = max_norm / (norm + 1e-6f);
        for (auto& la : m.layers)
            for (int i = 0; i < 4; i++) {
                adapter::LoraPair* lp = pair_of(la, i);
                int nA = lp->rank * lp->in_dim, nB = lp->out_dim * lp->rank;
                k_scale<<<(nA + 255) / 256, 256, 0, dev.stream()>>>(lp->gA.f32(), nA, s);
                k_scale<<<(nB + 255) / 256, 256, 0, dev.stream()>>>(lp->gB.f32(), nB, s);
            }
    }
    return norm;
}

// A tensor whose dtype tag says F32 (so CentroidAccumulator::accumulate's to_host_f32() does not
// throw) but whose leading bytes are the BF16 payload that accumulate() then reads through
// .bf16(): this feeds the reference's own loop (src/centroid/centroid_accumulator.cpp:54-69) the
// correctly-typed data its header documents.
static Tensor bf16_payload_in_f32_tensor(const Tensor& src, const Device& dev) {
    Tensor t = Tensor::zeros(src.shape(), DType::F32, dev);
    cudaMemcpyAsync(t.data(), src.data(), src.nbytes(), cudaMemcpyDeviceToDevice, dev.stream());
    return t;
}

// ───────────────────────── mode: op ─────────────────────────

static int mode_op(const std::string& dir, const std::string& out) {
    auto c = read_cfg(dir);
    int BT = (int)geti(c, "BT", 0), in = (int)geti(c, "in", 0), od = (int)geti(c, "out", 0);
    int r = (int)geti(c, "rank", 16);
    Device dev = Device::open("cuda:0");
    std::size_t sBT = BT, sin = in, sod = od, sr = r;

    // A one-layer stub base so AdapterModel::create can size its pairs; only lora_q is used and
    // then re-shaped to (in -> out).
    base::FrozenBase b; b.config.hidden_size = in; b.config.num_layers = 1;
    b.config.num_kv_heads = 1; b.config.head_dim = od;
    adapter::AdapterConfig a = make_acfg(c);
    adapter::AdapterModel m = adapter::AdapterModel::create(b, a, dev);
    adapter::LoraPair& lp = m.layers[0].lora_k;   // in = hidden, out = kv = od
    lp.A_f32 = load_f32(dir + "/A.bin", {sr, sin}, dev);
    lp.B_f32 = load_f32(dir + "/B.bin", {sod, sr}, dev);
    ops::cast_f32_to_bf16(lp.A_f32.f32(), lp.A_bf16.bf16(), r * in, dev.stream());
    ops::cast_f32_to_bf16(lp.B_f32.f32(), lp.B_bf16.bf16(), od * r, dev.stream());

    Tensor x  = load_or_fill_bf16(dir + "/x.bin",  {sBT, sin}, dev, 1, 1);
    Tensor W  = load_or_fill_bf16(dir + "/W.bin",  {sod, sin}, dev, 1, 2);
    Tensor dY = load_or_fill_bf16(dir + "/dY.bin", {sBT, sod}, dev, 1, 3);
    Tensor y  = Tensor::empty_bf16({sBT, sod}, dev);
    Tensor dX = Tensor::zeros({sBT, sin}, DType::BF16, dev);

    int iters = (int)geti(c, "iters", 1);
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    float best = 1e30f;
    for (int it = 0; it < iters; it++) {
        lp.gA.zero_(dev); lp.gB.zero_(dev);
        cudaEventRecord(e0, dev.stream());
        {   // proj_fwd, src/base/arch/qwen2.cu:21-30
            GemmParams p; p.transA = true; p.transB = false; p.M = od; p.N = BT; p.K = in;
            backend::cuda::gemm_bf16(dev, p, W.bf16(), in, x.bf16(), in, y.bf16(), od);
        }
        m.apply_lora_fwd(0, lp, x, y, BT, dev);
        {   // proj_bwd_x, src/base/arch/qwen2.cu:32-41 (beta = 0)
            GemmParams p; p.M = in; p.N = BT; p.K = od;
            backend::cuda::gemm_bf16(dev, p, W.bf16(), in, dY.bf16(), od, dX.bf16(), in);
        }
        m.apply_lora_bwd(lp, x, dY, dX, BT, dev);
        cudaEventRecord(e1, dev.stream());
        dev.sync();
        float ms; cudaEventElapsedTime(&ms, e0, e1); best = std::min(best, ms);
    }
    fs::create_directories(out);
    dump_tensor(out + "/y.bin", y);   dump_tensor(out + "/dX.bin", dX);
    dump_tensor(out + "/gA.bin", lp.gA); dump_tensor(out + "/gB.bin", lp.gB);
    std::printf("{\"mode\":\"op\",\"best_ms\":%.6f,\"iters\":%d}\n", best, iters);
    return 0;
}

// ───────────────────────── mode: step / bench ─────────────────────────

struct StepOut { float norm; double ms; };

static int mode_step(const std::string& dir, const std::string& out, bool bench) {
    auto c = read_cfg(dir);
    Device dev = Device::open("cuda:0");
    std::cerr << "[harness] dev.sm_major()=" << dev.sm_major() << " (>= 8 selects the batched cuBLAS SDPA path)\n";
    base::FrozenBase b = make_base(c, dir, dev);
    adapter::AdapterConfig a = make_acfg(c);
    adapter::AdapterModel m = adapter::AdapterModel::create(b, a, dev);
    if (!bench) inject_lora(m, dir, dev);
    trainer::AdamW opt(a);
    const base::BaseConfig& bc = b.config;
    int B = (int)a.batch_size, T = (int)a.seq_len, BT = B * T;
    int steps = (int)geti(c, "steps", 1), warm = (int)geti(c, "warmup_iters", 0);
    bool do_centroid = geti(c, "centroid", 1) != 0;
    if (!bench) fs::create_directories(out);

    centroid::CentroidAccumulator acc_asbuilt((int)bc.hidden_size, (bench ? dir : out) + "/centroids_asbuilt");
    centroid::CentroidAccumulator acc_typed  ((int)bc.hidden_size, (bench ? dir : out) + "/centroids_intended");

    std::vector<int32_t> tok(BT), tgt(BT);
    std::vector<double> times;
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);

    for (int s = 0; s < steps + warm; s++) {
        std::string ts = dir + "/tokens_" + std::to_string(s) + ".bin";
        if (exists(ts)) {
            auto tb = slurp(ts); std::memcpy(tok.data(), tb.data(), BT * 4);
            auto gb = slurp(dir + "/targets_" + std::to_string(s) + ".bin");
            std::memcpy(tgt.data(), gb.data(), BT * 4);
        } else {
            unsigned long long z = 0x1234567ull + s;
            for (int i = 0; i < BT; i++) {
                z = z * 6364136223846793005ull + 1442695040888963407ull;
                tok[i] = (int32_t)((z >> 33) % bc.vocab_size);
            }
            for (int i = 0; i < BT; i++) tgt[i] = tok[(i + 1) % BT];
        }
        auto w0 = std::chrono::steady_clock::now();
        cudaEventRecord(e0, dev.stream());
        Tensor tok_d = Tensor::from_host(core::TensorView{tok.data(), DType::I32, {(std::size_t)BT}}, dev);
        Tensor tgt_d = Tensor::from_host(core::TensorView{tgt.data(), DType::I32, {(std::size_t)BT}}, dev);
        m.zero_grad(dev);
        auto fwd = base::arch::Qwen2Base::forward(b, tok_d, B, T, dev, &m);
        Tensor loss = Tensor::empty_f32({(std::size_t)BT}, dev);
        ops::cross_entropy_fwd(fwd.logits.bf16(), tgt_d.i32(), loss.f32(), fwd.dlogits.bf16(),
                               BT, (int)bc.vocab_size, dev.stream());
        auto lg = base::arch::Qwen2Base::backward(b, fwd, B, T, dev, &m);

        if (do_centroid) {
            for (std::size_t l = 0; l < bc.num_layers; l++) {
                // as shipped: src/trainer/adapt_trainer.cu:210-232 (F32 up-cast, then accumulate)
                Tensor x32 = Tensor::empty_f32(fwd.layer_cache[l].x_normed.shape(), dev);
                ops::cast_bf16_to_f32(fwd.layer_cache[l].x_normed.bf16(), x32.f32(), (int)x32.numel(), dev.stream());
                Tensor g32 = Tensor::empty_f32(lg[l].dx_attn_in.shape(), dev);
                ops::cast_bf16_to_f32(lg[l].dx_attn_in.bf16(), g32.f32(), (int)g32.numel(), dev.stream());
                acc_asbuilt.accumulate(x32, g32, dev);
                if (!bench) {
                    Tensor xt = bf16_payload_in_f32_tensor(fwd.layer_cache[l].x_normed, dev);
                    Tensor gt = bf16_payload_in_f32_tensor(lg[l].dx_attn_in, dev);
                    acc_typed.accumulate(xt, gt, dev);
                }
            }
        }
        dev.sync();
        if (!bench && s == 0) {
            // dumps taken before clipping scales the gradients and before the optimiser touches anything
            dump_tensor(out + "/loss.bin", loss);
            if (geti(c, "dump_logits", 0)) dump_tensor(out + "/logits.bin", fwd.logits);
            if (geti(c, "dump_acts", 0)) {
                dump_tensor(out + "/l0_x_normed.bin", fwd.layer_cache[0].x_normed);
                dump_tensor(out + "/l0_Q.bin", fwd.layer_cache[0].Q);
                dump_tensor(out + "/l0_K.bin", fwd.layer_cache[0].K);
                dump_tensor(out + "/l0_attn_out.bin", fwd.layer_cache[0].attn_out);
                dump_tensor(out + "/x_final.bin", fwd.x_final);
                dump_tensor(out + "/l0_dx_attn_in.bin", lg[0].dx_attn_in);
                dump_tensor(out + "/l0_dQ.bin", lg[0].dQ);
                dump_tensor(out + "/l0_dK.bin", lg[0].dK);
                dump_tensor(out + "/l0_dV.bin", lg[0].dV);
                dump_tensor(out + "/l0_do_proj.bin", lg[0].do_proj);
            }
            for (std::size_t l = 0; l < m.layers.size(); l++)
                for (int i = 0; i < 4; i++) {
                    adapter::LoraPair* lp = pair_of(m.layers[l], i);
                    std::string p = out + "/l" + std::to_string(l) + "_lora_" + PN[i];
                    dump_tensor(p + "_gA.bin", lp->gA); dump_tensor(p + "_gB.bin", lp->gB);
                }
        }
        float norm = grad_norm_and_clip(m, a.grad_clip, dev);
        if (!bench && s == 0) dump(out + "/grad_norm.bin", &norm, 4);
        opt.step_all(m, a.lr, s + 1, dev);
        cudaEventRecord(e1, dev.stream());
        dev.sync();
        float ms; cudaEventElapsedTime(&ms, e0, e1);
        double wall = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - w0).count();
        if (s >= warm) times.push_back(bench ? wall : ms);
        if (!bench) {
            std::string sd = out + "/after_step_" + std::to_string(s);
            fs::create_directories(sd);
            for (std::size_t l = 0; l < m.layers.size(); l++)
                for (int i = 0; i < 4; i++) {
                    adapter::LoraPair* lp = pair_of(m.layers[l], i);
                    std::string p = sd + "/l" + std::to_string(l) + "_lora_" + PN[i];
                    dump_tensor(p + "_A.bin", lp->A_f32); dump_tensor(p + "_B.bin", lp->B_f32);
                }
            if (do_centroid) { acc_asbuilt.write_snapshot(s + 1); acc_typed.write_snapshot(s + 1); }
        }
    }
    if (!bench && geti(c, "write_checkpoint", 0)) {
        checkpoint::AdapterWriter w(out + "/ckpt");
        w.save_checkpoint(m, b, "synthetic/domain", steps, (std::size_t)steps * BT, out + "/ckpt/step-final");
    }
    std::sort(times.begin(), times.end());
    double med = times.empty() ? 0 : times[times.size() / 2];
    std::printf("{\"mode\":\"%s\",\"ms_per_step\":%.4f,\"tokens_per_step\":%d,\"steps\":%d,"
                "\"tokens_per_s\":%.2f,\"B\":%d,\"T\":%d,\"centroid\":%d}\n",
                bench ? "bench" : "step", med, BT, steps, med > 0 ? BT * 1000.0 / med : 0.0, B, T, (int)do_centroid);
    return 0;
}

// ───────────────────────── mode: trainer ─────────────────────────

static int mode_trainer(const std::string& dir, const std::string& out) {
    auto c = read_cfg(dir);
    Device dev = Device::open("cuda:0");
    base::FrozenBase b = make_base(c, dir, dev);
    adapter::AdapterConfig a = make_acfg(c);
    data::Dataset ds = data::Dataset::load(dir + "/train.bin");
    trainer::AdaptOptions o;
    o.domain = "synthetic/domain"; o.output_dir = out; o.checkpoint_every = geti(c, "ckpt_every", 1);
    int steps = (int)geti(c, "steps", 2);
    o.tokens = (std::size_t)steps * a.batch_size * a.seq_len; o.log_to_stdout = false;
    fs::create_directories(out);
    auto t = trainer::AdaptTrainer::create(b, a, ds, o, dev);
    std::ofstream mf(out + "/metrics.txt");
    mf.precision(9);
    while (!t.done()) {
        auto sm = t.step();
        mf << sm.step << " " << sm.tokens_consumed << " " << sm.loss << " " << sm.learning_rate
           << " " << sm.grad_norm << "\n";
    }
    t.save_adapter(out);
    return 0;
}

// ───────────────────────── mode: load ─────────────────────────
// BaseLoader::load on a Hugging Face style directory; dumps the derived config and every tensor
// (BF16 bits) so that the package's loader can be compared with it.

static int mode_load(const std::string& dir, const std::string& out) {
    Device dev = Device::open("cuda:0");
    base::FrozenBase b = base::BaseLoader::load(dir, dev);
    fs::create_directories(out);
    const base::BaseConfig& c = b.config;
    std::ofstream f(out + "/config.txt");
    f.precision(9);
    f << "arch_name " << c.arch_name << "\nbase_sha " << c.base_sha << "\nvocab " << c.vocab_size << "\nhidden "
      << c.hidden_size << "\nlayers " << c.num_layers << "\nhq " << c.num_q_heads << "\nhkv " << c.num_kv_heads
      << "\nhd " << c.head_dim << "\ninter " << c.intermediate_size << "\neps " << c.rms_norm_eps << "\ntheta "
      << c.rope_theta << "\ntie " << (c.tie_embeddings ? 1 : 0) << "\n";
    dump_tensor(out + "/embed.bin", b.embed_w);
    dump_tensor(out + "/final_norm.bin", b.final_norm_w);
    if (!c.tie_embeddings) dump_tensor(out + "/lm_head.bin", b.lm_head_w);
    for (std::size_t l = 0; l < b.layers.size(); l++) {
        const base::LayerWeights& w = b.layers[l];
        const std::string p = out + "/l" + std::to_string(l) + "_";
        dump_tensor(p + "input_norm.bin", w.input_norm_w); dump_tensor(p + "post_norm.bin", w.post_norm_w);
        dump_tensor(p + "q_w.bin", w.q_proj_w); dump_tensor(p + "q_b.bin", w.q_proj_b);
        dump_tensor(p + "k_w.bin", w.k_proj_w); dump_tensor(p + "k_b.bin", w.k_proj_b);
        dump_tensor(p + "v_w.bin", w.v_proj_w); dump_tensor(p + "v_b.bin", w.v_proj_b);
        dump_tensor(p + "o_w.bin", w.o_proj_w); dump_tensor(p + "gate_w.bin", w.gate_proj_w);
        dump_tensor(p + "up_w.bin", w.up_proj_w); dump_tensor(p + "down_w.bin", w.down_proj_w);
    }
    return 0;
}

int main(int argc, char** argv) {
    if (argc < 3) { std::cerr << "usage: ref_harness <op|step|trainer|bench|load> <case_dir> [out_dir]\n"; return 2; }
    std::string mode = argv[1], dir = argv[2], out = argc > 3 ? argv[3] : dir + "/out";
    try {
        if (mode == "op")      return mode_op(dir, out);
        if (mode == "step")    return mode_step(dir, out, false);
        if (mode == "bench")   return mode_step(dir, out, true);
        if (mode == "trainer") return mode_trainer(dir, out);
        if (mode == "load")    return mode_load(dir, out);
    } catch (const std::exception& e) {
        std::cerr << "ref_harness: " << e.what() << "\n";
        return 1;
    }
    std::cerr << "unknown mode " << mode << "\n";
    return 2;
}
