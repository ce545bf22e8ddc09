// tensor::trainer::AdaptTrainer (include/tensor/trainer/adapt_trainer.hpp:48-78, src/trainer/adapt_trainer.cu:96-330)
// on the library's trainer object: same construction, same step (next_batch, assistant-only masking, zero_grad,
// forward, loss, backward, centroid accumulation, clip, AdamW with the cosine schedule), same logging, same
// checkpoint cadence and files - so tools/tensor-adapt.cpp links and runs unchanged.
//
// What differs from the reference, by design:
//   * the frozen base is copied once, device to device, from the caller's FrozenBase into the library's weight
//     arena (the caller keeps ownership of its tensors, as before);
//   * a batch larger than 16384 tokens is processed in micro-batches with gradient accumulation (same result);
//   * the centroid side-channel accumulates the documented sum C = sum_t h_t * ||grad_t|| on the device.  Setting
//     the environment variable TA_SHIM_CENTROID=asbuilt selects instead what the shipped reference computes (its
//     trainer hands accumulate() FP32 copies that are re-read as BF16, adapt_trainer.cu:210-232);
//   * as in the reference, adapters go on q/k/v/o (inject_q..inject_o); inject_up / inject_down are declared by
//     AdapterConfig but wired nowhere in the reference (src/adapter/adapter_model.cu:82-87) and are ignored here
//     too unless TA_SHIM_TARGETS names the projections to adapt (letters of "qkvogud": g = gate, u = up,
//     d = down), which the library supports as an extension;
//   * checkpoints also carry optimizer.safetensors, and AdaptOptions::resume_from, which the reference ignores,
//     resumes from such a checkpoint.
#include <tensor/trainer/adapt_trainer.hpp>

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <filesystem>
#include <iostream>

#include "shim_ctx.hpp"

namespace fs = std::filesystem;

namespace tensor::trainer {

using Clock = std::chrono::steady_clock;
using backend::cuda::Tensor;

struct AdaptTrainer::Impl {
    const base::FrozenBase* base;
    adapter::AdapterConfig cfg;
    data::Dataset* dataset;
    AdaptOptions opts;
    const backend::cuda::Device* dev;
    ta_trainer* tr = nullptr;
    int centroid_mode = 0;           // 0 = documented accumulation, 1 = as the shipped reference computes it
    std::size_t step_count = 0, tokens_seen = 0, total_steps = 0;
    double ema_ms_per_step = 0.0;
    static constexpr double EMA_ALPHA = 0.1;

    Impl(const base::FrozenBase* b, const adapter::AdapterConfig& c, data::Dataset* ds, const AdaptOptions& o,
         const backend::cuda::Device* d)
        : base(b), cfg(c), dataset(ds), opts(o), dev(d) {
        const base::BaseConfig& bc = b->config;
        total_steps = opts.tokens / (cfg.batch_size * cfg.seq_len);
        ta_model_config mc{};
        mc.vocab = int(bc.vocab_size); mc.hidden = int(bc.hidden_size); mc.layers = int(bc.num_layers);
        mc.q_heads = int(bc.num_q_heads); mc.kv_heads = int(bc.num_kv_heads); mc.head_dim = int(bc.head_dim);
        mc.intermediate = int(bc.intermediate_size); mc.rms_eps = bc.rms_norm_eps; mc.rope_theta = bc.rope_theta;
        mc.tie_embeddings = bc.tie_embeddings ? 1 : 0;
        if (const char* e = std::getenv("TA_SHIM_CENTROID")) centroid_mode = std::strcmp(e, "asbuilt") == 0 ? 1 : 0;
        ta_adapter_config ac{};
        ac.rank = cfg.rank; ac.alpha = cfg.alpha;
        ac.targets = (cfg.inject_q ? TA_TARGET_Q : 0) | (cfg.inject_k ? TA_TARGET_K : 0) | (cfg.inject_v ? TA_TARGET_V : 0) |
                     (cfg.inject_o ? TA_TARGET_O : 0);
        if (const char* e = std::getenv("TA_SHIM_TARGETS")) {
            ac.targets = 0;
            for (const char* c = e; *c; c++) {
                const char* at = std::strchr("qkvogud", *c);
                if (at) ac.targets |= 1 << int(at - "qkvogud");
            }
        }
        ac.lr = cfg.lr; ac.grad_clip = cfg.grad_clip; ac.warmup_steps = int(cfg.warmup_steps);
        ac.beta1 = cfg.adam_beta1; ac.beta2 = cfg.adam_beta2; ac.eps = cfg.adam_eps; ac.weight_decay = cfg.weight_decay;
        ac.centroid_modes = 1 << centroid_mode;
        // largest divisor of the batch whose micro-batch stays within 16384 tokens of activations
        int micro = int(cfg.batch_size);
        while (micro > 1 && (std::size_t(micro) * cfg.seq_len > 16384 || cfg.batch_size % std::size_t(micro))) micro--;
        ta_shim::check(ta_trainer_create(ta_shim::ctx(), &mc, &ac, micro, int(cfg.seq_len), ta_shim::as_stream(d->stream()), &tr),
                       "AdaptTrainer::create");
        try {
            upload_base();
            ta_shim::check(ta_trainer_set_meta(tr, bc.arch_name.c_str(), bc.base_sha.c_str()), "AdaptTrainer::create");
            if (!opts.resume_from.empty()) resume();
        } catch (...) {
            ta_trainer_destroy(tr);
            throw;
        }
    }
    ~Impl() { ta_trainer_destroy(tr); }

    void copy_in(const std::string& name, const Tensor& src) {
        void* dst = nullptr; long rows = 0, cols = 0, pitch = 0; int dtype = 0;
        ta_shim::check(ta_trainer_tensor(tr, name.c_str(), &dst, &rows, &cols, &pitch, &dtype), "AdaptTrainer::create");
        if (src.dtype() != core::DType::BF16 || std::size_t(rows * cols) != src.numel() || pitch != cols)
            throw base::BaseError("tensor '" + name + "' of the frozen base has an unexpected dtype or size");
        CUDA_CHECK(cudaMemcpyAsync(dst, src.data(), src.nbytes(), cudaMemcpyDeviceToDevice, dev->stream()));
    }

    void upload_base() {
        const base::FrozenBase& b = *base;
        copy_in("embed", b.embed_w);
        copy_in("final_norm", b.final_norm_w);
        if (!b.config.tie_embeddings) copy_in("lm_head", b.lm_head_w);
        for (std::size_t l = 0; l < b.layers.size(); l++) {
            const base::LayerWeights& w = b.layers[l];
            const std::string p = "l" + std::to_string(l) + ".";
            copy_in(p + "input_norm", w.input_norm_w); copy_in(p + "post_norm", w.post_norm_w);
            copy_in(p + "q_w", w.q_proj_w); copy_in(p + "k_w", w.k_proj_w); copy_in(p + "v_w", w.v_proj_w);
            copy_in(p + "o_w", w.o_proj_w);
            copy_in(p + "q_b", w.q_proj_b); copy_in(p + "k_b", w.k_proj_b); copy_in(p + "v_b", w.v_proj_b);
            copy_in(p + "gate_w", w.gate_proj_w); copy_in(p + "up_w", w.up_proj_w); copy_in(p + "down_w", w.down_proj_w);
        }
        dev->sync();
    }

    void resume() {
        ta_shim::check(ta_trainer_resume(tr, opts.resume_from.c_str()), "AdaptTrainer resume");
        long st = 0, tk = 0;
        ta_shim::check(ta_trainer_counters(tr, &st, &tk), "AdaptTrainer resume");
        step_count = std::size_t(st); tokens_seen = std::size_t(tk);
        // the reference's Dataset has no seek: replay the reads of the steps already taken
        for (std::size_t s = 0; s < step_count; s++) dataset->next_batch(int(cfg.batch_size), int(cfg.seq_len));
        std::cerr << "[trainer] resumed from " << opts.resume_from << " at step " << step_count << "\n";
    }

    std::string snapshot_path(std::size_t step) const {
        const std::string d = opts.output_dir + "/centroids";
        fs::create_directories(d);
        return d + "/step-" + std::to_string(step) + ".centroid";
    }
    void write_snapshot(std::size_t step) {
        const std::string p = snapshot_path(step);
        float w = 0.f;
        ta_shim::check(ta_trainer_write_snapshot(tr, centroid_mode, p.c_str(), nullptr, &w), "write_snapshot");
        if (w != 0.f) std::cerr << "[centroid] snapshot → " << p << " (weight=" << w << ")\n";
    }
    void write_checkpoint(const std::string& dir) {
        fs::create_directories(dir);
        ta_shim::check(ta_trainer_save_checkpoint(tr, dir.c_str(), opts.domain.c_str(), long(step_count), long(tokens_seen), 0),
                       "save_checkpoint");
        ta_shim::check(ta_trainer_save_optimizer(tr, dir.c_str()), "save_checkpoint");
    }

    StepMetrics do_step() {
        const auto t0 = Clock::now();
        const int B = int(cfg.batch_size), T = int(cfg.seq_len), BT = B * T;
        auto [input_ids, target_ids] = dataset->next_batch(B, T);
        ta_mask_targets(input_ids.data(), target_ids.data(), B, T);        // assistant-only targets, adapt_trainer.cu:145-182
        ta_step_metrics m{};
        ta_shim::check(ta_trainer_step(tr, input_ids.data(), target_ids.data(), B, T, -1.f, long(total_steps), 1, &m),
                       "AdaptTrainer::step");
        step_count = std::size_t(m.step);
        tokens_seen = std::size_t(m.tokens_consumed);
        const double ms = std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
        ema_ms_per_step = step_count == 1 ? ms : EMA_ALPHA * ms + (1.0 - EMA_ALPHA) * ema_ms_per_step;
        const double tps = ema_ms_per_step > 0.0 ? BT * 1000.0 / ema_ms_per_step : 0.0;
        if (opts.checkpoint_every && step_count % opts.checkpoint_every == 0) {
            write_snapshot(step_count);
            write_checkpoint(opts.output_dir + "/step-" + std::to_string(step_count));
        }
        return StepMetrics{step_count, tokens_seen, m.loss, m.learning_rate, m.grad_norm, ms, ema_ms_per_step, tps};
    }
};

AdaptTrainer AdaptTrainer::create(const base::FrozenBase& base, const adapter::AdapterConfig& cfg, data::Dataset& dataset,
                                  const AdaptOptions& opts, const backend::cuda::Device& dev) {
    fs::create_directories(opts.output_dir);
    return AdaptTrainer(std::make_unique<Impl>(&base, cfg, &dataset, opts, &dev));
}

AdaptTrainer::AdaptTrainer(std::unique_ptr<Impl> impl) : impl_(std::move(impl)) {}
AdaptTrainer::~AdaptTrainer() = default;
AdaptTrainer::AdaptTrainer(AdaptTrainer&&) noexcept = default;
AdaptTrainer& AdaptTrainer::operator=(AdaptTrainer&&) noexcept = default;

bool AdaptTrainer::done() const { return impl_->tokens_seen >= impl_->opts.tokens; }
StepMetrics AdaptTrainer::step() { return impl_->do_step(); }

void AdaptTrainer::run() {
    while (!done()) {
        const StepMetrics m = step();
        if (impl_->opts.log_to_stdout && impl_->step_count % 10 == 0) {
            std::cerr << "[step " << m.step << "/" << impl_->total_steps << "]"
                      << " loss=" << m.loss << " lr=" << m.learning_rate << " grad=" << m.grad_norm
                      << " tok=" << m.tokens_consumed << " ms=" << static_cast<int>(m.step_ms)
                      << " ema=" << static_cast<int>(m.ema_ms) << " tok/s=" << static_cast<int>(m.tokens_per_sec) << "\n";
        }
    }
    save_adapter(impl_->opts.output_dir);
}

void AdaptTrainer::save_checkpoint(const std::string& dir) {
    impl_->write_snapshot(impl_->step_count);
    impl_->write_checkpoint(dir);
}

void AdaptTrainer::save_adapter(const std::string& dir) {
    impl_->write_snapshot(impl_->step_count);
    fs::create_directories(dir);
    int passes = 0;
    ta_shim::check(ta_trainer_merge_snapshots(impl_->tr, 16, (dir + "/adapter.centroid").c_str(), &passes), "save_adapter");
    ta_shim::check(ta_trainer_save_checkpoint(impl_->tr, dir.c_str(), impl_->opts.domain.c_str(), long(impl_->step_count),
                                              long(impl_->tokens_seen), 1),
                   "save_adapter");
    std::cerr << "[trainer] adapter saved → " << dir << "\n";
}

}  // namespace tensor::trainer
