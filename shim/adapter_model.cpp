// tensor::adapter::AdapterModel (include/tensor/adapter/adapter_model.hpp:26-95, src/adapter/adapter_model.cu:41-229)
// on the library: the same ten tensors per LoraPair, the same hash-Kaiming start for A and zeros for B, and the
// rank-r forward / backward as ONE library call each instead of the reference's GEMM + cast + add sequences.
//
// The library's rank-r kernels want rank to be a multiple of 16 (one tcgen05 K step); other ranks are refused
// here - the full trainer (adapt_trainer.cpp) pads any rank to 16 internally and has no such limit.
#include <tensor/adapter/adapter_model.hpp>

#include <vector>

#include "shim_ctx.hpp"

namespace tensor::adapter {

using core::DType;

LoraPair AdapterModel::make_pair(int in_dim, int out_dim, int rank, const Device& dev) {
    LoraPair lp;
    lp.in_dim = in_dim; lp.out_dim = out_dim; lp.rank = rank;
    const std::size_t r = rank, in = in_dim, out = out_dim;
    // A = hash-Kaiming values of src/adapter/adapter_model.cu:28-39 (seed 0x1234), FP32 master + its BF16 rounding
    std::vector<float> a(r * in);
    ta_kaiming_init_host(a.data(), in_dim, rank, 0x1234u);
    lp.A_f32 = Tensor::from_host(core::TensorView{a.data(), DType::F32, {r, in}}, dev);
    lp.A_bf16 = Tensor::empty_bf16({r, in}, dev);
    ta_shim::check(ta_cast_f32_to_bf16(ta_shim::ctx(), lp.A_f32.f32(), lp.A_bf16.bf16(), long(r * in), ta_shim::as_stream(dev.stream())),
                   "make_pair");
    lp.B_bf16 = Tensor::zeros({out, r}, DType::BF16, dev);
    lp.B_f32 = Tensor::zeros_f32({out, r}, dev);
    lp.mA = Tensor::zeros_f32({r, in}, dev);  lp.vA = Tensor::zeros_f32({r, in}, dev);
    lp.mB = Tensor::zeros_f32({out, r}, dev); lp.vB = Tensor::zeros_f32({out, r}, dev);
    lp.gA = Tensor::zeros_f32({r, in}, dev);  lp.gB = Tensor::zeros_f32({out, r}, dev);
    return lp;
}

AdapterModel AdapterModel::create(const base::FrozenBase& base, const AdapterConfig& cfg, const Device& dev) {
    AdapterModel m;
    m.cfg_ = cfg;
    const base::BaseConfig& bc = base.config;
    const int H = int(bc.hidden_size), kv = int(bc.num_kv_heads * bc.head_dim);
    m.layers.resize(bc.num_layers);
    for (auto& la : m.layers) {
        la.lora_q = make_pair(H, H, cfg.rank, dev);
        la.lora_k = make_pair(H, kv, cfg.rank, dev);
        la.lora_v = make_pair(H, kv, cfg.rank, dev);
        la.lora_o = make_pair(H, H, cfg.rank, dev);
    }
    return m;
}

// out += scale * (x.A^T).B^T   (src/adapter/adapter_model.cu:96-129)
void AdapterModel::apply_lora_fwd(std::size_t /*layer*/, LoraPair& lp, const Tensor& x, Tensor& out, int BT, const Device& dev) {
    ta_shim::check(ta_lora_linear_fwd(ta_shim::ctx(), x.bf16(), nullptr, nullptr, lp.A_bf16.bf16(), lp.B_bf16.bf16(), out.bf16(),
                                      out.bf16(), BT, lp.in_dim, lp.out_dim, lp.rank, cfg_.scale(), ta_shim::as_stream(dev.stream())),
                   "apply_lora_fwd");
}

// gB += s.dY^T.h, gA += s.dh^T.x, grad_x += s.dh.A   (src/adapter/adapter_model.cu:131-220)
void AdapterModel::apply_lora_bwd(LoraPair& lp, const Tensor& x, const Tensor& grad_out, Tensor& grad_x, int BT, const Device& dev) {
    ta_shim::check(ta_lora_linear_bwd(ta_shim::ctx(), x.bf16(), grad_out.bf16(), nullptr, lp.A_bf16.bf16(), lp.B_bf16.bf16(),
                                      grad_x.bf16(), 1, lp.gA.f32(), lp.gB.f32(), BT, lp.in_dim, lp.out_dim, lp.rank, cfg_.scale(),
                                      ta_shim::as_stream(dev.stream())),
                   "apply_lora_bwd");
}

void AdapterModel::zero_grad(const Device& dev) {
    for (auto& la : layers)
        for (LoraPair* lp : {&la.lora_q, &la.lora_k, &la.lora_v, &la.lora_o}) {
            lp->gA.zero_(dev);
            lp->gB.zero_(dev);
        }
}

std::size_t AdapterModel::param_count() const {
    std::size_t n = 0;
    for (const auto& la : layers)
        for (const LoraPair* lp : {&la.lora_q, &la.lora_k, &la.lora_v, &la.lora_o})
            n += std::size_t(lp->rank) * lp->in_dim + std::size_t(lp->out_dim) * lp->rank;
    return n;
}

}  // namespace tensor::adapter
