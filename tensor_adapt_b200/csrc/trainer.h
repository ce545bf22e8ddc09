// Host-side model / adapter / trainer state (internal C++ header).  Mirrors the roles of the
// reference's FrozenBase, AdapterModel, Qwen2Base, AdamW, CentroidAccumulator and AdaptTrainer, but
// with B200-first memory: three device arenas (frozen weights, LoRA parameter arrays, activations)
// allocated once, no per-op cudaMalloc, no device-host round trips inside the step.
#pragma once

#include <string>
#include <vector>

#include "lora.h"

namespace ta {

enum Target { T_Q = 0, T_K, T_V, T_O, T_GATE, T_UP, T_DOWN, T_COUNT };
extern const char* const kTargetNames[T_COUNT];

struct LoraSlot {
    bool on = false;
    int in = 0, out = 0;
    long offA = 0, offB = 0;   // element offsets into the flat LoRA arrays (shared by all five arrays)
    int h_ld = 0;              // row pitch of this projection's h_s / dh_s slice (r, or n*r inside a fused group)
};

struct LayerW {
    __nv_bfloat16 *input_norm, *post_norm, *q_w, *k_w, *v_w, *o_w, *q_b, *k_b, *v_b, *gate_w, *up_w, *down_w;
};

struct LayerCache {
    __nv_bfloat16 *r_in, *x_normed, *Q, *K, *V, *attn_out, *r_mid, *x_normed2, *gate, *up, *act;
    float *in_rms, *post_rms, *lse;
    __nv_bfloat16* h[T_COUNT];   // h_s = bf16(scale * x.A^T) per adapted projection, kept for the backward
};

struct DeviceArena {
    char* base = nullptr;
    size_t size = 0, used = 0;
    void* take(size_t bytes) {
        size_t at = (used + 255) & ~size_t(255);
        used = at + bytes;
        return base ? base + at : nullptr;
    }
};

}  // namespace ta

struct ta_comm;

namespace ta {
// csrc/comm.cu: bucketed gradient exchange on the attached communicator (no-ops without one)
int comm_reduce_slice(ta_trainer* t, long lo, long hi);
int comm_finish_step(ta_trainer* t);
}  // namespace ta

struct ta_trainer {
    ta_ctx* ctx = nullptr;
    cudaStream_t stream = nullptr;
    ta_model_config mc{};
    ta_adapter_config ac{};
    int r_pad = 0;            // rank rounded up to a multiple of 16 (padding rows/columns stay zero)
    float scale = 1.f;        // alpha / rank
    int micro_B = 1, T = 0;   // activation arena is sized for micro_B sequences of T tokens

    ta::DeviceArena weights, lora, acts;
    // frozen base
    __nv_bfloat16 *embed = nullptr, *final_norm = nullptr, *lm_head = nullptr;
    std::vector<ta::LayerW> L;
    // LoRA flat arrays
    long lora_n = 0;
    float *master = nullptr, *m = nullptr, *v = nullptr, *grad = nullptr;
    __nv_bfloat16* working = nullptr;
    std::vector<ta::LoraSlot> slots;   // [layer * T_COUNT + target]
    // activations / temporaries
    std::vector<ta::LayerCache> cache;
    __nv_bfloat16 *r_final = nullptr, *x_final_normed = nullptr, *logits = nullptr;
    float* final_rms = nullptr;
    __nv_bfloat16 *g_res = nullptr, *d_act = nullptr, *d_gate = nullptr, *d_up = nullptr, *d_xn = nullptr,
                  *d_attn = nullptr, *dQ = nullptr, *dK = nullptr, *dV = nullptr;
    __nv_bfloat16* dh[3] = {nullptr, nullptr, nullptr};
    float *delta = nullptr, *splitk = nullptr, *loss = nullptr;
    size_t splitk_bytes = 0;
    bool fuse_qkv = false, fuse_gu = false;   // projections sharing an input share one h / dh / gA pass
    // SwiGLU forward / backward inside the gate-up / down-dX GEMM epilogues.  Off by default: the 256-row tiles use
    // all of tensor memory, so their epilogue is not overlapped and the extra epilogue work costs more than the
    // separate HBM-bound kernels it removes (measured: 3.66 vs 3.27 ms forward, 2.30 vs 2.20 ms backward per layer).
    int fuse_swiglu = -1;           // 1 / 0: SwiGLU inside the GEMM epilogues or as separate kernels; -1: whichever is faster here
    int* tok = nullptr;
    int* tgt = nullptr;
    int logit_rows = 0;       // rows of the lm-head chunk buffer
    // centroid accumulator state + step statistics (device) and their pinned host mirror
    float *cen_acc = nullptr, *cen_w = nullptr, *cen_acc_ab = nullptr, *cen_w_ab = nullptr;
    float *cen_bank = nullptr, *cen_bank_w = nullptr;   // per-layer bank: [layers][hidden] sums and [layers] weights
    float* stats = nullptr;   // [0]=norm [1]=clip scale [2]=loss sum [3]=loss count
    float* h_stats = nullptr;
    // data parallelism: communicator attached with ta_trainer_set_comm, first element of every layer's gradient slice
    ta_comm* comm = nullptr;
    std::vector<long> layer_begin;   // [layers + 1] element offsets into the flat LoRA arrays
    // bookkeeping
    long step_count = 0, tokens_seen = 0;
    long pending_tokens = 0;  // tokens of the optimiser step in progress, added to tokens_seen when it completes
    std::string arch_name = "qwen2", base_sha;
    std::vector<std::vector<float>> snapshots;   // chronological, as CentroidAccumulator keeps them

    ta::LoraSlot& slot(int l, int t) { return slots[size_t(l) * ta::T_COUNT + t]; }
    ta::LoraRef ref(int l, int t) {
        ta::LoraRef r;
        ta::LoraSlot& s = slot(l, t);
        if (!s.on) return r;
        r.A = working + s.offA; r.B = working + s.offB; r.gA = grad + s.offA; r.gB = grad + s.offB; r.r = r_pad;
        return r;
    }
};
