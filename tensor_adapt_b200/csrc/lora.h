// LoRA-augmented linear layer on the segmented-K GEMM (internal C++ interface).
#pragma once
#include "seg_gemm.h"

namespace ta {

struct LoraRef {
    const __nv_bfloat16* A = nullptr;   // [r][in]  BF16 working copy
    const __nv_bfloat16* B = nullptr;   // [out][r]
    float* gA = nullptr;                // [r][in]  FP32 gradient accumulators
    float* gB = nullptr;                // [out][r]
    int r = 0;
    bool on() const { return A != nullptr && r > 0; }
};

// h_s[BT][r] = bf16(scale * x.A^T)
int lora_down(ta_ctx* ctx, cudaStream_t s, const __nv_bfloat16* x, int BT, int in, const LoraRef& l, float scale,
              __nv_bfloat16* h_s);

// bytes of scratch lora_linear_fwd / lora_linear_bwd need for one projection
size_t lora_fwd_scratch_bytes(int BT, int r);
size_t lora_bwd_scratch_bytes(const ta_ctx* ctx, int BT, int in, int out, int r);

}  // namespace ta
