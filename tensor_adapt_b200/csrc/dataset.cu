// Token stream resident in HBM.  data::Dataset (src/data/dataset.cpp:15-71) keeps the tokens in host
// memory and builds every batch with a host loop, the trainer then masks it on the host
// (src/trainer/adapt_trainer.cu:145-182) and uploads two arrays per step.  Here the whole stream is
// uploaded once (4 bytes per token: a billion tokens are 4 GB of 180) and one kernel per step gathers
// the windows, derives the next-token targets and applies the assistant-only mask: the step has no
// host-to-device traffic and no host loop left.
#include <algorithm>
#include <cstdio>
#include <filesystem>
#include <fstream>
#include <string>
#include <vector>

#include "trainer.h"

namespace fs = std::filesystem;

struct ta_dataset {
    ta_ctx* ctx = nullptr;
    int* tokens = nullptr;     // device, total entries
    long total = 0, pos = 0, consumed = 0;
    int *ids = nullptr, *tgt = nullptr;   // device staging for ta_trainer_step_dataset
    long staged = 0;
};

namespace ta {
namespace {

constexpr int IM_START = 151644, ASSISTANT = 77091, IM_END = 151645;
constexpr int kMaskThreads = 256;

// One block per sequence.  The mask is a state machine over the sequence ("inside an assistant turn"),
// restated as a scan: an <|im_start|> at i sets the state to (ids[i+1] == assistant), an <|im_end|>
// clears it; the state of token i is the value of the last such event at or before i.  Each thread
// scans a contiguous chunk, the chunks' last events are combined with a block scan.
__global__ void __launch_bounds__(kMaskThreads) dataset_batch_kernel(const int* __restrict__ tokens, long total, long pos0,
                                                                    int first_seq, int T, int* __restrict__ ids,
                                                                    int* __restrict__ tgt, int mask) {
    __shared__ int s_last[kMaskThreads];
    const int b = blockIdx.x;
    const long start = (pos0 + long(first_seq + b) * T) % total;
    int* my_ids = ids + long(b) * T;
    int* my_tgt = tgt + long(b) * T;
    const int per = (T + kMaskThreads - 1) / kMaskThreads;
    const int t0 = min(int(threadIdx.x) * per, T), t1 = min(t0 + per, T);
    // pass 1: gather + last event of the chunk (-1 none, else 0/1)
    int last = -1;
    for (int t = t0; t < t1; t++) {
        const int tok = tokens[(start + t) % total];
        const int nxt = tokens[(start + t + 1) % total];
        my_ids[t] = tok;
        my_tgt[t] = nxt;
        if (tok == IM_START) last = (t + 1 < T && nxt == ASSISTANT) ? 1 : 0;   // the peek never leaves the sequence
        else if (tok == IM_END) last = 0;
    }
    if (!mask) return;
    s_last[threadIdx.x] = last;
    __syncthreads();
    // state entering the chunk: the nearest earlier chunk that saw an event
    int state = 0;
    for (int j = int(threadIdx.x) - 1; j >= 0; j--)
        if (s_last[j] >= 0) { state = s_last[j]; break; }
    for (int t = t0; t < t1; t++) {
        const int tok = my_ids[t];
        if (tok == IM_START) state = (t + 1 < T && my_tgt[t] == ASSISTANT) ? 1 : 0;
        bool m = !state;
        if (tok == IM_START || tok == ASSISTANT) m = true;
        if (tok == IM_END) { state = 0; m = false; }
        if (m) my_tgt[t] = -1;
    }
}

__global__ void mask_targets_kernel(const int* __restrict__ ids, int* __restrict__ tgt, int T) {
    __shared__ int s_last[kMaskThreads];
    const int* my_ids = ids + long(blockIdx.x) * T;
    int* my_tgt = tgt + long(blockIdx.x) * T;
    const int per = (T + kMaskThreads - 1) / kMaskThreads;
    const int t0 = min(int(threadIdx.x) * per, T), t1 = min(t0 + per, T);
    int last = -1;
    for (int t = t0; t < t1; t++) {
        const int tok = my_ids[t];
        if (tok == IM_START) last = (t + 1 < T && my_ids[t + 1] == ASSISTANT) ? 1 : 0;
        else if (tok == IM_END) last = 0;
    }
    s_last[threadIdx.x] = last;
    __syncthreads();
    int state = 0;
    for (int j = int(threadIdx.x) - 1; j >= 0; j--)
        if (s_last[j] >= 0) { state = s_last[j]; break; }
    for (int t = t0; t < t1; t++) {
        const int tok = my_ids[t];
        if (tok == IM_START) state = (t + 1 < T && my_ids[t + 1] == ASSISTANT) ? 1 : 0;
        bool m = !state;
        if (tok == IM_START || tok == ASSISTANT) m = true;
        if (tok == IM_END) { state = 0; m = false; }
        if (m) my_tgt[t] = -1;
    }
}

}  // namespace
}  // namespace ta

using namespace ta;

extern "C" {

int ta_mask_targets_device(ta_ctx* ctx, const int* input_ids, int* target_ids, int B, int T, void* stream_) {
    if (!ctx || !input_ids || !target_ids || B < 0 || T <= 0) return TA_ERR_INVALID;
    if (B == 0) return TA_OK;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    mask_targets_kernel<<<B, kMaskThreads, 0, stream>>>(input_ids, target_ids, T);
    TA_LAUNCH_CHECK(ctx, "mask_targets_kernel");
    return TA_OK;
}

int ta_dataset_load(ta_ctx* ctx, const char* path, ta_dataset** out) {
    if (!ctx || !path || !out) return TA_ERR_INVALID;
    *out = nullptr;
    fs::path d(path);
    std::error_code ec;
    if (!fs::exists(d, ec)) return fail(ctx, TA_ERR_IO, std::string("path not found: ") + path);
    std::vector<fs::path> files;
    if (fs::is_regular_file(d, ec) && d.extension() == ".bin") {
        files.push_back(d);
    } else if (fs::is_directory(d, ec)) {
        for (const auto& e : fs::directory_iterator(d, ec))
            if (e.is_regular_file() && e.path().extension() == ".bin") files.push_back(e.path());
        std::sort(files.begin(), files.end());
    } else {
        return fail(ctx, TA_ERR_IO, std::string("expected a .bin file or directory of .bin files: ") + path);
    }
    if (files.empty()) return fail(ctx, TA_ERR_IO, std::string("no .bin files in: ") + path);
    long total = 0;
    std::vector<long> counts;
    for (auto& f : files) {
        const long n = long(fs::file_size(f, ec) / 4);   // whole 32-bit tokens, a ragged tail is dropped
        counts.push_back(n);
        total += n;
    }
    if (total == 0) return fail(ctx, TA_ERR_IO, std::string("no tokens in: ") + path);
    ta_dataset* ds = new ta_dataset();
    ds->ctx = ctx;
    ds->total = total;
    if (cudaMalloc(&ds->tokens, size_t(total) * 4) != cudaSuccess) {
        delete ds;
        return fail(ctx, TA_ERR_NOMEM, "cannot allocate the token stream on the device");
    }
    std::vector<char> buf(size_t(64) << 20);
    long at = 0;
    for (size_t i = 0; i < files.size(); i++) {
        std::ifstream f(files[i], std::ios::binary);
        if (!f) { cudaFree(ds->tokens); delete ds; return fail(ctx, TA_ERR_IO, "cannot open: " + files[i].string()); }
        long left = counts[i] * 4;
        while (left > 0) {
            const long n = std::min<long>(left, long(buf.size()));
            f.read(buf.data(), n);
            if (f.gcount() != n) { cudaFree(ds->tokens); delete ds; return fail(ctx, TA_ERR_IO, "short read: " + files[i].string()); }
            if (cudaMemcpy(reinterpret_cast<char*>(ds->tokens) + at, buf.data(), size_t(n), cudaMemcpyHostToDevice) != cudaSuccess) {
                cudaFree(ds->tokens); delete ds;
                return fail(ctx, TA_ERR_CUDA, "upload of the token stream failed");
            }
            at += n;
            left -= n;
        }
    }
    *out = ds;
    return TA_OK;
}

int ta_dataset_destroy(ta_dataset* ds) {
    if (!ds) return TA_OK;
    cudaFree(ds->tokens); cudaFree(ds->ids); cudaFree(ds->tgt);
    delete ds;
    return TA_OK;
}

int ta_dataset_info(const ta_dataset* ds, long* total_tokens, long* position, long* tokens_consumed) {
    if (!ds) return TA_ERR_INVALID;
    if (total_tokens) *total_tokens = ds->total;
    if (position) *position = ds->pos;
    if (tokens_consumed) *tokens_consumed = ds->consumed;
    return TA_OK;
}

int ta_dataset_seek(ta_dataset* ds, long position, long tokens_consumed) {
    if (!ds || position < 0) return TA_ERR_INVALID;
    ds->pos = position % ds->total;
    ds->consumed = tokens_consumed;
    return TA_OK;
}

int ta_dataset_next_batch(ta_dataset* ds, int B, int T, int first_seq, int n_seq, int* ids_dev, int* targets_dev, int mask,
                          void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!ds || B <= 0 || T <= 0 || first_seq < 0 || n_seq < 0 || first_seq + n_seq > B || (n_seq && (!ids_dev || !targets_dev)))
        return TA_ERR_INVALID;
    if (n_seq) {
        dataset_batch_kernel<<<n_seq, kMaskThreads, 0, stream>>>(ds->tokens, ds->total, ds->pos, first_seq, T, ids_dev, targets_dev, mask);
        TA_LAUNCH_CHECK(ds->ctx, "dataset_batch_kernel");
    }
    ds->pos = (ds->pos + long(B) * T) % ds->total;
    ds->consumed += long(B) * T;
    return TA_OK;
}

int ta_trainer_step_dataset(ta_trainer* t, ta_dataset* ds, int B, int mask, float lr, long total_steps, ta_step_metrics* out) {
    if (!t || !ds || B <= 0) return TA_ERR_INVALID;
    const long need = long(B) * t->T;
    if (ds->staged < need) {
        cudaFree(ds->ids); cudaFree(ds->tgt);
        ds->ids = ds->tgt = nullptr;
        ds->staged = 0;
        TA_CUDA(t->ctx, cudaMalloc(&ds->ids, size_t(need) * 4));
        TA_CUDA(t->ctx, cudaMalloc(&ds->tgt, size_t(need) * 4));
        ds->staged = need;
    }
    if (int rc = ta_dataset_next_batch(ds, B, t->T, 0, B, ds->ids, ds->tgt, mask, t->stream)) return rc;
    return ta_trainer_step(t, ds->ids, ds->tgt, B, t->T, lr, total_steps, 0, out);
}

}  // extern "C"
