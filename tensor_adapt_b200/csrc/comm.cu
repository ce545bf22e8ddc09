// Data-parallel exchange of the training step at the C level: NCCL all-reduce (sum) of the flat FP32 LoRA gradient
// array and of the (loss sum, loss count) pair, either as one call (ta_allreduce_grads) or - when a communicator is
// attached to the trainer - bucketed per layer and issued on a second stream as each layer's backward finishes, so
// the transfer overlaps the rest of the backward pass over NVLink.
//
// The reference has no multi-GPU code at all; this replaces nothing in it.  NCCL is resolved at run time
// (dlopen of the copy already in the process - the one torch loaded - else libnccl.so.2), so the library
// itself links against the CUDA runtime only and loads on machines without NCCL.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

#include "trainer.h"

namespace ta {
namespace {

struct NcclApi {
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclAllReduce) AllReduce = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
    decltype(&ncclGroupStart) GroupStart = nullptr;
    decltype(&ncclGroupEnd) GroupEnd = nullptr;
    bool ok = false;
};

const NcclApi& nccl() {
    static NcclApi api;
    static bool tried = false;
    if (tried) return api;
    tried = true;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);     // the copy the host process already uses, if any
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return api;
#define TA_SYM(name) api.name = reinterpret_cast<decltype(api.name)>(dlsym(h, "nccl" #name))
    TA_SYM(GetUniqueId); TA_SYM(CommInitRank); TA_SYM(CommDestroy); TA_SYM(AllReduce); TA_SYM(GetErrorString);
    TA_SYM(GroupStart); TA_SYM(GroupEnd);
#undef TA_SYM
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.GetErrorString && api.GroupStart &&
             api.GroupEnd;
    return api;
}

int nccl_fail(ta_ctx* ctx, ncclResult_t r, const char* what) {
    return fail(ctx, TA_ERR_CUDA, std::string(what) + ": NCCL " + (nccl().GetErrorString ? nccl().GetErrorString(r) : "error"));
}

}  // namespace
}  // namespace ta

struct ta_comm {
    ta_ctx* ctx = nullptr;
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    cudaStream_t stream = nullptr;      // the exchange runs here, beside the compute stream
    cudaEvent_t ready = nullptr, done = nullptr;
};

using namespace ta;

extern "C" {

int ta_comm_unique_id(void* out, size_t bytes) {
    if (!out || bytes < sizeof(ncclUniqueId)) return TA_ERR_INVALID;
    if (!nccl().ok) return TA_ERR_UNSUPPORTED;
    ncclUniqueId id;
    if (nccl().GetUniqueId(&id) != ncclSuccess) return TA_ERR_CUDA;
    std::memset(out, 0, bytes);
    std::memcpy(out, &id, sizeof(id));
    return TA_OK;
}

int ta_comm_create(ta_ctx* ctx, int rank, int world, const void* unique_id, size_t bytes, ta_comm** out) {
    if (!ctx || !out || !unique_id || bytes < sizeof(ncclUniqueId) || world < 1 || rank < 0 || rank >= world)
        return fail(ctx, TA_ERR_INVALID, "comm_create: bad argument");
    *out = nullptr;
    if (!nccl().ok) return fail(ctx, TA_ERR_UNSUPPORTED, "comm_create: libnccl.so.2 could not be loaded");
    TA_CUDA(ctx, cudaSetDevice(ctx->device));
    ncclUniqueId id;
    std::memcpy(&id, unique_id, sizeof(id));
    ta_comm* c = new ta_comm();
    c->ctx = ctx; c->rank = rank; c->world = world;
    const ncclResult_t r = nccl().CommInitRank(&c->comm, world, id, rank);
    if (r != ncclSuccess) { delete c; return nccl_fail(ctx, r, "ncclCommInitRank"); }
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ready, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->done, cudaEventDisableTiming) != cudaSuccess) {
        ta_comm_destroy(c);
        return fail(ctx, TA_ERR_CUDA, "comm_create: stream / event creation failed");
    }
    *out = c;
    return TA_OK;
}

int ta_comm_destroy(ta_comm* c) {
    if (!c) return TA_OK;
    if (c->stream) cudaStreamSynchronize(c->stream);
    if (c->comm) nccl().CommDestroy(c->comm);
    if (c->ready) cudaEventDestroy(c->ready);
    if (c->done) cudaEventDestroy(c->done);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
    return TA_OK;
}

int ta_comm_info(const ta_comm* c, int* rank, int* world) {
    if (!c) return TA_ERR_INVALID;
    if (rank) *rank = c->rank;
    if (world) *world = c->world;
    return TA_OK;
}

}  // extern "C"

namespace ta {

// Sum-reduce grad[lo, hi) in place on the communicator's stream once everything issued so far on the compute
// stream (the producers of that slice) has finished.
int comm_reduce_slice(ta_trainer* t, long lo, long hi) {
    ta_comm* c = t->comm;
    if (!c || hi <= lo) return TA_OK;
    TA_CUDA(t->ctx, cudaEventRecord(c->ready, t->stream));
    TA_CUDA(t->ctx, cudaStreamWaitEvent(c->stream, c->ready, 0));
    const ncclResult_t r = nccl().AllReduce(t->grad + lo, t->grad + lo, size_t(hi - lo), ncclFloat, ncclSum, c->comm, c->stream);
    if (r != ncclSuccess) return nccl_fail(t->ctx, r, "ncclAllReduce(lora.grad slice)");
    return TA_OK;
}

// (loss sum, loss count) of the step, then make the compute stream wait for the whole exchange.
int comm_finish_step(ta_trainer* t) {
    ta_comm* c = t->comm;
    if (!c) return TA_OK;
    TA_CUDA(t->ctx, cudaEventRecord(c->ready, t->stream));
    TA_CUDA(t->ctx, cudaStreamWaitEvent(c->stream, c->ready, 0));
    const ncclResult_t r = nccl().AllReduce(t->stats + 2, t->stats + 2, 2, ncclFloat, ncclSum, c->comm, c->stream);
    if (r != ncclSuccess) return nccl_fail(t->ctx, r, "ncclAllReduce(loss sum, count)");
    TA_CUDA(t->ctx, cudaEventRecord(c->done, c->stream));
    TA_CUDA(t->ctx, cudaStreamWaitEvent(t->stream, c->done, 0));
    return TA_OK;
}

}  // namespace ta

extern "C" {

int ta_trainer_set_comm(ta_trainer* t, ta_comm* comm) {
    if (!t) return TA_ERR_INVALID;
    if (comm && comm->ctx != t->ctx) return fail(t->ctx, TA_ERR_INVALID, "trainer_set_comm: communicator belongs to another context");
    t->comm = comm;
    return TA_OK;
}

int ta_allreduce_grads(ta_trainer* t, ta_comm* comm) {
    if (!t || !comm) return TA_ERR_INVALID;
    ta_comm* saved = t->comm;
    t->comm = comm;
    int rc = comm_reduce_slice(t, 0, t->lora_n);
    if (!rc) rc = comm_finish_step(t);
    t->comm = saved;
    return rc;
}

}  // extern "C"
