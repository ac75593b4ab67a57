// NCCL communicator behind the C ABI: the row exchanges of the multi-GPU build and search run on
// the context's own stream, next to the kernels that produce and consume the rows. The reference
// is a single-GPU program (its mains pin device 1, small_build.cu:33; no NCCL or MPI symbol in
// its tree), so nothing here restates reference code.
//
// libnccl is opened at run time (dlopen) the first time a communicator is asked for: a process
// that never shards needs no NCCL, and a process that already carries one (PyTorch loads its own
// libnccl.so.2) shares that copy instead of loading a second one.
#include <dlfcn.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/glide_b200.h"
#include "ctx.h"

namespace {

// The few NCCL declarations used, restated from NCCL's public header (nccl.h) so that the
// library builds where the header is absent. ncclUniqueId is 128 opaque bytes.
typedef struct ncclComm *ncclComm_t;
struct ncclUniqueIdBytes { char internal[128]; };
enum { kNcclSuccess = 0 };
enum { kNcclInt8 = 0, kNcclUint8 = 1, kNcclInt32 = 2, kNcclUint32 = 3, kNcclInt64 = 4, kNcclUint64 = 5 };
enum { kNcclSum = 0, kNcclProd = 1, kNcclMax = 2, kNcclMin = 3 };

struct NcclApi {
    void *handle = nullptr;
    int (*GetUniqueId)(ncclUniqueIdBytes *) = nullptr;
    int (*CommInitRank)(ncclComm_t *, int, ncclUniqueIdBytes, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*Broadcast)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    std::string load_error;
};

NcclApi g_nccl;
std::once_flag g_nccl_once;

void load_nccl() {
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *name : names) {
        // RTLD_NOLOAD first: reuse the copy the process already carries, if any
        g_nccl.handle = dlopen(name, RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
        if (g_nccl.handle) break;
    }
    for (const char *name : names) {
        if (g_nccl.handle) break;
        g_nccl.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
    }
    if (!g_nccl.handle) {
        g_nccl.load_error = std::string("libnccl.so.2 could not be opened: ") + (dlerror() ? dlerror() : "unknown");
        return;
    }
    bool ok = true;
    auto sym = [&](const char *name) {
        void *p = dlsym(g_nccl.handle, name);
        if (!p) { ok = false; g_nccl.load_error = std::string("libnccl lacks ") + name; }
        return p;
    };
    g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(sym("ncclGetUniqueId"));
    g_nccl.CommInitRank = reinterpret_cast<decltype(g_nccl.CommInitRank)>(sym("ncclCommInitRank"));
    g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(sym("ncclCommDestroy"));
    g_nccl.AllGather = reinterpret_cast<decltype(g_nccl.AllGather)>(sym("ncclAllGather"));
    g_nccl.Broadcast = reinterpret_cast<decltype(g_nccl.Broadcast)>(sym("ncclBroadcast"));
    g_nccl.AllReduce = reinterpret_cast<decltype(g_nccl.AllReduce)>(sym("ncclAllReduce"));
    g_nccl.GroupStart = reinterpret_cast<decltype(g_nccl.GroupStart)>(sym("ncclGroupStart"));
    g_nccl.GroupEnd = reinterpret_cast<decltype(g_nccl.GroupEnd)>(sym("ncclGroupEnd"));
    g_nccl.GetErrorString = reinterpret_cast<decltype(g_nccl.GetErrorString)>(sym("ncclGetErrorString"));
    if (!ok) { dlclose(g_nccl.handle); g_nccl.handle = nullptr; }
}

const NcclApi *nccl() {
    std::call_once(g_nccl_once, load_nccl);
    return g_nccl.handle ? &g_nccl : nullptr;
}

int fail(glide_ctx *ctx, int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx) ctx->error = buf;
    return code;
}

}  // namespace

struct glide_comm_state {
    ncclComm_t comm = nullptr;
    uint32_t world = 1, rank = 0;
};

#define GL_NCCL(ctx, api, call)                                                                       \
    do {                                                                                               \
        int r_ = (call);                                                                               \
        if (r_ != kNcclSuccess)                                                                        \
            return fail(ctx, GLIDE_ERR_NCCL, "%s: %s", #call, (api)->GetErrorString ? (api)->GetErrorString(r_) : "nccl error"); \
    } while (0)

void glide_comm_release(glide_ctx *ctx) {
    if (!ctx || !ctx->comm) return;
    const NcclApi *api = nccl();
    if (api && ctx->comm->comm) api->CommDestroy(ctx->comm->comm);
    delete ctx->comm;
    ctx->comm = nullptr;
}

extern "C" {

int glide_comm_unique_id(uint8_t out[128]) {
    if (!out) return GLIDE_ERR_BAD_ARG;
    const NcclApi *api = nccl();
    if (!api) return GLIDE_ERR_NCCL;
    ncclUniqueIdBytes id;
    if (api->GetUniqueId(&id) != kNcclSuccess) return GLIDE_ERR_NCCL;
    std::memcpy(out, id.internal, 128);
    return GLIDE_OK;
}

int glide_comm_init(glide_ctx *ctx, const uint8_t id[128], uint32_t world, uint32_t rank) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    if (!id || world == 0 || rank >= world) return fail(ctx, GLIDE_ERR_BAD_ARG, "comm_init: bad argument");
    if (ctx->comm) return fail(ctx, GLIDE_ERR_BAD_ARG, "comm_init: the context already has a communicator");
    const NcclApi *api = nccl();
    if (!api) return fail(ctx, GLIDE_ERR_NCCL, "comm_init: %s", g_nccl.load_error.c_str());
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e != cudaSuccess) return fail(ctx, GLIDE_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
    ncclUniqueIdBytes uid;
    std::memcpy(uid.internal, id, 128);
    glide_comm_state *st = new glide_comm_state();
    st->world = world;
    st->rank = rank;
    int r = api->CommInitRank(&st->comm, (int) world, uid, (int) rank);
    if (r != kNcclSuccess) {
        delete st;
        return fail(ctx, GLIDE_ERR_NCCL, "ncclCommInitRank: %s", api->GetErrorString(r));
    }
    ctx->comm = st;
    return GLIDE_OK;
}

int glide_comm_destroy(glide_ctx *ctx) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    glide_comm_release(ctx);
    return GLIDE_OK;
}

uint32_t glide_comm_world(const glide_ctx *ctx) { return (ctx && ctx->comm) ? ctx->comm->world : 1; }
uint32_t glide_comm_rank(const glide_ctx *ctx) { return (ctx && ctx->comm) ? ctx->comm->rank : 0; }

// In-place all-gather of unequal blocks: rank r owns bytes [offsets[r], offsets[r] + counts[r]) of
// d_buf and every rank ends with all of them. One grouped NCCL operation (a broadcast per owner),
// so there is neither padding nor a staging copy. Enqueued on the context's stream; returns
// without waiting.
int glide_comm_all_gather_v(glide_ctx *ctx, void *d_buf, const uint64_t *offsets, const uint64_t *counts) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    if (!ctx->comm) return fail(ctx, GLIDE_ERR_BAD_ARG, "all_gather_v: the context has no communicator");
    if (!d_buf || !offsets || !counts) return fail(ctx, GLIDE_ERR_BAD_ARG, "all_gather_v: null pointer");
    const NcclApi *api = nccl();
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e != cudaSuccess) return fail(ctx, GLIDE_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
    char *base = static_cast<char *>(d_buf);
    GL_NCCL(ctx, api, api->GroupStart());
    for (uint32_t r = 0; r < ctx->comm->world; r++) {
        if (counts[r] == 0) continue;
        int rc = api->Broadcast(base + offsets[r], base + offsets[r], counts[r], kNcclUint8, (int) r, ctx->comm->comm, ctx->stream);
        if (rc != kNcclSuccess) {
            api->GroupEnd();
            return fail(ctx, GLIDE_ERR_NCCL, "ncclBroadcast: %s", api->GetErrorString(rc));
        }
    }
    GL_NCCL(ctx, api, api->GroupEnd());
    return GLIDE_OK;
}

int glide_comm_broadcast(glide_ctx *ctx, void *d_buf, uint64_t bytes, uint32_t root) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    if (!ctx->comm) return fail(ctx, GLIDE_ERR_BAD_ARG, "broadcast: the context has no communicator");
    if (!d_buf || root >= ctx->comm->world) return fail(ctx, GLIDE_ERR_BAD_ARG, "broadcast: bad argument");
    const NcclApi *api = nccl();
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e != cudaSuccess) return fail(ctx, GLIDE_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
    if (bytes == 0) return GLIDE_OK;
    GL_NCCL(ctx, api, api->Broadcast(d_buf, d_buf, bytes, kNcclUint8, (int) root, ctx->comm->comm, ctx->stream));
    return GLIDE_OK;
}

// Element-wise reduction of `count` 64-bit unsigned words over the ranks, in place. op: 0 sum, 1 max, 2 min.
int glide_comm_all_reduce_u64(glide_ctx *ctx, uint64_t *d_buf, uint64_t count, int op) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    if (!ctx->comm) return fail(ctx, GLIDE_ERR_BAD_ARG, "all_reduce: the context has no communicator");
    if (!d_buf || op < 0 || op > 2) return fail(ctx, GLIDE_ERR_BAD_ARG, "all_reduce: bad argument");
    const NcclApi *api = nccl();
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e != cudaSuccess) return fail(ctx, GLIDE_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
    const int nccl_op = op == 0 ? kNcclSum : (op == 1 ? kNcclMax : kNcclMin);
    GL_NCCL(ctx, api, api->AllReduce(d_buf, d_buf, count, kNcclUint64, nccl_op, ctx->comm->comm, ctx->stream));
    return GLIDE_OK;
}

// Waits until everything enqueued on the context's stream, collectives included, is done.
int glide_ctx_synchronize(glide_ctx *ctx) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return fail(ctx, GLIDE_ERR_CUDA, "stream synchronize: %s", cudaGetErrorString(e));
    return GLIDE_OK;
}

}  // extern "C"
