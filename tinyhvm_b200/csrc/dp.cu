// dp.cu — data-parallel glue: one process and one backend instance per GPU, the
// gradient buffers of a training step summed across the processes with NCCL
// (NVLink / NVSwitch) on the backend's own stream, right behind the backward
// kernels that produced them.
//
// The reference has no multi-device code; its closest relative runs one TinyHVM
// context per thread (src/parallel/reduce.c:36-60), and its backends and
// scheduler keep process-global state (src/backend/cpu/pool.c:6-10,
// src/schedule/_.c:47-59), which is why the unit here is a process.  Training
// steps shard on the batch axis: every rank runs the same program on its slice
// of the batch, calls thvm_cuda_dp_allreduce_sum on the gradient buffers, and
// applies the update with lr / world.
//
// NCCL is opened with dlopen at dp_init, so a single-GPU user needs no NCCL.
#include <dlfcn.h>
#include <string.h>
#include <vector>
#include "state.h"

namespace thc {

typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0 };
enum { ncclFloat32 = 7 };
enum { ncclSum = 0 };

struct Nccl {
    void *lib = nullptr;
    int (*GetUniqueId)(ncclUniqueId *) = nullptr;
    int (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
};
static Nccl nccl;

static bool nccl_load() {
    if (nccl.lib) return true;
    const char *names[] = {getenv("THVM_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        if (!n) continue;
        nccl.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (nccl.lib) break;
    }
    if (!nccl.lib) { set_error("dp: cannot open libnccl (%s)", dlerror()); return false; }
    bool ok = true;
    auto sym = [&](const char *s) { void *p = dlsym(nccl.lib, s); if (!p) { set_error("dp: %s missing from libnccl", s); ok = false; } return p; };
    nccl.GetUniqueId = (int (*)(ncclUniqueId *))sym("ncclGetUniqueId");
    nccl.CommInitRank = (int (*)(ncclComm_t *, int, ncclUniqueId, int))sym("ncclCommInitRank");
    nccl.AllReduce = (int (*)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t))sym("ncclAllReduce");
    nccl.GroupStart = (int (*)())sym("ncclGroupStart");
    nccl.GroupEnd = (int (*)())sym("ncclGroupEnd");
    nccl.CommDestroy = (int (*)(ncclComm_t))sym("ncclCommDestroy");
    nccl.GetErrorString = (const char *(*)(int))sym("ncclGetErrorString");
    return ok;
}

static bool nccl_ok(int rc, const char *what) {
    if (rc == ncclSuccess) return true;
    set_error("dp: %s failed: %s", what, nccl.GetErrorString ? nccl.GetErrorString(rc) : "?");
    return false;
}

}  // namespace thc

using namespace thc;

extern "C" {

// 128-byte rendezvous token; rank 0 creates it and hands it to the other ranks out of band
int thvm_cuda_dp_unique_id(void *out128) {
    if (!nccl_load()) return 1;
    ncclUniqueId id;
    if (!nccl_ok(nccl.GetUniqueId(&id), "ncclGetUniqueId")) return 1;
    memcpy(out128, &id, sizeof id);
    return 0;
}

int thvm_cuda_dp_init(int rank, int world, const void *id128) {
    if (!g.ready) { set_error("dp_init: backend not initialised"); return 1; }
    if (world < 1 || rank < 0 || rank >= world) { set_error("dp_init: rank %d of %d", rank, world); return 1; }
    nccl.rank = rank; nccl.world = world;
    if (world == 1) return 0;
    if (!nccl_load()) return 1;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof id);
    THC_CUDA_OK(cudaSetDevice(g.device));
    if (!nccl_ok(nccl.CommInitRank(&nccl.comm, world, id, rank), "ncclCommInitRank")) return 1;
    return 0;
}

int thvm_cuda_dp_world(void) { return nccl.world; }
int thvm_cuda_dp_rank(void) { return nccl.rank; }

// in-place sum over all ranks of the first `n` floats of each buffer; one NCCL group
// (one bucket) per call, stream-ordered after the kernels that wrote the buffers
int thvm_cuda_dp_allreduce_sum(const uint32_t *buf_ids, const uint64_t *counts, uint32_t n_bufs) {
    // Validate and resolve everything before the group opens: a rank that left the group early would leave the
    // other ranks' collectives without a peer.
    if (n_bufs > 4096) { set_error("dp_allreduce: %u buffers in one call", n_bufs); return 1; }
    std::vector<void *> ptrs(n_bufs);
    for (uint32_t i = 0; i < n_bufs; i++) {
        const uint32_t id = buf_ids[i];
        if (id == 0 || id >= THC_MAX_BUFS || !g.bufs[id].live) { set_error("dp_allreduce: buffer id %u is not live", id); return 1; }
        if (counts[i] * 4 > g.bufs[id].bytes) { set_error("dp_allreduce: %llu floats exceed buffer %u", (unsigned long long)counts[i], id); return 1; }
    }
    if (nccl.world == 1) return 0;
    if (!nccl.comm) { set_error("dp_allreduce: dp_init has not run"); return 1; }
    for (uint32_t i = 0; i < n_bufs; i++) {
        ptrs[i] = buf_checked(buf_ids[i], "dp_allreduce").ptr;
        mark_device_written(buf_ids[i]);
    }
    bool ok = nccl_ok(nccl.GroupStart(), "ncclGroupStart");
    for (uint32_t i = 0; i < n_bufs && ok; i++)
        ok = nccl_ok(nccl.AllReduce(ptrs[i], ptrs[i], (size_t)counts[i], ncclFloat32, ncclSum, nccl.comm, g.stream), "ncclAllReduce");
    ok = nccl_ok(nccl.GroupEnd(), "ncclGroupEnd") && ok;
    return ok ? 0 : 1;
}

void thvm_cuda_dp_shutdown(void) {
    if (nccl.comm) {
        if (g.ready) cudaStreamSynchronize(g.stream);
        nccl.CommDestroy(nccl.comm);
        nccl.comm = nullptr;
    }
    nccl.world = 1; nccl.rank = 0;
}

}  // extern "C"
