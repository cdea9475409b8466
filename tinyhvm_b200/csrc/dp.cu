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
#include <initializer_list>
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


// ------------------------------------------------------------------ fused gradient sum + SGD update
// The optimizer step of a data-parallel training step as one call: the gradients of all parameter tensors are summed
// over the ranks and the update p <- p - lr * sum is applied, instead of one collective and one `a - b*c` dispatch plus
// a copy per parameter tensor (the reference's one-kernel optimizer is Backend.adam_step, src/nn/adam.c:103-118,
// arithmetic src/shaders.metal:406-420; this is its SGD counterpart with the collective folded in).
//
// Every rank owns an exchange arena (cudaMalloc, shared with the other rank processes through cudaIpc handles):
//     int   flags[64]            flags[r] = number of the last step whose gradients rank r has published (written BY rank r)
//     float slot[2][capacity]    this rank's packed gradients, two slots used in turn
// Small buckets (<= DP_ONESHOT_BYTES) take the one-shot path, two launches:
//   k_dp_pack    copies the gradient tensors into slot[step & 1]; the last CTA to finish publishes the step number in
//                every peer's flags[me] (plain stores to peer memory, behind a system-scope fence);
//   k_dp_reduce  one thread per CTA waits until flags[r] has reached the step for every r — a bounded wait: after
//                the poll limit it raises status bit 16 and the kernel returns without touching the parameters — then
//                all threads add the ranks' slots in rank order (plain loads from peer memory, not cached in L1) and
//                update the parameters in place.  Every rank adds in the same order, so all ranks hold bit-identical
//                parameters.
// A rank overwrites slot s again two steps later; by then it has seen every peer's flag of the step in between, which a
// peer publishes only after its own reduce of the earlier step has finished (stream order), so nobody still reads the slot.
// Large buckets: pack, ONE ncclAllReduce over the packed slot, update from the slot.  No multicast, no NVLS needed.
constexpr int DP_MAX_TENSORS = 64;
constexpr int DP_MAX_WORLD = 16;
constexpr uint64_t DP_ONESHOT_BYTES = 1ull << 20;
enum : int { ERR_DP_TIMEOUT = 16 };

struct DpTensors {
    float *param[DP_MAX_TENSORS];
    const float *grad[DP_MAX_TENSORS];
    unsigned long long start[DP_MAX_TENSORS + 1];     // prefix sums of the element counts
    unsigned n;
};
struct DpPeers {
    const float *slots[DP_MAX_WORLD];                 // rank r's two slots, `capacity` floats each (own memory for r == rank)
    int *flags[DP_MAX_WORLD];                         // rank r's flag array
    unsigned long long capacity;
    int world, rank;
};

__device__ __forceinline__ unsigned dp_find(const DpTensors &T, unsigned long long e) {
    unsigned lo = 0, hi = T.n;                        // the tensor holding flat element e
    while (hi - lo > 1) { const unsigned mid = (lo + hi) >> 1; if (T.start[mid] <= e) lo = mid; else hi = mid; }
    return lo;
}

// The slot is chosen on the device from the step counter (step s uses slot s & 1), not by the host: a step recorded
// once as a CUDA graph is launched again with the same arguments for every later step.
__global__ void __launch_bounds__(256) k_dp_pack(const __grid_constant__ DpTensors T, float *__restrict__ slots, const __grid_constant__ DpPeers P,
                                                 int *step_counter, unsigned *ticket, int publish) {
    const unsigned long long total = T.start[T.n];
    // (the counter moves only when the last CTA of this launch is done, after every CTA has read it here)
    float *slot = slots + (publish ? (unsigned long long)((*((volatile int *)step_counter) + 1) & 1) * P.capacity : 0ull);
    for (unsigned long long e = (unsigned long long)blockIdx.x * 256 + threadIdx.x; e < total; e += (unsigned long long)gridDim.x * 256) {
        const unsigned i = dp_find(T, e);
        slot[e] = T.grad[i][e - T.start[i]];
    }
    if (!publish) return;
    __threadfence_system();                            // this CTA's part of the slot is visible to the peers
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned done = atomicAdd(ticket, 1u) + 1u;
        if (done == gridDim.x) {                       // last CTA: the whole slot is out
            *ticket = 0;
            const int step = *step_counter + 1;
            *step_counter = step;
            __threadfence_system();
            for (int r = 0; r < P.world; r++) *((volatile int *)&P.flags[r][P.rank]) = step;
        }
    }
}

// poll_limit: iterations of the flag wait (each a few hundred ns) before giving up
__global__ void __launch_bounds__(256) k_dp_reduce(const __grid_constant__ DpTensors T, const __grid_constant__ DpPeers P, const float *__restrict__ lr_ptr,
                                                   const int *step_counter, unsigned long long poll_limit, int *status) {
    __shared__ int go;
    if (threadIdx.x == 0) {
        const int step = *((volatile const int *)step_counter);
        const volatile int *mine = P.flags[P.rank];
        int ok = 1;
        for (int r = 0; r < P.world && ok; r++) {
            unsigned long long polls = 0;
            while (mine[r] - step < 0) {               // rank r has not published this step yet
                if (++polls > poll_limit) { ok = 0; break; }
                __nanosleep(100);
            }
        }
        if (!ok) atomicOr(status, ERR_DP_TIMEOUT);
        __threadfence_system();
        go = ok;
    }
    __syncthreads();
    if (!go) return;                                   // a peer never arrived: leave the parameters as they are
    const float lr = lr_ptr[0];
    const unsigned long long total = T.start[T.n];
    const unsigned long long so = (unsigned long long)(*step_counter & 1) * P.capacity;
    for (unsigned long long e = (unsigned long long)blockIdx.x * 256 + threadIdx.x; e < total; e += (unsigned long long)gridDim.x * 256) {
        float sum = __ldcv(P.slots[0] + so + e);
        for (int r = 1; r < P.world; r++) sum = __fadd_rn(sum, __ldcv(P.slots[r] + so + e));
        const unsigned i = dp_find(T, e);
        float *p = T.param[i] + (e - T.start[i]);
        *p = __fsub_rn(*p, __fmul_rn(sum, lr));
    }
}

// update from one gradient source: the local gradient tensors (src == nullptr) or a packed slot
__global__ void __launch_bounds__(256) k_dp_update(const __grid_constant__ DpTensors T, const float *__restrict__ src, const float *__restrict__ lr_ptr) {
    const float lr = lr_ptr[0];
    const unsigned long long total = T.start[T.n];
    for (unsigned long long e = (unsigned long long)blockIdx.x * 256 + threadIdx.x; e < total; e += (unsigned long long)gridDim.x * 256) {
        const unsigned i = dp_find(T, e);
        const unsigned long long o = e - T.start[i];
        const float gsum = src ? src[e] : T.grad[i][o];
        T.param[i][o] = __fsub_rn(T.param[i][o], __fmul_rn(gsum, lr));
    }
}

struct DpArena {
    uint8_t *base = nullptr;                          // own arena
    uint64_t capacity = 0;                            // floats per slot
    uint8_t *peer[DP_MAX_WORLD] = {nullptr};          // mapped arenas (peer[rank] == base)
    bool attached[DP_MAX_WORLD] = {false};
    int *step_counter = nullptr;                      // device: steps published so far
    unsigned *ticket = nullptr;
    unsigned long long poll_limit = 20000000ull;      // ~2 s of 100 ns naps
};
static DpArena arena;
static constexpr uint64_t DP_FLAG_BYTES = 256;       // 64 ints

static float *arena_slot(uint8_t *base, uint64_t capacity, unsigned which) { return (float *)(base + DP_FLAG_BYTES) + (uint64_t)which * capacity; }

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

// ---- exchange arena (see the comment at k_dp_pack) ----
int thvm_cuda_dp_arena_create(uint64_t max_floats, void *out_handle64) {
    if (!g.ready) { set_error("dp_arena_create: backend not initialised"); return 1; }
    if (arena.base) { set_error("dp_arena_create: the arena exists already"); return 1; }
    if (max_floats == 0 || max_floats > (1ull << 30)) { set_error("dp_arena_create: %llu floats", (unsigned long long)max_floats); return 1; }
    const uint64_t cap = (max_floats + 63) & ~63ull, bytes = DP_FLAG_BYTES + 2 * cap * 4 + 64;
    THC_CUDA_OK(cudaMalloc((void **)&arena.base, bytes));
    THC_CUDA_OK(cudaMemset(arena.base, 0, bytes));
    arena.capacity = cap;
    arena.step_counter = (int *)(arena.base + DP_FLAG_BYTES + 2 * cap * 4);
    arena.ticket = (unsigned *)(arena.step_counter + 1);
    for (int r = 0; r < DP_MAX_WORLD; r++) { arena.peer[r] = nullptr; arena.attached[r] = false; }
    arena.peer[nccl.rank] = arena.base; arena.attached[nccl.rank] = true;
    if (out_handle64) {
        cudaIpcMemHandle_t h;
        cudaError_t e = cudaIpcGetMemHandle(&h, arena.base);
        if (e != cudaSuccess) { cudaGetLastError(); set_error("dp_arena_create: cudaIpcGetMemHandle: %s", cudaGetErrorString(e)); return 1; }
        static_assert(sizeof h == 64, "ipc handle size");
        memcpy(out_handle64, &h, 64);
    }
    return 0;
}

// map rank `peer_rank`'s arena (a handle made by its dp_arena_create) into this process
int thvm_cuda_dp_arena_attach(int peer_rank, const void *handle64) {
    if (!arena.base) { set_error("dp_arena_attach: create the local arena first"); return 1; }
    if (peer_rank < 0 || peer_rank >= DP_MAX_WORLD || peer_rank >= nccl.world) { set_error("dp_arena_attach: rank %d of %d", peer_rank, nccl.world); return 1; }
    if (peer_rank == nccl.rank) return 0;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { cudaGetLastError(); set_error("dp_arena_attach: cudaIpcOpenMemHandle(rank %d): %s", peer_rank, cudaGetErrorString(e)); return 1; }
    arena.peer[peer_rank] = (uint8_t *)p; arena.attached[peer_rank] = true;
    return 0;
}

// tests: stand-in for a peer that never shows up — the local arena plays rank `peer_rank` too, and nothing ever
// publishes a step for it
int thvm_cuda_dp_arena_attach_silent(int peer_rank) {
    if (!arena.base || peer_rank < 0 || peer_rank >= DP_MAX_WORLD) { set_error("dp_arena_attach_silent: bad rank or no arena"); return 1; }
    arena.peer[peer_rank] = arena.base; arena.attached[peer_rank] = true;
    if (peer_rank >= nccl.world) nccl.world = peer_rank + 1;
    return 0;
}
void thvm_cuda_dp_set_poll_limit(uint64_t polls) { arena.poll_limit = polls ? polls : 20000000ull; }

// p_i <- p_i - lr * (sum over ranks of g_i) for every listed parameter tensor; `lr_buf` holds the step size (one float)
int thvm_cuda_dp_sgd_step(const uint32_t *param_ids, const uint32_t *grad_ids, const uint64_t *counts, uint32_t n, uint32_t lr_buf) {
    if (!g.ready) { set_error("dp_sgd_step: backend not initialised"); return 1; }
    if (n == 0 || n > DP_MAX_TENSORS) { set_error("dp_sgd_step: %u tensors (1..%d)", n, DP_MAX_TENSORS); return 1; }
    // validate everything before anything is launched: a rank that bailed out half-way would leave its peers waiting
    for (uint32_t i = 0; i < n; i++) {
        for (const uint32_t id : {param_ids[i], grad_ids[i]})
            if (id == 0 || id >= THC_MAX_BUFS || !g.bufs[id].live || counts[i] * 4 > g.bufs[id].bytes) {
                set_error("dp_sgd_step: tensor %u: buffer %u is not live or shorter than %llu floats", i, id, (unsigned long long)counts[i]);
                return 1;
            }
    }
    if (lr_buf == 0 || lr_buf >= THC_MAX_BUFS || !g.bufs[lr_buf].live || g.bufs[lr_buf].bytes < 4) { set_error("dp_sgd_step: no step-size buffer"); return 1; }
    DpTensors T; memset(&T, 0, sizeof T);
    T.n = n;
    for (uint32_t i = 0; i < n; i++) {
        T.grad[i] = (const float *)buf_checked(grad_ids[i], "dp_sgd_step(grad)").ptr;
        T.param[i] = (float *)buf_checked(param_ids[i], "dp_sgd_step(param)").ptr;
        mark_device_written(param_ids[i]);
        T.start[i + 1] = T.start[i] + counts[i];
    }
    const float *lr = (const float *)buf_checked(lr_buf, "dp_sgd_step(lr)").ptr;
    const uint64_t total = T.start[n];
    const unsigned grid = grid_for(total, 256 * 4, 4);
    if (nccl.world == 1) {
        profile_begin();
        k_dp_update<<<grid, 256, 0, g.stream>>>(T, nullptr, lr);
        after_launch("sgd_update");
        return 0;
    }
    if (!arena.base || total > arena.capacity) { set_error("dp_sgd_step: %llu floats do not fit the exchange arena (%llu)", (unsigned long long)total, (unsigned long long)arena.capacity); return 1; }
    float *slot = arena_slot(arena.base, arena.capacity, 0);
    DpPeers P; memset(&P, 0, sizeof P);
    P.world = nccl.world; P.rank = nccl.rank; P.capacity = arena.capacity;
    bool all_attached = true;
    for (int r = 0; r < nccl.world; r++) {
        if (!arena.attached[r]) { all_attached = false; continue; }
        P.slots[r] = arena_slot(arena.peer[r], arena.capacity, 0);
        P.flags[r] = (int *)arena.peer[r];
    }
    const bool oneshot = all_attached && total * 4 <= DP_ONESHOT_BYTES;
    profile_begin();
    k_dp_pack<<<grid, 256, 0, g.stream>>>(T, slot, P, arena.step_counter, arena.ticket, oneshot ? 1 : 0);
    after_launch("dp_pack");
    if (oneshot) {
        profile_begin();
        k_dp_reduce<<<grid, 256, 0, g.stream>>>(T, P, lr, arena.step_counter, arena.poll_limit, g.dev_status);
        after_launch("dp_reduce_sgd");
        return 0;
    }
    if (!nccl.comm) { set_error("dp_sgd_step: dp_init has not run"); return 1; }
    if (!nccl_ok(nccl.AllReduce(slot, slot, (size_t)total, ncclFloat32, ncclSum, nccl.comm, g.stream), "ncclAllReduce")) return 1;
    g.launches++;
    profile_begin();
    k_dp_update<<<grid, 256, 0, g.stream>>>(T, slot, lr);
    after_launch("sgd_update");
    return 0;
}

static void dp_arena_release(void) {
    for (int r = 0; r < DP_MAX_WORLD; r++)
        if (arena.attached[r] && arena.peer[r] && arena.peer[r] != arena.base) cudaIpcCloseMemHandle(arena.peer[r]);
    if (arena.base) cudaFree(arena.base);
    arena = DpArena();
}

void thvm_cuda_dp_shutdown(void) {
    if (g.ready) cudaStreamSynchronize(g.stream);
    dp_arena_release();
    if (nccl.comm) {
        if (g.ready) cudaStreamSynchronize(g.stream);
        nccl.CommDestroy(nccl.comm);
        nccl.comm = nullptr;
    }
    nccl.world = 1; nccl.rank = 0;
}

}  // extern "C"
