// capture.cu — a whole training step recorded once as a CUDA graph and launched again
// for every later step: the counterpart of the reference's capture / replay of a step's
// GPU command sequence (jit_begin_capture / jit_end_capture / jit_replay,
// src/tinyhvm.h:1294-1300, src/backend/metal/jit.m:24-631), which exists to take the
// host's per-dispatch work out of the training loop.
//
// Between capture_begin and capture_end every vtable call does its host-side work as
// usual (plan lookup, buffer ids, reference counts) but its stream work — kernels,
// zero-fills, stream-ordered allocations and frees, copies, NCCL sums — is recorded
// instead of run.  What differs from an eager step:
//   * host->device writes that are not declared as inputs are constants of the step: placed
//     once in a part of the step arena that is never recycled (or, without an arena, staged
//     in pinned memory the graph owns and copied at every launch);
//   * data that changes from step to step is declared with capture_input: it travels through
//     device staging, uploaded before each launch (graph_set_input) or ahead of it on the
//     copy stream while the previous step runs (graph_prefetch_input);
//   * buf_read of device data records a copy into arena memory and hands back zeros;
//     the values of a launch are fetched afterwards with graph_result;
//   * nothing may wait for the stream, so the step must have run eagerly once before
//     (plans built, scratch grown), and must free every buffer it allocates (a step
//     that ends with pool_reset does): a graph that still owns memory cannot be
//     launched twice.
#include <string.h>
#include <vector>
#include "state.h"

namespace thc {

struct Capture {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    std::vector<uint8_t *> chunks;                 // pinned arena, CHUNK bytes each (large requests get their own)
    uint64_t chunk_pos = 0, chunk_cap = 0;
    // A per-step input reaches its buffer through device staging: the recorded node is a device-to-device copy from one
    // of three staging slots.  graph_set_input uploads into the slot the node reads, on the main stream, before the
    // launch; graph_prefetch_input uploads the NEXT step's bytes into another slot on the copy stream while the current
    // step runs, and the next launch re-points the node to it (three slots: the one being read by the running step, the
    // one the queued step will read, the one being filled).
    struct Input {
        cudaGraphNode_t node; void *dst; uint64_t bytes;
        uint8_t *stage[3]; cudaEvent_t filled[3], read[3]; bool read_valid[3];
        int cur, pending;                          // slot the node reads now; slot a prefetch has filled for the next launch (-1: none)
    };
    struct Result { uint8_t *host; uint64_t bytes; };
    std::vector<Input> inputs;
    std::vector<Result> results;
    uint64_t launches = 0, launches_at_begin = 0;
    uint32_t first_id = 0;
    // Step planner (the counterpart of the slot plan the reference's scheduler makes from liveness, src/schedule/_.c:2017-2112,
    // and of the Metal backend's step planner, src/backend/metal/pool.m:225-378): every buffer the captured step allocates
    // gets an offset in ONE arena instead of a stream-ordered allocation.  The step's alloc / free calls arrive in the
    // order the single stream will run the work, so a block may be handed out again as soon as the step has freed it:
    // a first-fit free list replays the liveness.  The recorded graph then holds no allocation or free nodes at all.
    uint8_t *arena = nullptr;
    uint64_t arena_bytes = 0, arena_high = 0, arena_served = 0;       // size, highest offset used, bytes handed out in total
    uint32_t arena_allocs = 0, pool_allocs = 0;                        // buffers placed in the arena / left to the pool (arena full)
    std::vector<std::pair<uint64_t, uint64_t>> free_list;              // (offset, bytes), sorted by offset
    // Step constants: what the host writes inside the step (scalars, small tables) is the same at every replay.  Instead of
    // one copy node each in the recorded chain, they sit in the top CONST_REGION bytes of the arena, which the free list
    // never sees, and are uploaded once while the step is recorded.  One that the step itself overwrites later (`dirty`)
    // gets a copy node at the end of the graph that puts its bytes back for the next replay.
    struct Const { uint8_t *dev; uint8_t *src; uint64_t bytes; bool dirty; };
    std::vector<Const> consts;
    uint64_t const_pos = 0, const_end = 0;                             // bump range inside the arena
    // host-side state of every buffer that existed when the capture began, put back if the capture is refused
    struct Snap { uint32_t id; void *ptr; uint32_t refcount; bool shadow_valid, zero_pending, plain_alloc; uint8_t shadow[256]; };
    std::vector<Snap> snaps;
    bool failed = false;
    std::string why;
};

static std::vector<Capture *> graphs;              // handle = index + 1
static uint64_t input_sizes[8];                    // capture: host writes of exactly these sizes count as inputs (beside writes above 1 MiB)
static uint32_t n_input_sizes = 0;
constexpr uint64_t ARENA_CHUNK = 4ull << 20;
constexpr uint64_t CONST_REGION = 16ull << 20;

bool capturing() { return g.cap != nullptr; }

void capture_fail(const char *why) {
    if (!g.cap || g.cap->failed) return;
    g.cap->failed = true;
    g.cap->why = why;
}

uint32_t capture_first_id() { return g.cap ? g.cap->first_id : 0; }

void *capture_arena_alloc(uint64_t bytes) {
    if (!g.cap || !g.cap->arena) return nullptr;
    Capture &c = *g.cap;
    const uint64_t need = (bytes + 255) & ~255ull;
    for (size_t i = 0; i < c.free_list.size(); i++) {
        if (c.free_list[i].second < need) continue;
        const uint64_t off = c.free_list[i].first;
        if (c.free_list[i].second == need) c.free_list.erase(c.free_list.begin() + (long)i);
        else { c.free_list[i].first += need; c.free_list[i].second -= need; }
        if (off + need > c.arena_high) c.arena_high = off + need;
        c.arena_served += need; c.arena_allocs++;
        return c.arena + off;
    }
    c.pool_allocs++;
    return nullptr;
}

void capture_arena_give_back(void *ptr, uint64_t bytes) {
    Capture &c = *g.cap;
    const uint64_t off = (uint64_t)((uint8_t *)ptr - c.arena), need = (bytes + 255) & ~255ull;
    size_t i = 0;
    while (i < c.free_list.size() && c.free_list[i].first < off) i++;
    c.free_list.insert(c.free_list.begin() + (long)i, {off, need});
    if (i + 1 < c.free_list.size() && c.free_list[i].first + c.free_list[i].second == c.free_list[i + 1].first) {
        c.free_list[i].second += c.free_list[i + 1].second; c.free_list.erase(c.free_list.begin() + (long)i + 1);
    }
    if (i > 0 && c.free_list[i - 1].first + c.free_list[i - 1].second == c.free_list[i].first) {
        c.free_list[i - 1].second += c.free_list[i].second; c.free_list.erase(c.free_list.begin() + (long)i);
    }
}
void *capture_const_place(const void *host, uint64_t host_bytes, uint64_t buf_bytes) {
    if (!g.cap || !g.cap->arena) return nullptr;
    Capture &c = *g.cap;
    const uint64_t need = (buf_bytes + 255) & ~255ull;
    if (host_bytes > buf_bytes || c.const_pos + need > c.const_end) return nullptr;
    uint8_t *dev = c.arena + c.const_pos;
    c.const_pos += need;
    uint8_t *src = capture_arena_take(need);           // pinned, lives as long as the graph: the upload below and a put-back node read it
    memset(src, 0, need);
    memcpy(src, host, host_bytes);
    THC_CUDA_OK(cudaMemcpyAsync(dev, src, need, cudaMemcpyHostToDevice, g.copy_stream));   // really runs: the copy stream is not recording
    c.consts.push_back({dev, src, need, false});
    c.arena_served += need; c.arena_allocs++;
    return dev;
}

void capture_const_dirty(void *dev) {
    if (!g.cap) return;
    for (Capture::Const &k : g.cap->consts) if (k.dev == dev) { k.dirty = true; return; }
}

bool capture_write_is_input(uint64_t bytes) { for (uint32_t i = 0; i < n_input_sizes; i++) if (input_sizes[i] == bytes) return true; return false; }

uint8_t *capture_arena_take(uint64_t bytes) {
    Capture &c = *g.cap;
    bytes = (bytes + 63) & ~63ull;
    if (c.chunks.empty() || c.chunk_pos + bytes > c.chunk_cap) {
        const uint64_t cap = bytes > ARENA_CHUNK ? bytes : ARENA_CHUNK;
        uint8_t *p = nullptr;
        THC_CUDA_OK(cudaHostAlloc((void **)&p, cap, cudaHostAllocDefault));
        c.chunks.push_back(p);
        c.chunk_pos = 0; c.chunk_cap = cap;
    }
    uint8_t *p = c.chunks.back() + c.chunk_pos;
    c.chunk_pos += bytes;
    return p;
}

// the node the stream's capture ended on (the operation just issued), or null
static cudaGraphNode_t last_captured_node() {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    const cudaGraphNode_t *deps = nullptr;
    size_t n = 0;
    if (cudaStreamGetCaptureInfo(g.stream, &st, nullptr, nullptr, &deps, &n) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return (st == cudaStreamCaptureStatusActive && n == 1) ? deps[0] : nullptr;
}

// host -> device copy recorded as an input of the step
int capture_add_input(void *dst, const void *src, uint64_t bytes) {
    Capture &c = *g.cap;
    Capture::Input in; memset(&in, 0, sizeof in);
    in.dst = dst; in.bytes = bytes; in.cur = 0; in.pending = -1;
    THC_CUDA_OK(cudaMalloc((void **)&in.stage[0], bytes));
    // the bytes given now really travel (copy stream, not recording), so a launch without graph_set_input replays them
    THC_CUDA_OK(cudaMemcpyAsync(in.stage[0], src, bytes, cudaMemcpyHostToDevice, g.copy_stream));
    THC_CUDA_OK(cudaStreamSynchronize(g.copy_stream));     // the caller may free `src` when the call returns
    THC_CUDA_OK(cudaMemcpyAsync(dst, in.stage[0], bytes, cudaMemcpyDeviceToDevice, g.stream));
    in.node = last_captured_node();
    if (!in.node) capture_fail("capture_input: the copy node could not be identified");
    c.inputs.push_back(in);
    return (int)c.inputs.size() - 1;
}

// device -> host read recorded as a result of the step
void capture_add_result(const void *src, uint64_t bytes) {
    Capture &c = *g.cap;
    uint8_t *host = capture_arena_take(bytes);
    THC_CUDA_OK(cudaMemcpyAsync(host, src, bytes, cudaMemcpyDeviceToHost, g.stream));
    c.results.push_back({host, bytes});
}

static void destroy(Capture *c) {
    if (!c) return;
    if (c->exec) cudaGraphExecDestroy(c->exec);
    if (c->graph) cudaGraphDestroy(c->graph);
    for (uint8_t *p : c->chunks) cudaFreeHost(p);
    for (Capture::Input &in : c->inputs)
        for (int k = 0; k < 3; k++) {
            if (in.stage[k]) cudaFree(in.stage[k]);
            if (in.filled[k]) cudaEventDestroy(in.filled[k]);
            if (in.read[k]) cudaEventDestroy(in.read[k]);
        }
    if (c->arena) cudaFree(c->arena);
    delete c;
}

void capture_shutdown() {
    if (g.cap) {
        cudaGraph_t gr = nullptr;
        cudaStreamEndCapture(g.stream, &gr);
        if (gr) cudaGraphDestroy(gr);
        cudaGetLastError();
        destroy(g.cap); g.cap = nullptr;
    }
    for (Capture *c : graphs) destroy(c);
    graphs.clear();
}

static Capture *graph_of(int handle, const char *who) {
    if (handle < 1 || (size_t)handle > graphs.size() || !graphs[handle - 1]) { set_error("%s: no graph %d", who, handle); return nullptr; }
    return graphs[handle - 1];
}

}  // namespace thc

using namespace thc;

extern "C" {

int thvm_cuda_capture_begin(void) {
    if (!g.ready) { set_error("capture_begin: backend not initialised"); return 1; }
    if (g.cap) { set_error("capture_begin: a capture is already running"); return 1; }
    THC_CUDA_OK(cudaStreamSynchronize(g.stream));
    Capture *c = new Capture();
    c->first_id = g.count;
    c->launches_at_begin = g.launches;
    for (uint32_t i = 1; i < c->first_id; i++) {
        const Buf &b = g.bufs[i];
        if (!b.live) continue;
        Capture::Snap sn{i, b.ptr, b.refcount, b.shadow_valid, b.zero_pending, b.plain_alloc, {0}};
        if (b.shadow) memcpy(sn.shadow, b.shadow, sizeof sn.shadow);
        c->snaps.push_back(sn);
    }
    // the arena: what the last finished step held at its peak, plus room for the holes a first-fit replay leaves
    if (g.last_step_peak) {
        c->arena_bytes = (g.last_step_peak + g.last_step_peak / 4 + (64ull << 20)) & ~255ull;     // (the constants' part starts at its end minus a multiple of 256)
        if (cudaMalloc((void **)&c->arena, c->arena_bytes) != cudaSuccess) { cudaGetLastError(); c->arena = nullptr; c->arena_bytes = 0; }
        else {
            c->const_end = c->arena_bytes;
            c->const_pos = c->arena_bytes > 4 * CONST_REGION ? c->arena_bytes - CONST_REGION : c->arena_bytes;
            c->free_list.push_back({0, c->const_pos});
        }
    }
    cudaError_t e = cudaStreamBeginCapture(g.stream, cudaStreamCaptureModeRelaxed);
    if (e != cudaSuccess) { cudaGetLastError(); set_error("capture_begin: %s", cudaGetErrorString(e)); destroy(c); return 1; }
    g.cap = c;
    return 0;
}

int thvm_cuda_capture_input(uint32_t id, const void *host, uint64_t bytes) {
    if (!g.cap) { set_error("capture_input: no capture is running"); return -1; }
    Buf &b = buf_for_output(id, "capture_input", bytes);
    if (bytes > b.bytes || bytes == 0) { set_error("capture_input: %llu bytes into buffer %u of %llu", (unsigned long long)bytes, id, (unsigned long long)b.bytes); return -1; }
    mark_device_written(id);                       // the host shadow no longer speaks for this buffer
    return capture_add_input(b.ptr, host, bytes);
}

int thvm_cuda_capture_end(void) {
    if (!g.cap) { set_error("capture_end: no capture is running"); return 0; }
    Capture *c = g.cap;
    for (uint32_t i = c->first_id; i < THC_MAX_BUFS && !c->failed; i++)
        if (g.bufs[i].live && g.bufs[i].ptr && !g.bufs[i].plain_alloc)     // (a buffer in the step arena counts too: its memory is the graph's)
            capture_fail("a buffer allocated inside the captured step is still live: the step must free what it allocates (end with pool_reset)");
    c->launches = g.launches - c->launches_at_begin;
    for (const Capture::Const &k : c->consts)          // constants the step overwrote: put back at the end of every replay
        if (k.dirty) THC_CUDA_OK(cudaMemcpyAsync(k.dev, k.src, k.bytes, cudaMemcpyHostToDevice, g.stream));
    cudaError_t e = cudaStreamEndCapture(g.stream, &c->graph);
    g.cap = nullptr;
    THC_CUDA_OK(cudaStreamSynchronize(g.copy_stream));     // the constants' uploads have landed before the first launch
    // buffers the step left behind point into memory of a graph that will never run: forget them
    // (no free call: the addresses belong to the graph) and rewind the ids, as if the step had not happened
    // The older buffers go back to the host-side state they had when the capture began: shadows, reference counts and
    // "host copy is current" flags changed by the step's writes and launches, none of which ran.  Device memory that
    // was attached to a host-only buffer meanwhile is released again (its upload came from the shadow being restored).
    auto forget_leftovers = [&]() {
        for (uint32_t i = c->first_id; i < THC_MAX_BUFS; i++)
            if (g.bufs[i].live) { free(g.bufs[i].shadow); g.bufs[i] = Buf(); }
        if (g.count > c->first_id) g.count = c->first_id;
        for (const Capture::Snap &sn : c->snaps) {
            Buf &b = g.bufs[sn.id];
            if (!b.live) continue;                     // the step freed it (already reported as the reason for the refusal)
            if (b.ptr && !sn.ptr) { cudaFree(b.ptr); b.ptr = nullptr; b.plain_alloc = false; }
            b.refcount = sn.refcount; b.shadow_valid = sn.shadow_valid;
            if (sn.ptr) b.zero_pending = b.zero_pending && sn.zero_pending;   // a zero-fill done meanwhile really ran
            else b.zero_pending = false;
            if (b.shadow) memcpy(b.shadow, sn.shadow, sizeof sn.shadow);
        }
    };
    if (e != cudaSuccess || !c->graph) { cudaGetLastError(); set_error("capture_end: %s", cudaGetErrorString(e)); forget_leftovers(); destroy(c); return 0; }
    if (c->failed) { set_error("capture_end: %s", c->why.c_str()); forget_leftovers(); destroy(c); return 0; }
    e = cudaGraphInstantiate(&c->exec, c->graph, 0);
    if (e != cudaSuccess) { cudaGetLastError(); set_error("capture_end: cudaGraphInstantiate: %s", cudaGetErrorString(e)); destroy(c); return 0; }
    graphs.push_back(c);
    return (int)graphs.size();
}

int thvm_cuda_graph_set_input(int graph, int input, const void *host) {
    Capture *c = graph_of(graph, "graph_set_input");
    if (!c) return 1;
    if (input < 0 || (size_t)input >= c->inputs.size() || !host) { set_error("graph_set_input: input %d of %zu", input, c->inputs.size()); return 1; }
    Capture::Input &in = c->inputs[input];
    // stream order puts this upload after every earlier launch (which read the slot) and before the next one
    THC_CUDA_OK(cudaMemcpyAsync(in.stage[in.cur], host, in.bytes, cudaMemcpyHostToDevice, g.stream));
    in.pending = -1;
    return 0;
}

int thvm_cuda_graph_prefetch_input(int graph, int input, const void *host) {
    Capture *c = graph_of(graph, "graph_prefetch_input");
    if (!c) return 1;
    if (input < 0 || (size_t)input >= c->inputs.size() || !host) { set_error("graph_prefetch_input: input %d of %zu", input, c->inputs.size()); return 1; }
    Capture::Input &in = c->inputs[input];
    const int slot = in.pending >= 0 ? in.pending : (in.cur + 1) % 3;
    if (!in.stage[slot]) THC_CUDA_OK(cudaMalloc((void **)&in.stage[slot], in.bytes));
    if (!in.filled[slot]) THC_CUDA_OK(cudaEventCreateWithFlags(&in.filled[slot], cudaEventDisableTiming));
    if (in.read_valid[slot]) THC_CUDA_OK(cudaStreamWaitEvent(g.copy_stream, in.read[slot], 0));    // the launch that last read this slot is done
    THC_CUDA_OK(cudaMemcpyAsync(in.stage[slot], host, in.bytes, cudaMemcpyHostToDevice, g.copy_stream));
    THC_CUDA_OK(cudaEventRecord(in.filled[slot], g.copy_stream));
    in.pending = slot;
    return 0;
}

int thvm_cuda_graph_launch(int graph) {
    Capture *c = graph_of(graph, "graph_launch");
    if (!c) return 1;
    if (g.cap) { set_error("graph_launch: a capture is running"); return 1; }
    for (Capture::Input &in : c->inputs) {
        if (in.pending < 0) continue;
        cudaError_t e = cudaGraphExecMemcpyNodeSetParams1D(c->exec, in.node, in.dst, in.stage[in.pending], in.bytes, cudaMemcpyDeviceToDevice);
        if (e != cudaSuccess) { cudaGetLastError(); set_error("graph_launch: re-pointing an input: %s", cudaGetErrorString(e)); return 1; }
        THC_CUDA_OK(cudaStreamWaitEvent(g.stream, in.filled[in.pending], 0));
        in.cur = in.pending; in.pending = -1;
    }
    cudaError_t e = cudaGraphLaunch(c->exec, g.stream);
    if (e != cudaSuccess) { cudaGetLastError(); set_error("graph_launch: %s", cudaGetErrorString(e)); return 1; }
    for (Capture::Input &in : c->inputs) {
        if (!in.read[in.cur]) THC_CUDA_OK(cudaEventCreateWithFlags(&in.read[in.cur], cudaEventDisableTiming));
        THC_CUDA_OK(cudaEventRecord(in.read[in.cur], g.stream));
        in.read_valid[in.cur] = true;
    }
    g.launches += c->launches;
    return 0;
}

int thvm_cuda_graph_result(int graph, int result, void *out, uint64_t bytes) {
    Capture *c = graph_of(graph, "graph_result");
    if (!c) return 1;
    if (result < 0 || (size_t)result >= c->results.size()) { set_error("graph_result: result %d of %zu", result, c->results.size()); return 1; }
    THC_CUDA_OK(cudaStreamSynchronize(g.stream));
    const Capture::Result &r = c->results[result];
    memcpy(out, r.host, bytes < r.bytes ? bytes : r.bytes);
    if (bytes > r.bytes) memset((uint8_t *)out + r.bytes, 0, bytes - r.bytes);
    return 0;
}

// Result `result` of the latest launch, copied to `out` in stream order (after that launch, before any later one) without
// waiting: the caller reads `out` once the stream has passed this point (an event recorded after the call, or thvm_cuda_sync).
// Lets a training loop fetch step k's loss while step k + 1 is already running.
int thvm_cuda_graph_result_async(int graph, int result, void *out, uint64_t bytes) {
    Capture *c = graph_of(graph, "graph_result_async");
    if (!c) return 1;
    if (result < 0 || (size_t)result >= c->results.size() || !out) { set_error("graph_result_async: result %d of %zu", result, c->results.size()); return 1; }
    const Capture::Result &r = c->results[result];
    THC_CUDA_OK(cudaMemcpyAsync(out, r.host, bytes < r.bytes ? bytes : r.bytes, cudaMemcpyHostToHost, g.stream));
    return 0;
}

// A host that uploads its per-step data with plain buf_write inside the captured step (the reference's drivers create a
// fresh tensor per batch) declares the byte sizes of those uploads: while capturing, every buf_write of exactly one of
// these sizes becomes an input, in call order, as if it had been announced with capture_input; all other staged writes
// stay constants of the step.  n = 0 clears the list.
void thvm_cuda_capture_input_sizes(const uint64_t *sizes, uint32_t n) {
    n_input_sizes = n > 8 ? 8 : n;
    for (uint32_t i = 0; i < n_input_sizes; i++) input_sizes[i] = sizes[i];
}

uint64_t thvm_cuda_graph_input_bytes(int graph, int input) {
    Capture *c = graph_of(graph, "graph_input_bytes");
    if (!c || input < 0 || (size_t)input >= c->inputs.size()) return 0;
    return c->inputs[input].bytes;
}

// memory plan of a captured step: bytes of its arena, highest offset the plan reached, buffers placed in the arena, buffers
// left to stream-ordered allocations inside the graph (arena full or absent), bytes requested over the whole step
int thvm_cuda_graph_memory(int graph, uint64_t *arena_bytes, uint64_t *arena_used, uint32_t *arena_buffers, uint32_t *pool_buffers, uint64_t *bytes_requested) {
    Capture *c = graph_of(graph, "graph_memory");
    if (!c) return 1;
    if (arena_bytes) *arena_bytes = c->arena_bytes;
    if (arena_used) *arena_used = c->arena_high;
    if (arena_buffers) *arena_buffers = c->arena_allocs;
    if (pool_buffers) *pool_buffers = c->pool_allocs;
    if (bytes_requested) *bytes_requested = c->arena_served;
    return 0;
}

int thvm_cuda_graph_counts(int graph, uint32_t *n_inputs, uint32_t *n_results, uint64_t *n_kernels) {
    Capture *c = graph_of(graph, "graph_counts");
    if (!c) return 1;
    if (n_inputs) *n_inputs = (uint32_t)c->inputs.size();
    if (n_results) *n_results = (uint32_t)c->results.size();
    if (n_kernels) *n_kernels = c->launches;
    return 0;
}

int thvm_cuda_graph_nodes(int graph, uint32_t *kernels, uint32_t *copies, uint32_t *memsets, uint32_t *others) {
    Capture *c = graph_of(graph, "graph_nodes");
    if (!c) return 1;
    size_t n = 0;
    if (cudaGraphGetNodes(c->graph, nullptr, &n) != cudaSuccess) { cudaGetLastError(); return 1; }
    std::vector<cudaGraphNode_t> nodes(n);
    if (n && cudaGraphGetNodes(c->graph, nodes.data(), &n) != cudaSuccess) { cudaGetLastError(); return 1; }
    uint32_t k = 0, cp = 0, ms = 0, ot = 0;
    for (size_t i = 0; i < n; i++) {
        cudaGraphNodeType t;
        if (cudaGraphNodeGetType(nodes[i], &t) != cudaSuccess) { cudaGetLastError(); return 1; }
        if (t == cudaGraphNodeTypeKernel) k++;
        else if (t == cudaGraphNodeTypeMemcpy) cp++;
        else if (t == cudaGraphNodeTypeMemset) ms++;
        else ot++;
    }
    if (kernels) *kernels = k;
    if (copies) *copies = cp;
    if (memsets) *memsets = ms;
    if (others) *others = ot;
    return 0;
}

void thvm_cuda_graph_destroy(int graph) {
    if (graph < 1 || (size_t)graph > graphs.size() || !graphs[graph - 1]) return;
    if (g.ready) cudaStreamSynchronize(g.stream);
    destroy(graphs[graph - 1]);
    graphs[graph - 1] = nullptr;
}

}  // extern "C"
