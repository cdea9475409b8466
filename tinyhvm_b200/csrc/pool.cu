// pool.cu — lifecycle, the device buffer pool behind the reference's integer
// buffer ids, and host<->device transfers.
//
// Contract followed (reference: src/tinyhvm.h:990-1001,1030-1031,1038-1039):
//   * ids are handed out in increasing order starting at 1; 0 means failure;
//     pool_reset(keep) frees ids > keep and rewinds the counter to keep+1
//     (src/backend/cpu/pool.c:14,19-26) — the scheduler indexes per-buffer
//     epochs by id (src/schedule/_.c:55), so the numbering must match;
//   * a fresh buffer reads as zero (the CPU backend callocs);
//   * buf_write may return before the DMA ran only if the source was staged,
//     because callers free the source right away (src/nn/loss.c:31-34);
//   * buf_read returns finished data, so it drains the stream
//     (src/ops/_.c:317-319 reads the result immediately);
//   * decref frees at zero unless the id is at or below the persistent floor
//     (Metal pool: src/backend/metal/pool.m:144-152).
// Memory comes from the device's stream-ordered pool (cudaMallocAsync) with the
// release threshold lifted, so a training step recycles its buffers without
// going back to the driver.  Buffers of <= 256 bytes (the reference turns every
// shape / axes / scalar constant into such a buffer, hundreds per training step)
// start out as a host shadow only: no allocation, no copy, and reading them back
// never waits for the GPU.  Device memory is attached, and the shadow uploaded,
// the first time a kernel or a device copy actually touches the buffer.
#include <stdarg.h>
#include <string.h>
#include <map>
#include "state.h"

namespace thc {

State g;

static const uint64_t RING_BYTES   = 16ull << 20;   // two 8 MiB halves
static const uint64_t RING_MAX_MSG = 1ull << 20;    // larger writes go direct

void set_error(const char *fmt, ...) {
    char tmp[512];
    va_list ap; va_start(ap, fmt); vsnprintf(tmp, sizeof tmp, fmt, ap); va_end(ap);
    if (g.last_error.empty()) g.last_error = tmp;      // sticky: keep the first
    fprintf(stderr, "thvm_cuda: %s\n", tmp);
}
void fatal(const char *fmt, ...) {
    char tmp[512];
    va_list ap; va_start(ap, fmt); vsnprintf(tmp, sizeof tmp, fmt, ap); va_end(ap);
    fprintf(stderr, "thvm_cuda: FATAL: %s\n", tmp);
    exit(1);   // the reference's backends exit on unrecoverable errors too (src/backend/metal/pool.m:49-53)
}

Buf &buf_live(uint32_t id, const char *who) {
    if (!g.ready) fatal("%s: backend not initialised (no CUDA device?)", who);
    if (id == 0 || id >= THC_MAX_BUFS || !g.bufs[id].live)
        fatal("%s: buffer id %u is not live", who, id);
    return g.bufs[id];
}

static uint8_t *ring_take(uint64_t bytes);
void fence_copy(Buf &b);
static const uint64_t SHADOW_MAX   = 256;

// A buffer that existed before a capture began outlives the recorded step, so what it needs to become usable — device
// memory, the upload of its host shadow, the zero-fill a fresh buffer owes — must really happen, not merely be recorded:
// it is done at once on the copy stream (which is not recording) and waited for.  The recorded step then finds the
// buffer in the state an eager step would, whether or not the capture ends up being used.
static void settle_outside_capture(Buf &b, bool attach) {
    const uint64_t sz = ((b.bytes + 15) & ~15ull) ? ((b.bytes + 15) & ~15ull) : 16;
    if (attach) {
        THC_CUDA_OK(cudaMalloc(&b.ptr, sz));
        b.plain_alloc = true;
        if (b.shadow && b.shadow_valid && b.bytes) {
            uint8_t tmp[SHADOW_MAX + 16] = {0};
            memcpy(tmp, b.shadow, b.bytes);
            THC_CUDA_OK(cudaMemcpyAsync(b.ptr, tmp, sz, cudaMemcpyHostToDevice, g.copy_stream));
        } else {
            THC_CUDA_OK(cudaMemsetAsync(b.ptr, 0, sz, g.copy_stream));
        }
    } else {
        THC_CUDA_OK(cudaMemsetAsync(b.ptr, 0, sz, g.copy_stream));
    }
    THC_CUDA_OK(cudaStreamSynchronize(g.copy_stream));
    b.zero_pending = false;
}

// `will_overwrite`: the caller is about to overwrite the whole buffer, so memory that is attached here needs no contents.
static Buf &buf_attach(uint32_t id, const char *who, bool will_overwrite) {
    Buf &b = buf_live(id, who);
    fence_copy(b);                                  // whatever comes next on the main stream stays behind a running read-back of b
    const bool outlives_capture = g.cap && id < capture_first_id();
    if (!b.ptr) {                                   // host-only so far: attach device memory now
        if (outlives_capture) { settle_outside_capture(b, true); return b; }
        uint64_t sz = (b.bytes + 15) & ~15ull;
        if (sz == 0) sz = 16;
        const bool have_data = b.shadow && b.shadow_valid && b.bytes && !will_overwrite;
        // inside a recorded step the host's bytes are a constant of the step: placed and uploaded once, no copy node
        if (g.cap && have_data && (b.ptr = capture_const_place(b.shadow, b.bytes, sz)) != nullptr) { b.in_arena = true; b.step_const = true; }
        else {
            if (g.cap && (b.ptr = capture_arena_alloc(sz)) != nullptr) b.in_arena = true;
            else THC_CUDA_OK(cudaMallocAsync(&b.ptr, sz, g.stream));
            if (have_data) {
                uint8_t *stage = ring_take(sz);
                memset(stage, 0, sz);
                memcpy(stage, b.shadow, b.bytes);
                THC_CUDA_OK(cudaMemcpyAsync(b.ptr, stage, sz, cudaMemcpyHostToDevice, g.stream));
            } else if (!will_overwrite) {
                THC_CUDA_OK(cudaMemsetAsync(b.ptr, 0, sz, g.stream));
            }
        }
    }
    if (b.zero_pending) {
        if (outlives_capture) { settle_outside_capture(b, false); return b; }
        THC_CUDA_OK(cudaMemsetAsync(b.ptr, 0, (b.bytes + 15) & ~15ull, g.stream));
        b.zero_pending = false;
    }
    return b;
}

Buf &buf_checked(uint32_t id, const char *who) { return buf_attach(id, who, false); }

void fence_copy(Buf &b) {
    if (!b.copy_pending) return;
    THC_CUDA_OK(cudaStreamWaitEvent(g.stream, g.copy_done, 0));    // copy_done follows the latest asynchronous read-back
    b.copy_pending = false;
}

Buf &buf_for_output(uint32_t id, const char *who, uint64_t bytes_written) {
    Buf &b = buf_live(id, who);
    fence_copy(b);
    // (not for a buffer that outlives a running capture: the overwrite is only being recorded)
    const bool whole = bytes_written >= b.bytes && !(g.cap && id < capture_first_id());
    if (b.ptr && b.zero_pending && whole) b.zero_pending = false;
    Buf &r = buf_attach(id, who, whole);
    if (r.step_const) capture_const_dirty(r.ptr);
    return r;
}

void *scratch_reserve(uint64_t bytes) {
    if (bytes <= g.scratch_bytes) return g.scratch;
    if (g.cap) { capture_fail("library scratch had to grow inside the captured step: run the step once before capturing it"); return g.scratch; }
    if (g.scratch) THC_CUDA_OK(cudaFreeAsync(g.scratch, g.stream));
    uint64_t want = bytes + (bytes >> 2);
    THC_CUDA_OK(cudaMallocAsync(&g.scratch, want, g.stream));
    g.scratch_bytes = want;
    return g.scratch;
}

// ---- per-family launch statistics (profile_report) ----
struct PlanStat { uint64_t launches = 0; double ms = 0; unsigned long long ops = 0, bytes = 0; };
static std::map<std::string, PlanStat> *plan_stats = nullptr;
static cudaEvent_t prof_ev[2] = {nullptr, nullptr};
static bool prof_open = false;

void after_launch(const char *plan) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) fatal("launch of %s failed: %s", plan, cudaGetErrorString(e));
    g.launches++;
    g.last_plan = plan;
    if (g.profile && !g.cap) {
        if (!plan_stats) plan_stats = new std::map<std::string, PlanStat>();
        PlanStat &s = (*plan_stats)[plan];
        s.launches++;
        // the estimates of a dispatch go to its first launch that is not an operand pre-pass of a contraction
        static const char *const prepass[] = {"conv_relayout_input", "conv_relayout_weights", "gemm_transpose_operand", "wgrad_pad_width"};
        bool pre = false;
        for (const char *q : prepass) pre = pre || strcmp(plan, q) == 0;
        const unsigned long long ops = pre ? 0 : g.prof_ops, bytes = pre ? 0 : g.prof_bytes;
        s.ops += ops; s.bytes += bytes;
        if (!pre) g.prof_ops = g.prof_bytes = 0;
        if (prof_open) {           // close the bracket opened by profile_begin
            THC_CUDA_OK(cudaEventRecord(prof_ev[1], g.stream));
            THC_CUDA_OK(cudaEventSynchronize(prof_ev[1]));
            float ms = 0; THC_CUDA_OK(cudaEventElapsedTime(&ms, prof_ev[0], prof_ev[1]));
            s.ms += ms; prof_open = false;
            if (g.profile_level >= 2 && (ms > 0.1f || g.profile_level >= 3))
                fprintf(stderr, "thvm_cuda slow launch: %-22s %8.3f ms (%9.2f GFLOPS %7.1f GB/s)  %s\n", plan, ms, ops / (ms * 1e6), bytes / (ms * 1e6), g.last_shape);
        }
    }
}
void profile_begin() {             // called by dispatchers right before a launch when profiling
    if (!g.profile || g.cap) return;
    if (!prof_ev[0]) { cudaEventCreate(&prof_ev[0]); cudaEventCreate(&prof_ev[1]); }
    THC_CUDA_OK(cudaEventRecord(prof_ev[0], g.stream));
    prof_open = true;
}

static void check_device_status(const char *who) {
    if (g.cap) return;                                 // nothing may wait for the stream while it records
    int st = 0;
    THC_CUDA_OK(cudaMemcpyAsync(&st, g.dev_status, sizeof st, cudaMemcpyDeviceToHost, g.stream));
    THC_CUDA_OK(cudaStreamSynchronize(g.stream));
    if (st) {
        set_error("%s: device status 0x%x (1=load out of bounds, 2=store out of bounds, 4=bad program, 8=contraction kernel wait ran out, 16=a data-parallel peer never arrived)", who, st);
        THC_CUDA_OK(cudaMemsetAsync(g.dev_status, 0, sizeof(int), g.stream));
    }
}

// ---- staging ring ----
static uint8_t *ring_take(uint64_t bytes) {
    if (g.cap) return capture_arena_take(bytes);       // a captured copy reads its staging bytes again at every launch
    const uint64_t half = g.ring_bytes / 2;
    bytes = (bytes + 63) & ~63ull;
    unsigned cur = (unsigned)(g.ring_pos / half);
    if (g.ring_pos % half + bytes > half) {            // leave this half: fence it, enter the other
        THC_CUDA_OK(cudaEventRecord(g.ring_half[cur], g.stream));
        g.ring_half_pending[cur] = true;
        cur ^= 1u;
        if (g.ring_half_pending[cur]) {
            THC_CUDA_OK(cudaEventSynchronize(g.ring_half[cur]));
            g.ring_half_pending[cur] = false;
        }
        g.ring_pos = (uint64_t)cur * half;
    }
    uint8_t *p = g.ring + g.ring_pos;
    g.ring_pos += bytes;
    return p;
}

void upload_small(void *dev_dst, const void *src, uint64_t bytes) {
    if (bytes > RING_MAX_MSG) fatal("upload_small: %llu bytes", (unsigned long long)bytes);
    uint8_t *stage = ring_take(bytes);
    memcpy(stage, src, bytes);
    THC_CUDA_OK(cudaMemcpyAsync(dev_dst, stage, bytes, cudaMemcpyHostToDevice, g.stream));
}

}  // namespace thc

using namespace thc;

extern "C" {

int thvm_cuda_init(void) {
    if (g.ready) thvm_cuda_shutdown();
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        cudaGetLastError();
        set_error("init: no CUDA device");
        return 1;
    }
    const char *ev = getenv("THVM_CUDA_DEVICE");
    if (!ev) ev = getenv("LOCAL_RANK");
    int dev = ev ? atoi(ev) : 0;
    if (dev < 0 || dev >= n) dev = dev % n;
    if (cudaSetDevice(dev) != cudaSuccess) { set_error("init: cudaSetDevice(%d) failed", dev); return 1; }
    cudaDeviceProp prop;
    THC_CUDA_OK(cudaGetDeviceProperties(&prop, dev));
    if (prop.major < 10) {
        set_error("init: device %d is sm_%d%d; this library is built for sm_100a only", dev, prop.major, prop.minor);
        return 1;
    }
    g.device = dev;
    g.sm_count = prop.multiProcessorCount;
    THC_CUDA_OK(cudaStreamCreateWithFlags(&g.stream, cudaStreamNonBlocking));
    THC_CUDA_OK(cudaStreamCreateWithFlags(&g.copy_stream, cudaStreamNonBlocking));
    THC_CUDA_OK(cudaEventCreateWithFlags(&g.copy_after, cudaEventDisableTiming));
    THC_CUDA_OK(cudaEventCreateWithFlags(&g.copy_done, cudaEventDisableTiming));
    cudaMemPool_t mp;
    THC_CUDA_OK(cudaDeviceGetDefaultMemPool(&mp, dev));
    uint64_t keep_all = UINT64_MAX;
    THC_CUDA_OK(cudaMemPoolSetAttribute(mp, cudaMemPoolAttrReleaseThreshold, &keep_all));
    THC_CUDA_OK(cudaHostAlloc((void **)&g.ring, RING_BYTES, cudaHostAllocDefault));
    g.ring_bytes = RING_BYTES; g.ring_pos = 0;
    for (int i = 0; i < 2; i++) {
        THC_CUDA_OK(cudaEventCreateWithFlags(&g.ring_half[i], cudaEventDisableTiming));
        g.ring_half_pending[i] = false;
    }
    THC_CUDA_OK(cudaMalloc((void **)&g.dev_status, sizeof(int)));
    THC_CUDA_OK(cudaMemset(g.dev_status, 0, sizeof(int)));
    for (uint32_t i = 0; i < THC_MAX_BUFS; i++) g.bufs[i] = Buf();
    g.count = 1; g.persistent = 0;
    g.scratch = nullptr; g.scratch_bytes = 0;
    g.launches = 0; g.last_plan = ""; g.last_error.clear();
    g.cur_bytes = g.peak_bytes = g.last_step_peak = 0;
    g.profile = getenv("THVM_PROFILE") != nullptr;
    g.profile_level = g.profile ? atoi(getenv("THVM_PROFILE")) : 0;
    g.ready = true;
    return 0;
}

static void release(uint32_t id) {
    Buf &b = g.bufs[id];
    fence_copy(b);
    if (b.ptr && g.cap && id < capture_first_id())
        capture_fail("the captured step frees a buffer that was allocated before the capture began");
    if (b.ptr) {
        if (b.in_arena) { if (g.cap && !b.step_const) capture_arena_give_back(b.ptr, ((b.bytes + 15) & ~15ull) ? ((b.bytes + 15) & ~15ull) : 16); }
        else if (b.plain_alloc) THC_CUDA_OK(cudaFree(b.ptr));
        else THC_CUDA_OK(cudaFreeAsync(b.ptr, g.stream));
        if (!g.cap && !b.in_arena && b.bytes > SHADOW_MAX) { const uint64_t sz = (b.bytes + 15) & ~15ull; g.cur_bytes = g.cur_bytes > sz ? g.cur_bytes - sz : 0; }
    }
    free(b.shadow);
    b = Buf();
}

void plan_cache_clear(void);   // plan.cu
void thvm_cuda_dp_shutdown(void);   // dp.cu

void thvm_cuda_shutdown(void) {
    if (!g.ready) return;
    capture_shutdown();
    thvm_cuda_dp_shutdown();
    cudaStreamSynchronize(g.stream);
    for (uint32_t i = 1; i < g.count; i++) if (g.bufs[i].live) release(i);
    plan_cache_clear();
    if (g.scratch) cudaFreeAsync(g.scratch, g.stream);
    g.scratch = nullptr; g.scratch_bytes = 0;
    cudaStreamSynchronize(g.stream);
    cudaFree(g.dev_status); g.dev_status = nullptr;
    cudaFreeHost(g.ring); g.ring = nullptr;
    for (int i = 0; i < 2; i++) { cudaEventDestroy(g.ring_half[i]); g.ring_half[i] = nullptr; }
    cudaStreamSynchronize(g.copy_stream);
    cudaEventDestroy(g.copy_after); cudaEventDestroy(g.copy_done); g.copy_after = g.copy_done = nullptr;
    cudaStreamDestroy(g.copy_stream); g.copy_stream = nullptr;
    cudaStreamDestroy(g.stream); g.stream = nullptr;
    g.count = 1;
    g.ready = false;
}

uint32_t thvm_cuda_buf_alloc(uint64_t bytes) {
    if (!g.ready) fatal("buf_alloc: backend not initialised (no CUDA device?)");
    if (g.count >= THC_MAX_BUFS) { set_error("buf_alloc: id space exhausted (%u)", THC_MAX_BUFS); return 0; }
    void *p = nullptr;
    bool in_arena = false;
    if (bytes > SHADOW_MAX) {
        uint64_t sz = (bytes + 15) & ~15ull;
        if (g.cap && (p = capture_arena_alloc(sz)) != nullptr) in_arena = true;     // planned: no allocator call in the recorded step
        else {
            cudaError_t e = cudaMallocAsync(&p, sz, g.stream);
            if (e != cudaSuccess) {
                cudaGetLastError();
                set_error("buf_alloc: %llu bytes: %s", (unsigned long long)bytes, cudaGetErrorString(e));
                return 0;
            }
        }
        if (!g.cap) { g.cur_bytes += sz; if (g.cur_bytes > g.peak_bytes) g.peak_bytes = g.cur_bytes; }
    }
    uint32_t id = g.count++;
    Buf &b = g.bufs[id];
    b.live = true; b.ptr = p; b.bytes = bytes; b.refcount = 1; b.in_arena = in_arena;
    b.zero_pending = p != nullptr;                 // the zero-fill is issued on first use, and dropped if that use overwrites everything
    if (bytes <= SHADOW_MAX) {
        b.shadow = (uint8_t *)calloc(1, SHADOW_MAX);
        b.shadow_valid = true;                     // zeros, like a fresh device buffer
    }
    return id;
}

void thvm_cuda_buf_free(uint32_t id) {
    if (!g.ready || id == 0 || id >= THC_MAX_BUFS || !g.bufs[id].live) return;
    release(id);
}

void thvm_cuda_buf_incref(uint32_t id) {
    if (!g.ready || id == 0 || id >= THC_MAX_BUFS || !g.bufs[id].live) return;
    g.bufs[id].refcount++;
}

void thvm_cuda_buf_decref(uint32_t id) {
    if (!g.ready || id == 0 || id >= THC_MAX_BUFS || !g.bufs[id].live) return;
    if (id <= g.persistent) return;
    Buf &b = g.bufs[id];
    if (b.refcount > 0) b.refcount--;
    if (b.refcount == 0) release(id);
}

void thvm_cuda_mem_checkpoint(uint32_t *leaf_buf_ids, uint32_t n_leaves) {
    (void)leaf_buf_ids; (void)n_leaves;   // stream-ordered frees need no checkpoint
}
void thvm_cuda_buf_mark_use(uint32_t id) { (void)id; }

void thvm_cuda_buf_write(uint32_t id, const void *data, uint64_t bytes) {
    Buf &b = buf_live(id, "buf_write");
    if (bytes > b.bytes) {
        set_error("buf_write: %llu bytes into buffer %u of %llu", (unsigned long long)bytes, id, (unsigned long long)b.bytes);
        bytes = b.bytes;
    }
    if (bytes == 0) return;
    if (b.shadow) {
        // the shadow speaks for the whole buffer only if it did before, or if this write covers all of it
        // (after a kernel wrote the buffer, a partial host write leaves the rest on the device only)
        if (b.shadow_valid || bytes >= b.bytes) { memcpy(b.shadow, data, bytes); b.shadow_valid = true; }
    }
    if (!b.ptr) return;                            // host-only buffer: uploaded if and when the device needs it
    fence_copy(b);
    if (g.cap && b.in_arena && !b.step_const && b.zero_pending && bytes <= RING_MAX_MSG && !capture_write_is_input(bytes)) {
        // a constant of the recorded step, written into a buffer nothing has read or written yet: move the buffer to the
        // constants' part of the arena and upload it once (zero-padded), instead of a copy node in the chain
        const uint64_t sz = ((b.bytes + 15) & ~15ull) ? ((b.bytes + 15) & ~15ull) : 16;
        void *p = capture_const_place(data, bytes, sz);
        if (p) {
            capture_arena_give_back(b.ptr, sz);
            b.ptr = p; b.step_const = true; b.zero_pending = false;
            return;
        }
    }
    if (b.zero_pending) {
        if (g.cap && id < capture_first_id()) settle_outside_capture(b, false);
        else {
            if (bytes < b.bytes) THC_CUDA_OK(cudaMemsetAsync(b.ptr, 0, (b.bytes + 15) & ~15ull, g.stream));
            b.zero_pending = false;
        }
    }
    if (g.cap && capture_write_is_input(bytes)) { capture_add_input(b.ptr, data, bytes); return; }
    if (b.step_const) capture_const_dirty(b.ptr);      // written again inside the step: the first bytes are put back at the end
    if (bytes <= RING_MAX_MSG) {
        uint8_t *stage = ring_take(bytes);
        memcpy(stage, data, bytes);
        THC_CUDA_OK(cudaMemcpyAsync(b.ptr, stage, bytes, cudaMemcpyHostToDevice, g.stream));
    } else {
        // Large payloads go straight from the caller's memory (full PCIe rate
        // when it is pinned) and the call waits for the DMA, after which the
        // caller may reuse the source.
        if (g.cap) { capture_add_input(b.ptr, data, bytes); return; }   // an input of the captured step: the caller keeps `data` alive
        THC_CUDA_OK(cudaMemcpyAsync(b.ptr, data, bytes, cudaMemcpyHostToDevice, g.stream));
        THC_CUDA_OK(cudaStreamSynchronize(g.stream));
    }
}

static void read_impl(uint32_t id, void *out, uint64_t bytes, bool sync) {
    Buf &b = buf_live(id, "buf_read");
    uint64_t n = bytes < b.bytes ? bytes : b.bytes;
    if (bytes > n) memset((uint8_t *)out + n, 0, bytes - n);   // past the end reads as zero (src/backend/metal/pool.m:214-218)
    if (n == 0) return;
    if (b.shadow && b.shadow_valid) { memcpy(out, b.shadow, n); return; }
    if (!b.ptr || b.zero_pending) { memset(out, 0, n); return; }
    if (g.cap) { capture_add_result(b.ptr, n); memset(out, 0, n); return; }   // values come from graph_result after a launch
    THC_CUDA_OK(cudaMemcpyAsync(out, b.ptr, n, cudaMemcpyDeviceToHost, g.stream));
    if (sync) check_device_status("buf_read");                // drains the stream
}
void thvm_cuda_buf_read(uint32_t id, void *out, uint64_t bytes) { read_impl(id, out, bytes, true); }
// The vtable's buf_read_nosync serves META_READ (src/interact/_.c:8-11): small metadata the host wrote itself, read
// back "without a GPU flush", and the caller uses the bytes as soon as the call returns.  Host-written buffers of up
// to 256 bytes come from their host shadow without touching the device; anything else is read like buf_read.
void thvm_cuda_buf_read_nosync(uint32_t id, void *out, uint64_t bytes) { read_impl(id, out, bytes, true); }
// Asynchronous read-back (no vtable slot): the copy is ordered after the work already queued on the main stream and
// runs on a copy stream of its own, so it overlaps later uploads and kernels; `out` (pinned memory keeps it truly
// asynchronous) holds the data after thvm_cuda_sync().  The library keeps later writes to and frees of the same
// buffer behind the copy.
void thvm_cuda_buf_read_async(uint32_t id, void *out, uint64_t bytes) {
    Buf &b = buf_live(id, "buf_read_async");
    uint64_t n = bytes < b.bytes ? bytes : b.bytes;
    if (bytes > n) memset((uint8_t *)out + n, 0, bytes - n);
    if (n == 0) return;
    if ((b.shadow && b.shadow_valid) || !b.ptr || b.zero_pending || g.cap) { read_impl(id, out, bytes, false); return; }
    THC_CUDA_OK(cudaEventRecord(g.copy_after, g.stream));
    THC_CUDA_OK(cudaStreamWaitEvent(g.copy_stream, g.copy_after, 0));
    THC_CUDA_OK(cudaMemcpyAsync(out, b.ptr, n, cudaMemcpyDeviceToHost, g.copy_stream));
    THC_CUDA_OK(cudaEventRecord(g.copy_done, g.copy_stream));
    b.copy_pending = true;
}

void thvm_cuda_buf_copy(uint32_t dst_buf, uint32_t src_buf, uint64_t nbytes) {
    Buf &dl = buf_live(dst_buf, "buf_copy(dst)");
    Buf &sl = buf_live(src_buf, "buf_copy(src)");
    if (!dl.ptr && !sl.ptr && dl.shadow && sl.shadow && sl.shadow_valid && nbytes <= dl.bytes && nbytes <= sl.bytes) {
        memcpy(dl.shadow, sl.shadow, nbytes); dl.shadow_valid = true;      // both still host-only
        return;
    }
    Buf &s = buf_checked(src_buf, "buf_copy(src)");
    Buf &d = buf_for_output(dst_buf, "buf_copy(dst)", nbytes);
    uint64_t n = nbytes;
    if (n > d.bytes || n > s.bytes) {
        set_error("buf_copy: %llu bytes exceed dst %llu / src %llu", (unsigned long long)n,
                  (unsigned long long)d.bytes, (unsigned long long)s.bytes);
        n = d.bytes < s.bytes ? d.bytes : s.bytes;
    }
    if (n == 0) return;
    THC_CUDA_OK(cudaMemcpyAsync(d.ptr, s.ptr, n, cudaMemcpyDeviceToDevice, g.stream));
    if (d.shadow && s.shadow && s.shadow_valid && (d.shadow_valid || n >= d.bytes)) { memcpy(d.shadow, s.shadow, n); d.shadow_valid = true; }
    else d.shadow_valid = false;
}

void thvm_cuda_pool_reset(uint32_t keep) {
    if (!g.ready) return;
    uint32_t first = keep + 1;
    if (first < 1) first = 1;
    for (uint32_t i = first; i < g.count; i++) if (g.bufs[i].live) release(i);
    if (first < g.count) g.count = first;
    if (!g.cap) {                                  // a step ended: remember how much it held at its peak above what stays
        g.last_step_peak = g.peak_bytes > g.cur_bytes ? g.peak_bytes - g.cur_bytes : 0;
        g.peak_bytes = g.cur_bytes;
    }
}

void thvm_cuda_pool_set_persistent(uint32_t max_buf) { g.persistent = max_buf; }

void thvm_cuda_begin_batch(void) {}
void thvm_cuda_end_batch(void) {}   // one stream already orders and batches the work

void thvm_cuda_profile_report(void) {
    if (!plan_stats) { fprintf(stderr, "thvm_cuda profile: no launches recorded (set THVM_PROFILE=1 before init)\n"); return; }
    // per family: launches, device time, and the estimated operations / algorithmic bytes of its dispatches with the
    // rates they come to (the figures the Metal backend prints per kernel, src/backend/metal/profile_kernel.m:45-62)
    fprintf(stderr, "thvm_cuda profile: %-22s %10s %12s %12s %10s %12s %10s\n", "kernel family", "launches", "gpu ms", "Gop", "GFLOPS", "GB", "GB/s");
    for (auto &kv : *plan_stats) {
        const PlanStat &s = kv.second;
        const double per_sec = s.ms > 0 ? 1e3 / s.ms : 0.0;     // families that are never timed on their own report no rate
        fprintf(stderr, "thvm_cuda profile: %-22s %10llu %12.3f %12.3f %10.1f %12.3f %10.1f\n", kv.first.c_str(),
                (unsigned long long)s.launches, s.ms, s.ops * 1e-9, s.ops * 1e-9 * per_sec, s.bytes * 1e-9, s.bytes * 1e-9 * per_sec);
    }
}
void thvm_cuda_profile_reset(void) { if (plan_stats) plan_stats->clear(); g.launches = 0; }

const char *thvm_cuda_last_error(void) {
    if (g.ready && g.last_error.empty()) check_device_status("last_error");
    return g.last_error.c_str();
}
void thvm_cuda_clear_error(void) { g.last_error.clear(); }
void *thvm_cuda_stream(void) { return (void *)g.stream; }
void thvm_cuda_sync(void) {
    if (!g.ready || g.cap) return;
    THC_CUDA_OK(cudaStreamSynchronize(g.stream));
    THC_CUDA_OK(cudaStreamSynchronize(g.copy_stream));
}
void *thvm_cuda_buf_ptr(uint32_t id) {
    if (!(g.ready && id && id < THC_MAX_BUFS && g.bufs[id].live)) return nullptr;
    Buf &b = buf_checked(id, "buf_ptr");    // attaches device memory if the buffer was host-only
    b.shadow_valid = false;                 // the caller may write through the pointer: the host shadow no longer speaks for it
    return b.ptr;
}
uint64_t thvm_cuda_buf_bytes(uint32_t id) { return (g.ready && id && id < THC_MAX_BUFS && g.bufs[id].live) ? g.bufs[id].bytes : 0; }
uint64_t thvm_cuda_launch_count(void) { return g.launches; }
const char *thvm_cuda_last_plan(void) { return g.last_plan; }
void thvm_cuda_set_force_generic(int on) { g.force_generic = on; }

}  // extern "C"
