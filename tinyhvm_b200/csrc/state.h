// state.h — process-global state of the backend (host side).
//
// The reference's vtable carries no context pointer and its backends keep
// file-scope state (src/backend/cpu/pool.c:6-10), so this library does too:
// one process, one GPU, one stream.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string>
#include "../../include/thvm_cuda.h"

namespace thc {

struct Buf {
    bool     live     = false;     // id handed out and not yet freed
    void    *ptr      = nullptr;   // device memory; null while a small host-written buffer lives only in its shadow
    uint64_t bytes    = 0;         // size asked for by the caller
    uint32_t refcount = 0;
    uint8_t *shadow   = nullptr;   // host copy of a small host-written buffer
    bool     shadow_valid = false; // false once a kernel or copy wrote the buffer
    bool     zero_pending = false; // fresh device memory whose zero-fill has not been issued yet
    bool     copy_pending = false; // an asynchronous read-back of this buffer may still be in flight on the copy stream
    bool     plain_alloc = false;  // ptr came from cudaMalloc (attached while a step was being captured), not from the stream-ordered pool
    bool     in_arena = false;     // ptr lies in the step arena of the capture that is running (capture.cu): nothing to free
    bool     step_const = false;   // in_arena, in the part that is never handed out twice: a constant of the recorded step, uploaded once
};

struct Capture;                    // capture.cu: the step being recorded as a CUDA graph

struct State {
    bool         ready = false;
    int          device = 0;
    int          sm_count = 148;
    cudaStream_t stream = nullptr;
    cudaStream_t copy_stream = nullptr;   // device->host copies of buf_read_async, so they overlap uploads and kernels on `stream`
    cudaEvent_t  copy_after = nullptr, copy_done = nullptr;
    Buf          bufs[THC_MAX_BUFS];
    uint32_t     count = 1;          // next id; 0 is the null buffer
    uint32_t     persistent = 0;     // ids <= this survive decref
    Capture     *cap = nullptr;      // non-null while a step is being captured
    // pinned staging ring for small host->device writes
    uint8_t     *ring = nullptr;
    uint64_t     ring_bytes = 0, ring_pos = 0;
    cudaEvent_t  ring_half[2] = {nullptr, nullptr};
    bool         ring_half_pending[2] = {false, false};
    // pinned bounce buffer for reads
    uint8_t     *bounce = nullptr;
    uint64_t     bounce_bytes = 0;
    // device status word raised by kernels (load/store out of bounds ...)
    int         *dev_status = nullptr;
    // library-owned scratch (two-pass reductions, operand splits); grow-only
    void        *scratch = nullptr;
    uint64_t     scratch_bytes = 0;
    // device bytes behind live buffers: now, highest since the last pool_reset, and that peak of the last finished step
    // above what stayed live (sizes the step arena of a capture)
    uint64_t     cur_bytes = 0, peak_bytes = 0, last_step_peak = 0;
    // bookkeeping
    uint64_t     launches = 0;
    const char  *last_plan = "";
    int          force_generic = 0;
    std::string  last_error;
    // profiling (THVM_PROFILE / profile_report)
    bool         profile = false;
    unsigned long long prof_ops = 0, prof_bytes = 0;   // estimates of the dispatch about to launch (profile_report)
    int          profile_level = 0;   // THVM_PROFILE=2: also print every launch slower than 0.1 ms with its shape; 3: every launch
    char         last_shape[160] = {0};
};

extern State g;

void set_error(const char *fmt, ...);
[[noreturn]] void fatal(const char *fmt, ...);

#define THC_CUDA_OK(expr)                                                         \
    do {                                                                          \
        cudaError_t _e = (expr);                                                  \
        if (_e != cudaSuccess)                                                    \
            ::thc::fatal("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),  \
                         __FILE__, __LINE__);                                     \
    } while (0)

// a live buffer with device memory behind it (materialised on demand), or a fatal error
Buf &buf_checked(uint32_t id, const char *who);
// the output buffer of a launch that overwrites its first `bytes_written` bytes: the zero-fill a fresh
// buffer owes is dropped when that covers the whole buffer.  Resolve the inputs of the launch first.
Buf &buf_for_output(uint32_t id, const char *who, uint64_t bytes_written);
// a live buffer that may still be host-only
Buf &buf_live(uint32_t id, const char *who);
// scratch of at least `bytes` (stream-ordered reuse: all users run on g.stream)
void *scratch_reserve(uint64_t bytes);
// before `b` is overwritten or freed on the main stream: wait for a read-back of it that may still be running
void fence_copy(Buf &b);
// mark a buffer as written by the device
void capture_const_dirty(void *dev);             // capture.cu: a step constant is overwritten inside the recorded step
inline void mark_device_written(uint32_t id) { g.bufs[id].shadow_valid = false; if (g.bufs[id].step_const) capture_const_dirty(g.bufs[id].ptr); }
// grid size helper: enough CTAs to fill the machine `waves` times over
inline unsigned grid_for(uint64_t work_items, unsigned per_cta, unsigned max_ctas_per_sm = 16) {
    uint64_t need = (work_items + per_cta - 1) / per_cta;
    uint64_t cap  = (uint64_t)g.sm_count * max_ctas_per_sm;
    if (need < 1) need = 1;
    return (unsigned)(need < cap ? need : cap);
}
// bracket a launch: profile_begin() before, after_launch() after
void profile_begin();
void after_launch(const char *plan);
// host -> device copy of a small block through the pinned staging ring
void upload_small(void *dev_dst, const void *src, uint64_t bytes);

// ---- step capture (capture.cu) ----
bool capturing();
// mark the running capture unusable (capture_end will then fail with this reason); no-op outside a capture
void capture_fail(const char *why);
uint32_t capture_first_id();                                    // first buffer id handed out inside the capture
// the step planner: memory for a buffer allocated inside a capture, from the capture's arena (null: arena full or absent);
// give_back returns a block when the captured step frees the buffer
void *capture_arena_alloc(uint64_t bytes);
void capture_arena_give_back(void *ptr, uint64_t bytes);
// A constant of the step being recorded (bytes the host wrote inside the step, the same at every replay): device memory
// in the part of the step arena that is never handed out twice, filled now, outside the recording.  Null if there is no room.
void *capture_const_place(const void *host, uint64_t host_bytes, uint64_t buf_bytes);
bool capture_write_is_input(uint64_t bytes);                    // a host write of this size made inside a capture is per-step data, not a constant
uint8_t *capture_arena_take(uint64_t bytes);                    // pinned host memory that lives as long as the graph
int  capture_add_input(void *dst, const void *src, uint64_t bytes);
void capture_add_result(const void *src, uint64_t bytes);
void capture_shutdown();

}  // namespace thc
