// backend/cuda/_.c — CUDA backend hub for TinyHVM: the `Backend cuda_backend`
// vtable instance, bound at run time to libthvm_cuda.so.
//
// This is the reference-side half of the drop-in: it is written against the
// reference's own header (src/tinyhvm.h:988-1046, struct Backend) and is meant
// to sit beside src/backend/cpu/_.c and src/backend/metal/_.m.  A driver
// includes it after "tinyhvm.c" exactly like the other hubs
// (test/test_mm_dup_2arm.m:14-18):
//
//     #include "tinyhvm.c"
//     #include "backend/cpu/_.c"
//     #include "backend/cuda/_.c"
//
// The library is opened with dlopen on first init, so a build of this file
// has no link-time CUDA dependency and a host without a GPU can still run the
// CPU backend.  There is no silent fallback: if "cuda" is requested and the
// library or a device is missing, thvm_init_device() aborts.
//
// Every slot is the like-named entry point of include/thvm_cuda.h; the PODs
// (View, ShapeTracker, FusedOp, ReduceSpec, UOpKernel) cross the boundary by
// pointer and are layout-identical (checked below).
#ifndef THVM_BACKEND_CUDA_HUB
#define THVM_BACKEND_CUDA_HUB

#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "thvm_cuda.h"

_Static_assert(sizeof(thc_shape_t) == sizeof(Shape), "Shape mirror");
_Static_assert(sizeof(thc_view_t) == sizeof(View), "View mirror");
_Static_assert(offsetof(thc_view_t, compound_masks) == offsetof(View, compound_masks), "View mirror");
_Static_assert(sizeof(thc_tracker_t) == sizeof(ShapeTracker), "ShapeTracker mirror");
_Static_assert(sizeof(thc_fused_op_t) == sizeof(FusedOp), "FusedOp mirror");
_Static_assert(sizeof(thc_reduce_spec_t) == sizeof(ReduceSpec), "ReduceSpec mirror");
_Static_assert(sizeof(thc_uop_kernel_t) == sizeof(UOpKernel), "UOpKernel mirror");

#define THVM_DEV_CUDA 2   // backends[0] = cpu, [1] = metal (src/tinyhvm.h:1052-1054)

Backend cuda_backend;     // filled by cuda_hub_init
static void *cuda_hub_lib = NULL;

static void *cuda_hub_sym(const char *name) {
    void *p = dlsym(cuda_hub_lib, name);
    if (!p) { fprintf(stderr, "TinyHVM cuda: %s missing from libthvm_cuda.so\n", name); exit(1); }
    return p;
}

// Backend.init: open the library, bind all slots, run the library's init.
static int cuda_hub_init(void) {
    if (!cuda_hub_lib) {
        const char *path = getenv("THVM_CUDA_LIB");
        cuda_hub_lib = dlopen(path ? path : "libthvm_cuda.so", RTLD_NOW | RTLD_LOCAL);
        if (!cuda_hub_lib) { fprintf(stderr, "TinyHVM cuda: %s\n", dlerror()); return 1; }
        Backend *b = &cuda_backend;
        b->shutdown            = cuda_hub_sym("thvm_cuda_shutdown");
        b->buf_alloc           = cuda_hub_sym("thvm_cuda_buf_alloc");
        b->buf_free            = cuda_hub_sym("thvm_cuda_buf_free");
        b->buf_incref          = cuda_hub_sym("thvm_cuda_buf_incref");
        b->buf_decref          = cuda_hub_sym("thvm_cuda_buf_decref");
        b->mem_checkpoint      = cuda_hub_sym("thvm_cuda_mem_checkpoint");
        b->buf_mark_use        = cuda_hub_sym("thvm_cuda_buf_mark_use");
        b->buf_write           = cuda_hub_sym("thvm_cuda_buf_write");
        b->buf_read            = cuda_hub_sym("thvm_cuda_buf_read");
        b->op_unary            = cuda_hub_sym("thvm_cuda_op_unary");
        b->op_binary           = cuda_hub_sym("thvm_cuda_op_binary");
        b->op_mm               = cuda_hub_sym("thvm_cuda_op_mm");
        b->op_reduce           = cuda_hub_sym("thvm_cuda_op_reduce");
        b->dispatch_kernel_rs  = cuda_hub_sym("thvm_cuda_dispatch_kernel_rs");
        b->contiguify          = cuda_hub_sym("thvm_cuda_contiguify");
        b->buf_copy            = cuda_hub_sym("thvm_cuda_buf_copy");
        b->buf_read_nosync     = cuda_hub_sym("thvm_cuda_buf_read_nosync");
        b->adam_step           = cuda_hub_sym("thvm_cuda_adam_step");
        b->pool_reset          = cuda_hub_sym("thvm_cuda_pool_reset");
        b->pool_set_persistent = cuda_hub_sym("thvm_cuda_pool_set_persistent");
        b->begin_batch         = cuda_hub_sym("thvm_cuda_begin_batch");
        b->end_batch           = cuda_hub_sym("thvm_cuda_end_batch");
        b->profile_report      = cuda_hub_sym("thvm_cuda_profile_report");
        b->profile_reset       = cuda_hub_sym("thvm_cuda_profile_reset");
    }
    // The scheduler prefers the lowered KOP form whenever this slot is set
    // (src/schedule/_.c:2370).  The structured form carries the views and the
    // reduce spec the kernel selection needs, so the slot stays NULL unless
    // THVM_CUDA_UOP=1 asks for the KOP interpreter (looked at on every init).
    cuda_backend.dispatch_uop_kernel = getenv("THVM_CUDA_UOP") ? cuda_hub_sym("thvm_cuda_dispatch_uop_kernel") : NULL;
    int (*lib_init)(void) = cuda_hub_sym("thvm_cuda_init");
    return lib_init();
}

Backend cuda_backend = { .init = cuda_hub_init };

// thvm_init with a "cuda" branch, mirroring the Metal branch of the
// reference's thvm_init (src/ctx/init.c:24-35).  `base_init` is the reference's
// own thvm_init (a driver that cannot edit src/ctx/init.c renames it with
// `#define thvm_init thvm_init_base` around `#include "tinyhvm.c"`).
static TinyHVM *thvm_init_device(TinyHVM *(*base_init)(const char *), const char *device) {
    TinyHVM *ctx = base_init(device);
    if (device && (strcmp(device, "cuda") == 0 || strcmp(device, "b200") == 0)) {
        if (cuda_backend.init() != 0) {
            fprintf(stderr, "TinyHVM: requested cuda backend unavailable (no CPU fallback)\n");
            exit(1);
        }
        ctx->backends[THVM_DEV_CUDA] = &cuda_backend;
        ctx->n_backends = THVM_DEV_CUDA + 1;
        ctx->default_device = THVM_DEV_CUDA;
    }
    return ctx;
}

// ---- step capture / replay: the reference's JIT entry points (src/tinyhvm.h:1294-1300), which it declares for Apple
// builds only and implements in src/backend/metal/jit.m:24-631.  Same call sequence as there (test/archive/test_jit_dense.m):
//     jit_begin_capture(n_persistent);  <one training step through thvm_eval / thvm_reduce>;  jit_end_capture();
//     then per step: refresh the inputs, jit_replay().
// Differences a driver has to know: the captured step is recorded, not run (its first execution is the first
// jit_replay; values read inside it come back as zeros and are fetched afterwards with jit_result), the step must have
// run eagerly before (kernel plans exist) and must free what it allocates (end with thvm_reset).  Per-step data that the
// step uploads with buf_write (a fresh tensor per batch) is declared by its byte size with jit_declare_input before
// jit_begin_capture; jit_set_input points input k at this step's host memory before jit_replay.
#ifndef __APPLE__
static int cuda_jit_graph = 0;
static u64 cuda_jit_sizes[8];
static u32 cuda_jit_n_sizes = 0;
void jit_declare_input(u64 bytes) { if (cuda_jit_n_sizes < 8) cuda_jit_sizes[cuda_jit_n_sizes++] = bytes; }   // addition of this backend
void jit_begin_capture(u32 n_persistent_bufs) {
    (void)n_persistent_bufs;                       // buffers that exist now are the persistent ones
    void (*sizes)(const u64 *, u32) = cuda_hub_sym("thvm_cuda_capture_input_sizes");
    int (*begin)(void) = cuda_hub_sym("thvm_cuda_capture_begin");
    if (cuda_jit_graph) { void (*destroy)(int) = cuda_hub_sym("thvm_cuda_graph_destroy"); destroy(cuda_jit_graph); cuda_jit_graph = 0; }
    sizes(cuda_jit_sizes, cuda_jit_n_sizes);
    if (begin() != 0) { fprintf(stderr, "TinyHVM cuda: jit_begin_capture failed\n"); exit(1); }
}
void jit_end_capture(void) {
    int (*end)(void) = cuda_hub_sym("thvm_cuda_capture_end");
    void (*sizes)(const u64 *, u32) = cuda_hub_sym("thvm_cuda_capture_input_sizes");
    const char *(*err)(void) = cuda_hub_sym("thvm_cuda_last_error");
    cuda_jit_graph = end();
    sizes(NULL, 0); cuda_jit_n_sizes = 0;
    if (!cuda_jit_graph) { fprintf(stderr, "TinyHVM cuda: jit_end_capture: %s\n", err()); exit(1); }
}
void jit_flush(void) { void (*sync)(void) = cuda_hub_sym("thvm_cuda_sync"); sync(); }
void jit_replay(void) {
    int (*launch)(int) = cuda_hub_sym("thvm_cuda_graph_launch");
    if (!cuda_jit_graph || launch(cuda_jit_graph) != 0) { fprintf(stderr, "TinyHVM cuda: jit_replay without a captured step\n"); exit(1); }
}
// additions of this backend
u32 jit_input_count(void) {
    int (*counts)(int, u32 *, u32 *, u64 *) = cuda_hub_sym("thvm_cuda_graph_counts");
    u32 n = 0; counts(cuda_jit_graph, &n, NULL, NULL); return n;
}
u64 jit_input_bytes(u32 k) { u64 (*f)(int, int) = cuda_hub_sym("thvm_cuda_graph_input_bytes"); return f(cuda_jit_graph, (int)k); }
void jit_set_input(u32 k, const void *host) {
    int (*f)(int, int, const void *) = cuda_hub_sym("thvm_cuda_graph_set_input");
    if (f(cuda_jit_graph, (int)k, host) != 0) { fprintf(stderr, "TinyHVM cuda: jit_set_input(%u) failed\n", k); exit(1); }
}
void jit_result(u32 k, void *out, u64 bytes) {
    int (*f)(int, int, void *, u64) = cuda_hub_sym("thvm_cuda_graph_result");
    if (f(cuda_jit_graph, (int)k, out, bytes) != 0) { fprintf(stderr, "TinyHVM cuda: jit_result(%u) failed\n", k); exit(1); }
}
#endif

#endif  // THVM_BACKEND_CUDA_HUB
