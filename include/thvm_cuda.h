/* thvm_cuda.h — C ABI of libthvm_cuda.so, the B200 (sm_100a) backend for
 * TinyHVM's realized-kernel path.
 *
 * Every entry point below has exactly the signature of one slot of the
 * reference's `struct Backend` vtable (reference: src/tinyhvm.h:988-1046), so
 * a `Backend cuda_backend = { .init = thvm_cuda_init, ... }` is a drop-in
 * beside `cpu_backend` (reference: src/backend/cpu/_.c:21-35).  The POD
 * structs are layout-identical mirrors of the reference's `Shape`, `View`,
 * `ShapeTracker`, `FusedOp`, `ReduceSpec`, `KOp` and `UOpKernel`
 * (reference: src/tinyhvm.h:531-717); the vtable shim static_asserts the
 * sizes against the reference header.
 *
 * State is process-global (the vtable has no context argument): one process
 * drives one GPU.  All work is issued on one CUDA stream; `buf_read`
 * synchronises it.  Nothing here falls back to the CPU: without a CUDA device
 * `thvm_cuda_init` returns non-zero and every other call aborts.
 */
#ifndef THVM_CUDA_H
#define THVM_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- limits (reference: src/tinyhvm.h:528-529, 571, 657-658, 674, 720) ---- */
#define THC_MAX_DIM      8
#define THC_MAX_VIEWS    4
#define THC_MAX_OPS      64
#define THC_MAX_LEAVES   64
#define THC_KOP_MAX      512
#define THC_MAX_BUFS     16384

/* ---- dtypes (reference: src/tinyhvm.h:417-421) ---- */
#define THC_F32 0
#define THC_F16 1
#define THC_I32 2
#define THC_U32 3

/* ---- UOp codes that reach the backend (reference: src/tinyhvm.h:116-137) ---- */
#define THC_NEG   3
#define THC_EXP   4
#define THC_LOG   5
#define THC_RELU  6
#define THC_CAST  7
#define THC_SQRT  8
#define THC_ADD   9
#define THC_MUL  10
#define THC_DIV  11
#define THC_MAX  12
#define THC_CMP  13
#define THC_SUB  14
#define THC_SUM  15
#define THC_RMAX 16

/* ---- POD mirrors ---- */
typedef struct {                       /* Shape, src/tinyhvm.h:531-534 */
    uint32_t dims[THC_MAX_DIM];
    uint32_t rank;
} thc_shape_t;

typedef struct {                       /* View, src/tinyhvm.h:549-566 */
    thc_shape_t shape;
    int32_t  strides[THC_MAX_DIM];     /* elements; 0 = broadcast */
    int32_t  offset;                   /* elements; may be negative (PAD) */
    uint32_t numel;
    uint8_t  contiguous;
    uint8_t  has_mask;
    uint32_t mask_begin[THC_MAX_DIM];
    uint32_t mask_end[THC_MAX_DIM];
    uint8_t  n_compound_masks;
    struct { uint8_t dim_a, dim_b; int32_t stride_a; uint32_t begin, end; } compound_masks[2];
    uint32_t mod_size[THC_MAX_DIM];
} thc_view_t;

typedef struct {                       /* ShapeTracker, src/tinyhvm.h:571-575 */
    thc_view_t views[THC_MAX_VIEWS];
    uint8_t    n_views;
} thc_tracker_t;

typedef struct {                       /* FusedOp, src/tinyhvm.h:659 */
    uint32_t uop, arg_a, arg_b, aux;
} thc_fused_op_t;

typedef struct {                       /* ReduceSpec, src/tinyhvm.h:660-672 */
    uint8_t  is_reduce[THC_MAX_DIM];
    uint32_t reduce_type;              /* 0, THC_SUM or THC_RMAX */
    uint32_t post_reduce_start;
    uint32_t n_post_leaves;
    uint32_t reduce2_type;
    uint32_t reduce2_start;
    uint8_t  is_reduce2[THC_MAX_DIM];
} thc_reduce_spec_t;

typedef enum {                         /* KOpType, src/tinyhvm.h:675-691 */
    THC_KOP_NOOP = 0, THC_KOP_GID, THC_KOP_CONST_F, THC_KOP_CONST_U,
    THC_KOP_RANGE, THC_KOP_ENDRANGE, THC_KOP_LOAD, THC_KOP_STORE,
    THC_KOP_ALU, THC_KOP_ACC_INIT, THC_KOP_ACC, THC_KOP_IDX,
    THC_KOP_MOD, THC_KOP_DIV, THC_KOP_MASK
} thc_kop_type_t;

typedef struct {                       /* KOp, src/tinyhvm.h:693-700 */
    thc_kop_type_t type;
    uint32_t arg[3];
    union { float f; uint32_t u; } imm;
} thc_kop_t;

typedef struct {                       /* UOpKernel, src/tinyhvm.h:702-717 */
    thc_kop_t   ops[THC_KOP_MAX];
    uint32_t    n_ops, n_bufs, n_leaves;
    thc_view_t  leaf_views[THC_MAX_LEAVES];
    uint32_t    leaf_dtypes[THC_MAX_LEAVES];
    uint32_t    coord_uop[THC_MAX_DIM];
    uint32_t    rank;
    thc_shape_t full_shape;
    uint32_t    grid[3], tg[3];
    uint32_t    local_size, reduce_numel, out_dtype;
} thc_uop_kernel_t;

/* ================= vtable entry points (one per Backend slot) ================= */

/* Backend.init / shutdown — src/tinyhvm.h:990-991 (CPU: src/backend/cpu/pool.c:12-13).
 * Device = $THVM_CUDA_DEVICE, else $LOCAL_RANK, else 0.  Returns 0 on success. */
int      thvm_cuda_init(void);
void     thvm_cuda_shutdown(void);

/* Buffers — src/tinyhvm.h:994-1001 (CPU: src/backend/cpu/pool.c:14-17).
 * Ids are small integers handed out in increasing order, 0 = failure.  Fresh
 * buffers read as zero.  `decref` frees at refcount 0 unless id <= the
 * persistent floor. */
uint32_t thvm_cuda_buf_alloc(uint64_t bytes);
void     thvm_cuda_buf_free(uint32_t id);
void     thvm_cuda_buf_incref(uint32_t id);
void     thvm_cuda_buf_decref(uint32_t id);
void     thvm_cuda_mem_checkpoint(uint32_t *leaf_buf_ids, uint32_t n_leaves);
void     thvm_cuda_buf_mark_use(uint32_t id);
void     thvm_cuda_buf_write(uint32_t id, const void *data, uint64_t bytes);
void     thvm_cuda_buf_read(uint32_t id, void *out, uint64_t bytes);

/* Single-op forms — src/tinyhvm.h:1004-1016 (CPU: src/backend/cpu/ops.c:15-130). */
void     thvm_cuda_op_unary(uint32_t uop, uint32_t dst, const thc_view_t *dv, uint32_t dst_dtype,
                            uint32_t src, const thc_view_t *sv, uint32_t src_dtype);
void     thvm_cuda_op_binary(uint32_t uop, uint32_t dst, const thc_view_t *dv, uint32_t dst_dtype,
                             uint32_t a, const thc_view_t *av, uint32_t a_dtype,
                             uint32_t b, const thc_view_t *bv, uint32_t b_dtype);
void     thvm_cuda_op_mm(uint32_t dst, uint32_t dst_dtype,
                         uint32_t a, const thc_view_t *av, uint32_t a_dtype,
                         uint32_t b, const thc_view_t *bv, uint32_t b_dtype,
                         uint32_t M, uint32_t K, uint32_t N);
void     thvm_cuda_op_reduce(uint32_t uop, uint32_t dst, uint32_t dst_numel, uint32_t dst_dtype,
                             uint32_t src, uint32_t src_numel, uint32_t src_dtype, uint32_t reduce_dim);

/* Fused elementwise(+reduce) kernel over strided/broadcast/masked views —
 * src/tinyhvm.h:1019-1025 (CPU: src/backend/cpu/dispatch.c:119-282; caller:
 * src/schedule/_.c:2370-2378).  `leaf_sts` may be NULL; `reduce` may be NULL;
 * side outputs are ignored as in the CPU backend. */
void     thvm_cuda_dispatch_kernel_rs(uint32_t out_buf,
                                      uint32_t *leaf_bufs, const thc_view_t **leaf_views,
                                      const thc_tracker_t *const *leaf_sts, uint32_t n_leaves,
                                      thc_fused_op_t *ops, uint32_t n_ops,
                                      const thc_shape_t *full_shape, const thc_reduce_spec_t *reduce,
                                      uint32_t *side_bufs, const uint32_t *side_op_indices,
                                      uint32_t n_side_outputs,
                                      const uint32_t *leaf_dtypes, uint32_t out_dtype);

/* Lowered KOP program — src/tinyhvm.h:1026-1028 (CPU: src/backend/cpu/uop.c:118-155).
 * Every KOP_LOAD is bounds-checked against the pool's recorded buffer size. */
void     thvm_cuda_dispatch_uop_kernel(uint32_t out_buf, const uint32_t *leaf_bufs, uint32_t n_leaves,
                                       const thc_uop_kernel_t *kernel, uint64_t cache_key);

/* Strided view -> contiguous f32 copy, device-to-device copy, unsynchronised
 * read — src/tinyhvm.h:1029-1031 (callers: src/interact/tensor_ops.c:93-147). */
void     thvm_cuda_contiguify(uint32_t dst_buf, uint32_t numel, uint32_t src_buf, const thc_view_t *src_view);
void     thvm_cuda_buf_copy(uint32_t dst_buf, uint32_t src_buf, uint64_t nbytes);
void     thvm_cuda_buf_read_nosync(uint32_t id, void *out, uint64_t bytes);
/* Extra, no vtable slot: asynchronous read-back on a copy stream of the library's own, ordered after the work
 * already queued; `out` (pinned memory) is valid after thvm_cuda_sync().  Overlaps later uploads and kernels. */
void     thvm_cuda_buf_read_async(uint32_t id, void *out, uint64_t bytes);

/* In-place Adam — src/tinyhvm.h:1033-1035 (math: src/shaders.metal:406-420). */
void     thvm_cuda_adam_step(uint32_t param, uint32_t grad, uint32_t m, uint32_t v,
                             float lr, float beta1, float beta2, float eps,
                             float bc1, float bc2, uint32_t n);

/* Pool — src/tinyhvm.h:1038-1039 (CPU: src/backend/cpu/pool.c:19-26).
 * `pool_reset(keep)` frees ids > keep and rewinds the id counter to keep+1. */
void     thvm_cuda_pool_reset(uint32_t keep);
void     thvm_cuda_pool_set_persistent(uint32_t max_buf);

/* Batching / profiling — src/tinyhvm.h:1041-1045. */
void     thvm_cuda_begin_batch(void);
void     thvm_cuda_end_batch(void);
void     thvm_cuda_profile_report(void);
void     thvm_cuda_profile_reset(void);

/* ================= additions with no vtable slot ================= */

/* Sticky last-error text ("" when none).  The vtable returns void almost
 * everywhere (the reference exits on error); a host can poll this instead. */
const char *thvm_cuda_last_error(void);
void        thvm_cuda_clear_error(void);

/* The backend's CUDA stream (a cudaStream_t) and a blocking wait on it, so a
 * host can time with CUDA events on the launching stream. */
void    *thvm_cuda_stream(void);
void     thvm_cuda_sync(void);
/* Raw device pointer / byte size of a live buffer (NULL / 0 if not live). */
void    *thvm_cuda_buf_ptr(uint32_t id);
uint64_t thvm_cuda_buf_bytes(uint32_t id);
/* Kernel launches issued by this library since init (or the last reset). */
uint64_t thvm_cuda_launch_count(void);
/* Name of the kernel family chosen for the most recent dispatch ("ew_vec4",
 * "reduce_inner", "generic", ...), for tests and profiles. */
const char *thvm_cuda_last_plan(void);
/* Plan selection override for tests: 0 = automatic, 1 = always the generic
 * descriptor-driven kernel. */
void     thvm_cuda_set_force_generic(int on);
/* Number of plans in the signature-keyed cache (a dispatch refused while a step is being
 * captured leaves none behind). */
uint64_t thvm_cuda_plan_count(void);

/* Signature of a dispatch, the same FNV-style mix the reference computes as
 * `normalized_sig` (src/tinyhvm.h:828-856); the plan cache is keyed by it. */
uint64_t thvm_cuda_signature(const thc_fused_op_t *ops, uint32_t n_ops,
                             const thc_view_t *const *leaf_views,
                             const thc_tracker_t *const *leaf_sts, uint32_t n_leaves,
                             const thc_shape_t *full_shape, const thc_reduce_spec_t *reduce);

/* ---- data parallelism (no vtable slot; the reference has no multi-device code, its
 * nearest relative is one context per thread, src/parallel/reduce.c:36-60) ----
 * One process per GPU.  Rank 0 makes a 128-byte token and passes it to the other
 * ranks out of band; every rank calls dp_init after thvm_cuda_init.
 * dp_allreduce_sum adds, across ranks and in place, the first counts[i] floats of
 * each listed buffer (NCCL over NVLink, one group per call, ordered on the
 * backend's stream after the kernels that wrote them).  All return 0 on success. */
int      thvm_cuda_dp_unique_id(void *out128);
int      thvm_cuda_dp_init(int rank, int world, const void *id128);
int      thvm_cuda_dp_world(void);
int      thvm_cuda_dp_rank(void);
int      thvm_cuda_dp_allreduce_sum(const uint32_t *buf_ids, const uint64_t *counts, uint32_t n_bufs);
void     thvm_cuda_dp_shutdown(void);
/* The optimizer step of a data-parallel training step in one call: p_i <- p_i - lr * (sum over ranks of g_i) for the
 * listed parameter / gradient buffers (counts in floats), lr read from the first float of `lr_buf`.  SGD counterpart of
 * Backend.adam_step (src/nn/adam.c:103-118) with the gradient sum folded in; replaces, per parameter tensor, one
 * all-reduce, one `a - b*c` dispatch and the ASSIGN copy (src/interact/tensor_ops.c:93-147).  World 1: one kernel.
 * Several ranks: the gradients travel through an exchange arena each rank creates once (dp_arena_create, after
 * dp_init; sized for the largest sum of counts) and the others map (dp_arena_attach with the 64-byte handle, passed
 * between the rank processes out of band).  Buckets up to 1 MiB with every peer attached: two kernels, each rank adds
 * the peers' packed gradients over NVLink with plain loads, in rank order, so all ranks end with identical
 * parameters; the wait for the peers is bounded (about two seconds; status bit 16 and an untouched parameter set on
 * expiry, reported by thvm_cuda_last_error).  Larger buckets: pack, one ncclAllReduce, update.  0 on success. */
int      thvm_cuda_dp_arena_create(uint64_t max_floats, void *out_handle64);
int      thvm_cuda_dp_arena_attach(int peer_rank, const void *handle64);
int      thvm_cuda_dp_sgd_step(const uint32_t *param_ids, const uint32_t *grad_ids, const uint64_t *counts, uint32_t n_tensors, uint32_t lr_buf);
/* Tests of the bounded wait: the local arena stands in for rank `peer_rank`, which then never publishes a step;
 * poll limit of the wait in units of 100 ns (0 = default). */
int      thvm_cuda_dp_arena_attach_silent(int peer_rank);
void     thvm_cuda_dp_set_poll_limit(uint64_t polls);

/* ---- step capture: record one training step as a CUDA graph, launch it for every later step ----
 * The counterpart of jit_begin_capture / jit_end_capture / jit_replay (src/tinyhvm.h:1294-1300,
 * src/backend/metal/jit.m:24-631).  Between capture_begin and capture_end the vtable calls do their
 * host-side work as usual, but kernels, fills, stream-ordered allocations / frees, copies and NCCL
 * sums are recorded instead of run.  Rules for the captured step:
 *   - it has run eagerly at least once (plans built, library scratch grown);
 *   - it frees every buffer it allocates (a step that ends with pool_reset does) and frees none
 *     that existed before;
 *   - data that differs between steps enters through capture_input (returns the input's index,
 *     -1 on error); host writes made with buf_write are baked into the graph as constants, except
 *     writes above 1 MiB, which count as inputs in call order; the host memory of an input must be
 *     valid at every launch (pinned memory keeps the copy asynchronous);
 *   - buf_read of device data returns zeros while capturing and becomes result k (k counts from 0
 *     in call order), fetched after a launch with graph_result, which waits for the stream.
 * capture_end returns a graph handle >= 1, or 0 with the reason in thvm_cuda_last_error(); nothing of
 * the captured step has run at that point.  graph_launch enqueues the whole step on the backend's
 * stream.  All other functions return 0 on success. */
int      thvm_cuda_capture_begin(void);
int      thvm_cuda_capture_input(uint32_t id, const void *host, uint64_t bytes);
int      thvm_cuda_capture_end(void);
int      thvm_cuda_graph_set_input(int graph, int input, const void *host);
/* Inputs travel host -> device staging -> buffer; the recorded node is the second hop.  graph_set_input uploads `host` on the
 * backend's stream, after the launches already queued and before the next one (the bytes are read when the stream gets
 * there: keep them unchanged until then).  graph_prefetch_input uploads the NEXT launch's bytes on the library's copy
 * stream instead, into another of three staging slots, so the upload overlaps the step that is running; the next
 * graph_launch waits for it and reads from that slot.  A launch with neither call replays the bytes of the one before. */
int      thvm_cuda_graph_prefetch_input(int graph, int input, const void *host);
int      thvm_cuda_graph_launch(int graph);
int      thvm_cuda_graph_result(int graph, int result, void *out, uint64_t bytes);
/* graph_result without the wait: the copy to `out` (pinned host memory) is queued behind the latest launch; `out` is
 * valid once the stream has passed it (record an event on thvm_cuda_stream() after the call, or thvm_cuda_sync). */
int      thvm_cuda_graph_result_async(int graph, int result, void *out, uint64_t bytes);
int      thvm_cuda_graph_counts(int graph, uint32_t *n_inputs, uint32_t *n_results, uint64_t *n_kernels);
/* Node census of the recorded graph: kernel nodes, copy nodes (inputs, staged constants, read-backs), memset nodes
 * (zero-fills), everything else (allocation / free nodes, empty nodes).  0 = ok. */
int      thvm_cuda_graph_nodes(int graph, uint32_t *kernels, uint32_t *copies, uint32_t *memsets, uint32_t *others);
/* For hosts that upload their per-step data with plain buf_write inside the step (the reference's drivers make a fresh
 * tensor per batch): the byte sizes of those uploads, declared before capture_begin.  While capturing, a buf_write of
 * exactly one of these sizes is an input, in call order; every other staged write stays a constant of the step (n = 0
 * clears the list, at most 8 sizes).  graph_input_bytes tells the inputs apart afterwards. */
void     thvm_cuda_capture_input_sizes(const uint64_t *sizes, uint32_t n);
uint64_t thvm_cuda_graph_input_bytes(int graph, int input);
void     thvm_cuda_graph_destroy(int graph);
/* Memory plan of a captured step.  The buffers a captured step allocates are placed at offsets of ONE arena by replaying
 * the step's alloc / free order (liveness) through a first-fit free list — the counterpart of the scheduler's slot plan
 * (src/schedule/_.c:2017-2112) and of the Metal backend's step planner (src/backend/metal/pool.m:225-378) — so the
 * recorded graph contains no allocation or free nodes.  The arena is sized from the peak of the last eager step (which
 * ended with pool_reset); buffers that do not fit fall back to stream-ordered allocations inside the graph.  Reports: arena
 * size, highest offset used, buffers placed in the arena, buffers left to the pool, sum of all bytes requested. */
int      thvm_cuda_graph_memory(int graph, uint64_t *arena_bytes, uint64_t *arena_used, uint32_t *arena_buffers,
                                uint32_t *pool_buffers, uint64_t *bytes_requested);

/* ---- index-producing kernels (integer outputs, bit-exact) ----
 * 2x2 stride-2 max-pool of `planes` contiguous [H, W] f32 planes: values to `out_val`
 * ([planes, H/2, W/2] f32) and, when `out_idx` != 0, the position of the winner inside
 * its window as u8 0..3 in scan order (0,0),(0,1),(1,0),(1,1); strict '>' so the first
 * maximum wins.  Replaces the arithmetic of the reference's max-pool shader
 * (src/shaders.metal:427-458); the value half equals what the RMAX dispatch of
 * thvm_maxpool2d (src/nn/conv.c:484-513) produces.  0 = launched, 1 = bad argument. */
int      thvm_cuda_maxpool2x2_index(uint32_t out_val, uint32_t out_idx, uint32_t x, uint32_t planes, uint32_t H, uint32_t W);
/* Per-row argmax of a contiguous [rows, cols] f32 buffer into u32[rows]: the first index
 * whose value is strictly greater than every earlier one.  Replaces the host loop of
 * thvm_argmax (src/ops/_.c:502-524), which reads the whole tensor back first. */
int      thvm_cuda_argmax_rows(uint32_t out_u32, uint32_t x, uint32_t rows, uint32_t cols);

/* ---- allocation-free variant (no counterpart in the reference) ----
 * out[c] = sum over b and i of x[b][c][i] for a contiguous f32 tensor x[B][C][HW]
 * (the batch-norm channel statistic), computed by the same split reduce kernels
 * as thvm_cuda_dispatch_kernel_rs but without touching any allocator: the
 * partial sums go to a 256 KiB array that is part of the library image, so the
 * call is usable where allocating is forbidden — inside a host that owns all
 * device memory through its own arena, while a step is being recorded for
 * replay, or in a loop that must not stall on an allocator.  `x` and `out` are
 * device pointers owned by the caller, `stream` a cudaStream_t (NULL = default
 * stream).  The library need not be initialised.
 *   - C may not exceed 65536 (the number of partial sums the array holds);
 *     larger shapes are rejected with return code 1 and a message in
 *     thvm_cuda_last_error(); 2 = CUDA error, 3 = bad argument, 0 = launched.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call
 *     before recording a stream.
 *   - All calls on a device share the array and it keeps the previous call's
 *     contents; every slot is rewritten before it is read, so no clearing is
 *     needed, but two calls whose kernels overlap on the GPU (different
 *     streams) race on it — serialise them.
 *   - The first call on a device is not safe against another host thread making
 *     its own first call on that device at the same moment: make one call per
 *     device from one thread before sharing the entry point between threads. */
int      thvm_cuda_channel_sums_noalloc(const float *x, float *out, uint32_t B, uint32_t C, uint32_t HW, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* THVM_CUDA_H */
