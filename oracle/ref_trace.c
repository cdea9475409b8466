/* ref_trace.c — a recording backend for the reference's vtable; included by ref_host.c.
 *
 * TEST / FIXTURE INFRASTRUCTURE.  thvm_init("record") registers a backend that
 * writes every vtable call the reference's host runtime makes (buffer
 * allocation, host writes, dispatch_kernel_rs with all its views and ops,
 * copies, frees, pool resets) to a binary trace and forwards the call to the
 * reference's CPU backend; thvm_init("record-dry") logs without executing the
 * dispatches, which records a full-size training step in seconds (the host
 * program does not branch on tensor values).  The traces are the step programs
 * the product replays against libthvm_cuda.so (tinyhvm_b200/replay.py): the
 * counterpart of the Metal backend's capture/replay of a training step
 * (src/backend/metal/jit.m:24-631).
 *
 * Record layout: u32 op, u32 payload bytes, payload.  Large host writes are not
 * stored; the driver names them (rec_note) and the replayer regenerates them.
 */
#include <stdio.h>

enum { TR_ALLOC = 1, TR_WRITE, TR_READ, TR_DISPATCH, TR_COPY, TR_CONTIGUIFY, TR_FREE, TR_INCREF, TR_DECREF,
       TR_POOL_RESET, TR_SET_PERSISTENT, TR_ALLREDUCE, TR_MARK };
#define TR_INLINE_MAX 8192

static FILE *tr_file = NULL;
static int tr_dry = 0;
static char tr_note[32] = "";
static u64 tr_note_min = 0;

static void tr_rec(u32 op, const void *payload, u32 bytes, const void *extra, u32 extra_bytes) {
    if (!tr_file) return;
    u32 hdr[2] = {op, bytes + extra_bytes};
    fwrite(hdr, 4, 2, tr_file);
    if (bytes) fwrite(payload, 1, bytes, tr_file);
    if (extra_bytes) fwrite(extra, 1, extra_bytes, tr_file);
}

/* name the next host write of at least `min_bytes` bytes; the replayer supplies its data */
void rec_note(const char *name, u64 min_bytes) { if (!tr_file) return; snprintf(tr_note, sizeof tr_note, "%s", name); tr_note_min = min_bytes; }
void rec_mark(const char *name) { char b[32] = {0}; snprintf(b, sizeof b, "%s", name); tr_rec(TR_MARK, b, 32, NULL, 0); }
int rec_open(const char *path) {
    tr_file = fopen(path, "wb");
    if (!tr_file) return 1;
    u32 magic[2] = {0x52544854u /* THTR */, 1};
    fwrite(magic, 4, 2, tr_file);
    return 0;
}
void rec_close(void) { if (tr_file) fclose(tr_file); tr_file = NULL; }

static u32 rec_buf_alloc(u64 bytes) {
    u32 id = cpu_backend.buf_alloc(bytes);
    struct { u32 id; u32 pad; u64 bytes; } r = {id, 0, bytes};
    tr_rec(TR_ALLOC, &r, sizeof r, NULL, 0);
    return id;
}
static void rec_buf_free(u32 id) { tr_rec(TR_FREE, &id, 4, NULL, 0); cpu_backend.buf_free(id); }
static void rec_buf_incref(u32 id) { tr_rec(TR_INCREF, &id, 4, NULL, 0); }
static void rec_buf_decref(u32 id) { tr_rec(TR_DECREF, &id, 4, NULL, 0); }   /* the CPU pool keeps everything until reset */
static void rec_buf_write(u32 id, const void *data, u64 bytes) {
    struct { u32 id; u32 external; u64 bytes; char name[32]; } r;
    memset(&r, 0, sizeof r);
    r.id = id; r.bytes = bytes;
    int named = tr_note[0] && bytes >= tr_note_min;
    if (named) { memcpy(r.name, tr_note, 32); tr_note[0] = 0; }
    r.external = (named || bytes > TR_INLINE_MAX) ? 1 : 0;
    if (r.external && !named) snprintf(r.name, sizeof r.name, "unnamed");
    tr_rec(TR_WRITE, &r, sizeof r, r.external ? NULL : data, r.external ? 0 : (u32)((bytes + 3) & ~3ull));
    cpu_backend.buf_write(id, data, bytes);
}
static void rec_buf_read(u32 id, void *out, u64 bytes) {
    struct { u32 id; u32 pad; u64 bytes; } r = {id, 0, bytes};
    tr_rec(TR_READ, &r, sizeof r, NULL, 0);
    cpu_backend.buf_read(id, out, bytes);
}
static void rec_dispatch_kernel_rs(u32 out_buf, u32 *leaf_bufs, const View **leaf_views, const ShapeTracker *const *leaf_sts,
                                   u32 n_leaves, FusedOp *ops, u32 n_ops, const Shape *full_shape, const ReduceSpec *reduce,
                                   u32 *side_bufs, const u32 *side_op_indices, u32 n_side_outputs,
                                   const u32 *leaf_dtypes, u32 out_dtype) {
    if (tr_file) {
        int has_sts = 0;
        for (u32 i = 0; leaf_sts && i < n_leaves; i++) if (leaf_sts[i] && leaf_sts[i]->n_views >= 2) has_sts = 1;
        size_t cap = 64 + sizeof(Shape) + sizeof(ReduceSpec) + n_leaves * (8 + sizeof(View) + 1 + sizeof(ShapeTracker)) + n_ops * sizeof(FusedOp);
        u8 *b = malloc(cap), *w = b;
        u32 head[6] = {out_buf, n_leaves, n_ops, out_dtype, reduce && reduce->reduce_type ? 1u : 0u, (u32)has_sts};
        memcpy(w, head, sizeof head); w += sizeof head;
        memcpy(w, full_shape, sizeof(Shape)); w += sizeof(Shape);
        ReduceSpec rs; memset(&rs, 0, sizeof rs); if (reduce) rs = *reduce;
        memcpy(w, &rs, sizeof rs); w += sizeof rs;
        memcpy(w, leaf_bufs, 4 * n_leaves); w += 4 * n_leaves;
        for (u32 i = 0; i < n_leaves; i++) { u32 dt = leaf_dtypes ? leaf_dtypes[i] : DTYPE_F32; memcpy(w, &dt, 4); w += 4; }
        for (u32 i = 0; i < n_leaves; i++) { memcpy(w, leaf_views[i], sizeof(View)); w += sizeof(View); }
        memcpy(w, ops, n_ops * sizeof(FusedOp)); w += n_ops * sizeof(FusedOp);
        if (has_sts)
            for (u32 i = 0; i < n_leaves; i++) {
                u8 present = leaf_sts[i] && leaf_sts[i]->n_views >= 2;
                *w++ = present;
                if (present) { memcpy(w, leaf_sts[i], sizeof(ShapeTracker)); w += sizeof(ShapeTracker); }
            }
        tr_rec(TR_DISPATCH, b, (u32)(w - b), NULL, 0);
        free(b);
    }
    if (!tr_dry)
        cpu_backend.dispatch_kernel_rs(out_buf, leaf_bufs, leaf_views, leaf_sts, n_leaves, ops, n_ops, full_shape, reduce,
                                       side_bufs, side_op_indices, n_side_outputs, leaf_dtypes, out_dtype);
}
/* the ASSIGN rule copies through these two (src/interact/tensor_ops.c:113-121); the CPU backend has neither,
 * so they are carried out on the CPU pool directly */
static void rec_buf_copy(u32 dst, u32 src, u64 nbytes) {
    struct { u32 dst, src; u64 bytes; } r = {dst, src, nbytes};
    tr_rec(TR_COPY, &r, sizeof r, NULL, 0);
    memcpy(cpu_pool.bufs[dst], cpu_pool.bufs[src], nbytes);
}
static void rec_pool_reset(u32 keep) { tr_rec(TR_POOL_RESET, &keep, 4, NULL, 0); cpu_backend.pool_reset(keep); }
static void rec_pool_set_persistent(u32 m) { tr_rec(TR_SET_PERSISTENT, &m, 4, NULL, 0); }
static int rec_init(void) { return 0; }

static Backend rec_backend = {
    .init = rec_init, .buf_alloc = rec_buf_alloc, .buf_free = rec_buf_free, .buf_incref = rec_buf_incref,
    .buf_decref = rec_buf_decref, .buf_write = rec_buf_write, .buf_read = rec_buf_read,
    .dispatch_kernel_rs = rec_dispatch_kernel_rs, .buf_copy = rec_buf_copy,
    .pool_reset = rec_pool_reset, .pool_set_persistent = rec_pool_set_persistent,
};

/* gradient all-reduce as a trace record (the DP hook of a recording run) */
static int rec_dp_hook(const u32 *buf_ids, const u64 *counts, u32 n) {
    u8 b[4 + 32 * 12];
    memcpy(b, &n, 4); memcpy(b + 4, buf_ids, 4 * n); memcpy(b + 4 + 4 * n, counts, 8 * n);
    tr_rec(TR_ALLREDUCE, b, 4 + 12 * n, NULL, 0);
    return 0;
}
