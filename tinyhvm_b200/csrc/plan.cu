// plan.cu — the compute entry points of the vtable: validate a dispatch on the
// host, find (or build and cache) its plan by signature, launch.
//
// The plan cache plays the role of the reference's kernel cache keyed by
// `normalized_sig` (docs/kernel_cache.md; Metal: src/backend/metal/codegen.m:8-24,
// 768-827): the key is the same FNV-style mix over ops, iteration shape, reduce
// spec and every leaf view/tracker (src/tinyhvm.h:766-856), extended by the
// dtypes, which select different load/store code here.
#include <string.h>
#include <unordered_map>
#include <vector>
#include "gen_desc.h"
#include "plans.h"
#include "device_common.cuh"
#include "state.h"

namespace thc {

// ---------------- signature ----------------
static inline uint64_t mix(uint64_t h, uint64_t v) { return (h ^ v) * 0x100000001b3ULL; }

static uint64_t sig_view(uint64_t h, const thc_view_t *v) {
    if (!v) return mix(h, 0);
    h = mix(h, v->shape.rank);
    h = mix(h, v->numel);
    h = mix(h, (uint64_t)(uint32_t)v->offset);
    h = mix(h, v->has_mask);
    for (uint32_t d = 0; d < v->shape.rank && d < THC_MAX_DIM; d++) {
        h = mix(h, v->shape.dims[d]);
        h = mix(h, (uint64_t)(uint32_t)v->strides[d]);
        if (v->has_mask) { h = mix(h, v->mask_begin[d]); h = mix(h, v->mask_end[d]); }
        h = mix(h, v->mod_size[d]);
    }
    h = mix(h, v->n_compound_masks);
    for (uint32_t i = 0; i < v->n_compound_masks && i < 2; i++) {
        h = mix(h, v->compound_masks[i].dim_a);
        h = mix(h, v->compound_masks[i].dim_b);
        h = mix(h, (uint64_t)(uint32_t)v->compound_masks[i].stride_a);
        h = mix(h, v->compound_masks[i].begin);
        h = mix(h, v->compound_masks[i].end);
    }
    return h;
}

static uint64_t signature(const thc_fused_op_t *ops, uint32_t n_ops, const thc_view_t *const *views,
                          const thc_tracker_t *const *sts, uint32_t n_leaves,
                          const thc_shape_t *full, const thc_reduce_spec_t *red) {
    uint64_t h = 0x5448564d4b45524eULL;
    h = mix(h, n_ops);
    h = mix(h, n_leaves);
    for (uint32_t i = 0; i < n_ops; i++) {
        h = mix(h, ops[i].uop); h = mix(h, ops[i].arg_a); h = mix(h, ops[i].arg_b); h = mix(h, ops[i].aux);
    }
    if (!full) h = mix(h, 0);
    else {
        h = mix(h, full->rank);
        for (uint32_t d = 0; d < full->rank && d < THC_MAX_DIM; d++) h = mix(h, full->dims[d]);
    }
    if (!red) h = mix(h, 0);
    else {
        h = mix(h, red->reduce_type); h = mix(h, red->post_reduce_start); h = mix(h, red->n_post_leaves);
        h = mix(h, red->reduce2_type); h = mix(h, red->reduce2_start);
        for (uint32_t d = 0; d < THC_MAX_DIM; d++) { h = mix(h, red->is_reduce[d]); h = mix(h, red->is_reduce2[d]); }
    }
    for (uint32_t i = 0; i < n_leaves; i++) {
        const thc_view_t *v = views ? views[i] : nullptr;
        const thc_tracker_t *st = sts ? sts[i] : nullptr;
        if (!st || st->n_views == 0) h = sig_view(h, v);
        else {
            h = mix(h, st->n_views);
            for (uint32_t k = 0; k < st->n_views && k < THC_MAX_VIEWS; k++) h = sig_view(h, &st->views[k]);
        }
    }
    h = mix(h, 0);   // no side outputs
    return h;
}

// ---------------- plan cache ----------------
static std::unordered_map<uint64_t, Plan *> *cache = nullptr;

static void plan_free(Plan *p) {
    if (p->dev_desc) cudaFreeAsync(p->dev_desc, g.stream);
    if (p->dev_trackers) cudaFreeAsync(p->dev_trackers, g.stream);
    free_fast(p);
    delete p;
}


// Build the host descriptor; returns false (with the error set) if the
// dispatch is malformed.
static bool build_desc(Plan *p, const thc_view_t **views, const thc_tracker_t *const *sts, uint32_t n_leaves,
                       const thc_fused_op_t *ops, uint32_t n_ops, const thc_shape_t *full,
                       const thc_reduce_spec_t *red, const uint32_t *leaf_dtypes, uint32_t out_dtype) {
    GenDesc &D = p->host;
    memset(&D, 0, sizeof D);
    uint32_t rank = full->rank ? full->rank : 1;
    if (rank > THC_MAX_DIM) { set_error("dispatch: rank %u > %d", rank, THC_MAX_DIM); return false; }
    if (n_leaves > THC_MAX_LEAVES || n_ops > THC_MAX_OPS) { set_error("dispatch: %u leaves / %u ops exceed 64", n_leaves, n_ops); return false; }
    if (n_leaves == 0) { set_error("dispatch: no leaves"); return false; }
    D.n_leaves = n_leaves; D.n_ops = n_ops; D.rank = rank; D.out_dtype = out_dtype;
    D.has_reduce = (red && red->reduce_type) ? 1 : 0;
    D.reduce_type = D.has_reduce ? red->reduce_type : 0;
    if (D.has_reduce && D.reduce_type != THC_SUM && D.reduce_type != THC_RMAX) {
        set_error("dispatch: reduce type %u is neither SUM nor RMAX", D.reduce_type); return false;
    }
    D.full_numel = 1; D.out_numel = 1; D.reduce_numel = 1;
    for (uint32_t d = 0; d < rank; d++) {
        uint32_t dim = full->dims[d];
        D.full_dims[d] = dim;
        bool r = D.has_reduce && red->is_reduce[d];
        D.out_dims[d] = r ? 1 : dim;
        D.full_numel *= dim;
        if (r) { D.reduce_numel *= dim; D.rdim[D.n_rdims++] = d; }
        else   { D.out_numel *= dim;    D.kdim[D.n_kdims++] = d; }
    }
    D.post_start = D.has_reduce ? red->post_reduce_start : 0;
    D.n_post_leaves = D.has_reduce ? red->n_post_leaves : 0;
    if (D.post_start > n_ops) { set_error("dispatch: post_reduce_start %u > %u ops", D.post_start, n_ops); return false; }
    if (D.n_post_leaves > n_leaves) { set_error("dispatch: %u post-reduce leaves > %u leaves", D.n_post_leaves, n_leaves); return false; }
    const uint32_t n_eval = D.post_start ? D.post_start : n_ops;
    for (uint32_t i = 0; i < n_ops; i++) {
        D.ops[i] = ops[i];
        // operands must name a leaf or an earlier op of the same phase window
        uint32_t lim = n_leaves + (i < n_eval ? n_eval : n_ops);
        if (ops[i].arg_a >= lim || ops[i].arg_b >= lim) {
            set_error("dispatch: op %u reads value %u/%u beyond %u", i, ops[i].arg_a, ops[i].arg_b, lim - 1);
            return false;
        }
    }
    std::vector<DTracker> trackers;
    for (uint32_t i = 0; i < n_leaves; i++) {
        DLeaf &L = D.leaves[i];
        L.dtype = leaf_dtypes ? leaf_dtypes[i] : THC_F32;
        L.tracker = -1;
        const thc_tracker_t *st = sts ? sts[i] : nullptr;
        if (st && st->n_views >= 2) {
            DTracker t; memset(&t, 0, sizeof t);
            t.n_views = st->n_views > THC_MAX_VIEWS ? THC_MAX_VIEWS : st->n_views;
            for (uint32_t k = 0; k < t.n_views; k++) dview_from(t.views[k], st->views[k]);
            L.tracker = (int32_t)trackers.size();
            trackers.push_back(t);
            if (views && views[i]) dview_from(L.v, *views[i]);
        } else {
            if (!views || !views[i]) { set_error("dispatch: leaf %u has no view", i); return false; }
            dview_from(L.v, *views[i]);
        }
    }
    p->n_trackers = (uint32_t)trackers.size();
    if (!trackers.empty()) {
        uint64_t bytes = trackers.size() * sizeof(DTracker);
        THC_CUDA_OK(cudaMallocAsync((void **)&p->dev_trackers, bytes, g.stream));   // never inside a capture: the caller refuses first
        THC_CUDA_OK(cudaMemcpyAsync(p->dev_trackers, trackers.data(), bytes, cudaMemcpyHostToDevice, g.stream));
        THC_CUDA_OK(cudaStreamSynchronize(g.stream));        // `trackers` dies with this scope
        D.trackers = p->dev_trackers;
    }
    return true;
}

// What profile_report divides the measured time into: the Metal backend estimates out_numel * reduce_numel * n_ops
// operations and (n_leaves * iteration points + outputs) * 4 bytes (src/backend/metal/codegen.m:1023-1031); here the
// bytes are the algorithmic ones, each leaf counted over the dims it actually walks, in its own dtype.
static void estimate(Plan *p) {
    const GenDesc &D = p->host;
    p->est_ops = D.full_numel * (unsigned long long)((D.n_ops ? D.n_ops : 1) + (D.has_reduce ? 1 : 0));
    p->est_out_bytes = (D.has_reduce ? D.out_numel : D.full_numel) * dtype_bytes(D.out_dtype);
    for (uint32_t i = 0; i < D.n_leaves; i++) {
        const DLeaf &L = D.leaves[i];
        unsigned long long n = 1;
        if (L.tracker >= 0) n = D.full_numel;       // stacked views: no cheap bound, count every point
        else for (uint32_t d = 0; d < D.rank && d < L.v.rank; d++) {
            if (L.v.strides[d] == 0 || L.v.dims[d] <= 1) continue;
            uint32_t ext = L.v.dims[d] < D.full_dims[d] ? L.v.dims[d] : D.full_dims[d];
            if (L.v.has_mask && L.v.me[d] > L.v.mb[d] && L.v.me[d] - L.v.mb[d] < ext) ext = L.v.me[d] - L.v.mb[d];
            n *= ext;
        }
        p->est_leaf_bytes[i] = n * dtype_bytes(L.dtype);
    }
}

// The device copy of the descriptor, made the first time the generic kernel runs the plan.  Memory allocated while a
// step is being recorded would belong to the recorded graph, so inside a capture this refuses instead (false).
static bool ensure_dev_desc(Plan *p) {
    if (p->dev_desc) return true;
    if (capturing()) {
        capture_fail("a dispatch met the descriptor-driven kernel for the first time inside the captured step: run the step once before capturing it");
        return false;
    }
    THC_CUDA_OK(cudaMallocAsync((void **)&p->dev_desc, sizeof(GenDesc), g.stream));
    upload_small(p->dev_desc, &p->host, sizeof(GenDesc));
    return true;
}

void launch_generic(const GenDesc &H, const GenDesc *dev_desc, const GenArgs &args);   // generic.cu

}  // namespace thc

using namespace thc;

extern "C" {

// number of cached plans (tests: a dispatch refused inside a capture must leave none behind)
uint64_t thvm_cuda_plan_count(void) { return cache ? (uint64_t)cache->size() : 0; }

void plan_cache_clear(void) {
    if (!cache) return;
    for (auto &kv : *cache) plan_free(kv.second);
    cache->clear();
}

uint64_t thvm_cuda_signature(const thc_fused_op_t *ops, uint32_t n_ops, const thc_view_t *const *leaf_views,
                             const thc_tracker_t *const *leaf_sts, uint32_t n_leaves,
                             const thc_shape_t *full_shape, const thc_reduce_spec_t *reduce) {
    return signature(ops, n_ops, leaf_views, leaf_sts, n_leaves, full_shape, reduce);
}

void thvm_cuda_dispatch_kernel_rs(uint32_t out_buf, uint32_t *leaf_bufs, const thc_view_t **leaf_views,
                                  const thc_tracker_t *const *leaf_sts, uint32_t n_leaves,
                                  thc_fused_op_t *ops, uint32_t n_ops, const thc_shape_t *full_shape,
                                  const thc_reduce_spec_t *reduce, uint32_t *side_bufs,
                                  const uint32_t *side_op_indices, uint32_t n_side_outputs,
                                  const uint32_t *leaf_dtypes, uint32_t out_dtype) {
    (void)side_bufs; (void)side_op_indices; (void)n_side_outputs;   // ignored by the CPU backend too (dispatch.c:126)
    if (!g.ready) fatal("dispatch_kernel_rs: backend not initialised (no CUDA device?)");
    if (!full_shape) { set_error("dispatch: no iteration shape"); return; }
    if (n_leaves > THC_MAX_LEAVES || n_ops > THC_MAX_OPS) { set_error("dispatch: %u leaves / %u ops exceed 64", n_leaves, n_ops); return; }
    const thc_reduce_spec_t *red = (reduce && reduce->reduce_type) ? reduce : nullptr;

    uint64_t key = signature(ops, n_ops, leaf_views, leaf_sts, n_leaves, full_shape, red);
    key = mix(key, out_dtype);
    for (uint32_t i = 0; i < n_leaves; i++) key = mix(key, leaf_dtypes ? leaf_dtypes[i] : THC_F32);
    key = mix(key, (uint64_t)g.force_generic);

    if (!cache) cache = new std::unordered_map<uint64_t, Plan *>();
    Plan *p = nullptr;
    auto it = cache->find(key);
    if (it != cache->end()) p = it->second;
    else {
        // Building a plan allocates device tables and waits for their upload; neither can happen while the stream is
        // recording.  The step is refused before anything is allocated, and nothing enters the cache.
        if (capturing()) { capture_fail("a plan was built inside the captured step: run the step once before capturing it"); return; }
        p = new Plan();
        if (!build_desc(p, leaf_views, leaf_sts, n_leaves, ops, n_ops, full_shape, red, leaf_dtypes, out_dtype)) {
            plan_free(p);
            return;
        }
        p->kind = PLAN_GENERIC;
        if (!g.force_generic) classify_plan(p);
        estimate(p);
        (*cache)[key] = p;
    }

    GenArgs args;
    for (uint32_t i = 0; i < n_leaves; i++) {
        Buf &lb = buf_checked(leaf_bufs[i], "dispatch(leaf)");
        args.leaf[i] = lb.ptr;
        args.cap[i] = lb.bytes / dtype_bytes(p->host.leaves[i].dtype);
        if (g.profile) g.prof_bytes = (i ? g.prof_bytes : p->est_out_bytes) + (p->est_leaf_bytes[i] < lb.bytes ? p->est_leaf_bytes[i] : lb.bytes);
    }
    if (g.profile) g.prof_ops = p->est_ops;
    uint64_t need_out = p->host.has_reduce ? p->host.out_numel : p->host.full_numel;
    Buf &ob = buf_for_output(out_buf, "dispatch(out)", need_out * dtype_bytes(p->host.out_dtype));   // after the leaves: out may alias one
    args.out = ob.ptr;
    args.out_cap = ob.bytes / dtype_bytes(p->host.out_dtype);
    args.status = g.dev_status;
    mark_device_written(out_buf);

    if (need_out > args.out_cap) {
        set_error("dispatch: output buffer %u holds %llu elements, kernel writes %llu", out_buf,
                  (unsigned long long)args.out_cap, (unsigned long long)need_out);
        return;
    }
    if (p->kind != PLAN_GENERIC && launch_fast(p, args)) return;
    if (!ensure_dev_desc(p)) return;
    launch_generic(p->host, p->dev_desc, args);
}

// ---- single-op forms, expressed as one-op fused dispatches ----
static void contiguous_view(thc_view_t *v, const uint32_t *dims, uint32_t rank) {
    memset(v, 0, sizeof *v);
    v->shape.rank = rank;
    uint32_t n = 1;
    for (uint32_t d = 0; d < rank; d++) { v->shape.dims[d] = dims[d]; n *= dims[d]; }
    int32_t s = 1;
    for (int d = (int)rank - 1; d >= 0; d--) { v->strides[d] = dims[d] == 1 ? 0 : s; s *= (int32_t)dims[d]; }
    v->numel = n; v->contiguous = 1;
}

static bool same_shape(const thc_view_t *a, const thc_view_t *b) {
    if (a->shape.rank != b->shape.rank) return false;
    for (uint32_t d = 0; d < a->shape.rank; d++) if (a->shape.dims[d] != b->shape.dims[d]) return false;
    return true;
}

// The CPU forms address a source by decomposing the flat output index over
// the source view's own shape and ignore masks (src/backend/cpu/ops.c:4-13).
// With equal shapes that is plain coordinate addressing; otherwise the same
// arithmetic is a two-view tracker (iteration space -> source shape).
static void as_leaf(const thc_view_t *src, const thc_view_t *iter, thc_view_t *view_out, thc_tracker_t *st_out, bool *use_st) {
    *view_out = *src;
    view_out->has_mask = 0; view_out->n_compound_masks = 0;
    *use_st = !same_shape(src, iter);
    if (*use_st) {
        memset(st_out, 0, sizeof *st_out);
        st_out->n_views = 2;
        st_out->views[0] = *view_out;
        contiguous_view(&st_out->views[1], iter->shape.dims, iter->shape.rank);
    }
}

void thvm_cuda_op_unary(uint32_t uop, uint32_t dst, const thc_view_t *dv, uint32_t dst_dtype,
                        uint32_t src, const thc_view_t *sv, uint32_t src_dtype) {
    // iterate dv->numel outputs; the source is addressed through its own shape
    thc_view_t iter, lv; thc_tracker_t st; bool use_st;
    if (dv->numel == sv->numel) contiguous_view(&iter, sv->shape.dims, sv->shape.rank);
    else { uint32_t n = dv->numel; contiguous_view(&iter, &n, 1); }
    as_leaf(sv, &iter, &lv, &st, &use_st);
    thc_fused_op_t op = {uop, 0, 0, 0};
    bool is_op = uop == THC_NEG || uop == THC_RELU || uop == THC_EXP || uop == THC_LOG || uop == THC_SQRT;
    const thc_view_t *views[1] = {&lv};
    const thc_tracker_t *sts[1] = {&st};
    uint32_t bufs[1] = {src}, dts[1] = {src_dtype};
    thvm_cuda_dispatch_kernel_rs(dst, bufs, views, use_st ? sts : nullptr, 1, &op, is_op ? 1 : 0, &iter.shape,
                                 nullptr, nullptr, nullptr, 0, dts, dst_dtype);
}

void thvm_cuda_op_binary(uint32_t uop, uint32_t dst, const thc_view_t *dv, uint32_t dst_dtype,
                         uint32_t a, const thc_view_t *av, uint32_t a_dtype,
                         uint32_t b, const thc_view_t *bv, uint32_t b_dtype) {
    thc_view_t iter, la, lb; thc_tracker_t sa, sb; bool ua, ub;
    contiguous_view(&iter, dv->shape.dims, dv->shape.rank);
    as_leaf(av, &iter, &la, &sa, &ua);
    as_leaf(bv, &iter, &lb, &sb, &ub);
    bool is_op = uop == THC_ADD || uop == THC_MUL || uop == THC_DIV || uop == THC_SUB || uop == THC_MAX || uop == THC_CMP;
    thc_fused_op_t op = {uop, 0, 1, 0};
    const thc_view_t *views[2] = {&la, &lb};
    const thc_tracker_t *sts[2] = {ua ? &sa : nullptr, ub ? &sb : nullptr};
    uint32_t bufs[2] = {a, b}, dts[2] = {a_dtype, b_dtype};
    thvm_cuda_dispatch_kernel_rs(dst, bufs, views, (ua || ub) ? sts : nullptr, 2, &op, is_op ? 1 : 0, &iter.shape,
                                 nullptr, nullptr, nullptr, 0, dts, dst_dtype);
}

void thvm_cuda_op_mm(uint32_t dst, uint32_t dst_dtype, uint32_t a, const thc_view_t *av, uint32_t a_dtype,
                     uint32_t b, const thc_view_t *bv, uint32_t b_dtype, uint32_t M, uint32_t K, uint32_t N) {
    // C[i,j] = sum_k A[i,k] * B[k,j] (src/backend/cpu/ops.c:99-112) as the
    // [M,K,N] MUL + SUM{1} contraction the lazy path also produces
    // (src/ctx/init.c:555-582).
    if (av->shape.rank != 2 || bv->shape.rank != 2 || av->shape.dims[0] != M || av->shape.dims[1] != K ||
        bv->shape.dims[0] != K || bv->shape.dims[1] != N) {
        set_error("op_mm: operand views must be rank-2 [M,K] and [K,N]");
        return;
    }
    uint32_t dims[3] = {M, K, N};
    thc_view_t la, lb;
    uint32_t da[3] = {M, K, 1}, db[3] = {1, K, N};
    contiguous_view(&la, da, 3); contiguous_view(&lb, db, 3);
    la.strides[0] = av->strides[0]; la.strides[1] = av->strides[1]; la.strides[2] = 0; la.offset = av->offset;
    lb.strides[0] = 0; lb.strides[1] = bv->strides[0]; lb.strides[2] = bv->strides[1]; lb.offset = bv->offset;
    la.contiguous = lb.contiguous = 0;
    thc_shape_t full; memset(&full, 0, sizeof full); full.rank = 3; memcpy(full.dims, dims, sizeof dims);
    thc_reduce_spec_t red; memset(&red, 0, sizeof red); red.is_reduce[1] = 1; red.reduce_type = THC_SUM;
    thc_fused_op_t op = {THC_MUL, 0, 1, 0};
    const thc_view_t *views[2] = {&la, &lb};
    uint32_t bufs[2] = {a, b}, dts[2] = {a_dtype, b_dtype};
    thvm_cuda_dispatch_kernel_rs(dst, bufs, views, nullptr, 2, &op, 1, &full, &red, nullptr, nullptr, 0, dts, dst_dtype);
}

void thvm_cuda_op_reduce(uint32_t uop, uint32_t dst, uint32_t dst_numel, uint32_t dst_dtype,
                         uint32_t src, uint32_t src_numel, uint32_t src_dtype, uint32_t reduce_dim) {
    (void)src_numel;
    if (uop != THC_SUM && uop != THC_RMAX) { set_error("op_reduce: uop %u is neither SUM nor RMAX", uop); return; }
    uint32_t dims[2] = {dst_numel, reduce_dim};
    thc_view_t lv; contiguous_view(&lv, dims, 2);
    thc_shape_t full; memset(&full, 0, sizeof full); full.rank = 2; full.dims[0] = dst_numel; full.dims[1] = reduce_dim;
    thc_reduce_spec_t red; memset(&red, 0, sizeof red); red.is_reduce[1] = 1; red.reduce_type = uop;
    const thc_view_t *views[1] = {&lv};
    uint32_t bufs[1] = {src}, dts[1] = {src_dtype};
    thvm_cuda_dispatch_kernel_rs(dst, bufs, views, nullptr, 1, nullptr, 0, &full, &red, nullptr, nullptr, 0, dts, dst_dtype);
}

void thvm_cuda_contiguify(uint32_t dst_buf, uint32_t numel, uint32_t src_buf, const thc_view_t *src_view) {
    // The slot carries no dtype (src/tinyhvm.h:1029); its only caller requires
    // equal source and destination dtypes (src/interact/tensor_ops.c:118-120),
    // so the element width is taken from the destination's size.
    Buf &d = buf_checked(dst_buf, "contiguify(dst)");
    uint32_t dt = (numel && d.bytes == (uint64_t)numel * 2) ? THC_F16 : THC_F32;
    const thc_view_t *views[1] = {src_view};
    uint32_t bufs[1] = {src_buf}, dts[1] = {dt};
    thvm_cuda_dispatch_kernel_rs(dst_buf, bufs, views, nullptr, 1, nullptr, 0, &src_view->shape, nullptr,
                                 nullptr, nullptr, 0, dts, dt);
}

}  // extern "C"
