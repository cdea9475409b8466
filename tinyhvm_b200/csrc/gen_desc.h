// gen_desc.h — device-resident description of one fused kernel, as consumed by
// the descriptor-driven ("generic") kernels.  One descriptor is built per
// distinct dispatch signature and cached; per-launch data (buffer pointers and
// capacities) travels as kernel parameters.
#pragma once
#include <stdint.h>
#include "../../include/thvm_cuda.h"

namespace thc {

struct DView {                       // one View, trimmed to what indexing needs
    uint32_t rank;
    uint32_t dims[THC_MAX_DIM];
    int32_t  strides[THC_MAX_DIM];
    int32_t  offset;
    uint32_t has_mask;
    uint32_t n_cm;
    uint32_t mb[THC_MAX_DIM], me[THC_MAX_DIM];
    struct { uint32_t da, db; int32_t sa; uint32_t begin, end; } cm[2];
};

struct DTracker { uint32_t n_views; DView views[THC_MAX_VIEWS]; };

struct DLeaf {
    DView    v;
    uint32_t dtype;
    int32_t  tracker;                // index into GenDesc::trackers, or -1
};

struct GenDesc {
    uint32_t n_leaves, n_ops, rank;
    uint32_t full_dims[THC_MAX_DIM];
    uint32_t out_dims[THC_MAX_DIM];  // reduced dims collapsed to 1
    uint32_t has_reduce, reduce_type;
    uint32_t n_kdims, kdim[THC_MAX_DIM];   // kept dims, outermost first
    uint32_t n_rdims, rdim[THC_MAX_DIM];   // reduced dims, outermost first
    uint32_t post_start, n_post_leaves;
    uint32_t out_dtype;
    uint64_t full_numel, out_numel, reduce_numel;
    thc_fused_op_t ops[THC_MAX_OPS];
    DLeaf    leaves[THC_MAX_LEAVES];
    const DTracker *trackers;        // device pointer (may be null)
};

struct GenArgs {                     // kernel parameters
    void       *out;
    uint64_t    out_cap;             // elements
    const void *leaf[THC_MAX_LEAVES];
    uint64_t    cap[THC_MAX_LEAVES]; // elements
    int        *status;
};

// host side: fill a DView from a reference-layout view
inline void dview_from(DView &d, const thc_view_t &v) {
    d.rank = v.shape.rank > THC_MAX_DIM ? THC_MAX_DIM : v.shape.rank;
    for (int i = 0; i < THC_MAX_DIM; i++) {
        d.dims[i] = v.shape.dims[i]; d.strides[i] = v.strides[i];
        d.mb[i] = v.mask_begin[i];   d.me[i] = v.mask_end[i];
    }
    d.offset = v.offset;
    d.has_mask = v.has_mask ? 1u : 0u;
    d.n_cm = v.n_compound_masks > 2 ? 2u : v.n_compound_masks;
    for (int i = 0; i < 2; i++) {
        d.cm[i].da = v.compound_masks[i].dim_a; d.cm[i].db = v.compound_masks[i].dim_b;
        d.cm[i].sa = v.compound_masks[i].stride_a;
        d.cm[i].begin = v.compound_masks[i].begin; d.cm[i].end = v.compound_masks[i].end;
    }
}

}  // namespace thc
