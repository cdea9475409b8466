// plans.h — a cached plan for one dispatch signature: which kernel family
// runs it and the family's precomputed parameters.
#pragma once
#include "gen_desc.h"

namespace thc {

enum PlanKind : int {
    PLAN_GENERIC = 0,   // descriptor-driven interpreter (generic.cu)
    PLAN_EW,            // collapsed-dims elementwise, vectorised inner dim (ew.cu)
    PLAN_REDUCE,        // collapsed-dims reduce (reduce.cu)
    PLAN_CONTRACT,      // SUM(MUL(a,b)) with separable operands -> GEMM (gemm.cu)
    PLAN_POOL,          // RMAX over the 2x2 windows of contiguous planes -> pooling kernel (uop.cu)
    PLAN_POOL_BWD,      // the mask-form gradient of that pool -> pooling backward kernel (uop.cu)
    PLAN_PAD2D,         // padding of contiguous planes materialised (layout.cu)
    PLAN_WIN2PLANE,     // 2x2-window layout copied back to plane layout (layout.cu)
    PLAN_CROP2D,        // a window cut out of every plane of a larger pitch (layout.cu)
};

struct FastDesc;        // family-specific, defined in fast_desc.h

struct Plan {
    int        kind = PLAN_GENERIC;
    GenDesc    host;                    // full description (host copy)
    GenDesc   *dev_desc = nullptr;      // uploaded lazily, only if the generic kernel runs
    DTracker  *dev_trackers = nullptr;
    uint32_t   n_trackers = 0;
    FastDesc  *fast = nullptr;          // owned; null for PLAN_GENERIC
    void      *contract = nullptr;      // owned (gemm.cu); set for PLAN_CONTRACT
    unsigned long long pool_planes = 0; // PLAN_POOL: contiguous [planes, pool_h, pool_w] input starting at element pool_off
    uint32_t   pool_h = 0, pool_w = 0;
    long long  pool_off = 0, pool_g_off = 0, pool_m_off = 0, pool_one_off = 0;
    // estimates for profile_report: op evaluations (reduce accumulation counted as one op) and algorithmic bytes
    // (every leaf element addressed once: dims walked with stride 0 do not count, and a leaf never counts for more than
    // its buffer holds, which is what overlapping convolution windows come to; plus the output)
    unsigned long long est_ops = 0, est_out_bytes = 0, est_leaf_bytes[THC_MAX_LEAVES] = {};
};

// Decide the family for a freshly built plan (sets kind / fast).
void classify_plan(Plan *p);
// Launch a non-generic plan; false means "could not, use the generic kernel".
bool launch_fast(Plan *p, const GenArgs &args);
void free_fast(Plan *p);
// SUM(MUL(a,b)) with separable operands -> tensor-core contraction (gemm.cu)
bool try_contraction(Plan *p);
bool launch_contraction(Plan *p, const GenArgs &args);
void free_contraction(Plan *p);
// RMAX over 2x2 stride-2 windows of contiguous planes -> pooling kernel (uop.cu)
bool try_pool2x2(Plan *p);
bool launch_pool2x2(Plan *p, const GenArgs &args);
bool try_pool2x2_bwd(Plan *p);
bool launch_pool2x2_bwd(Plan *p, const GenArgs &args);
// layout-changing copies (layout.cu)
bool try_pad2d(Plan *p);
bool launch_pad2d(Plan *p, const GenArgs &args);
bool try_crop2d(Plan *p);
bool launch_crop2d(Plan *p, const GenArgs &args);
bool try_window_to_plane(Plan *p);
bool launch_window_to_plane(Plan *p, const GenArgs &args);

}  // namespace thc
