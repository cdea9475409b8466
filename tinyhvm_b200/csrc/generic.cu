// generic.cu — the descriptor-driven kernels: correct for every dispatch the
// reference can emit (rank <= 8, <= 64 leaves, <= 64 ops, stride-0 broadcast,
// negative offsets, per-dim and compound masks, stacked views, all dtypes,
// post-reduce ops), at the price of interpreting the op list per element.
// The specialised families (ew.cu, reduce.cu, ...) take the hot shapes; this
// file is what everything else runs on, and what they are checked against.
//
// Semantics restated from the reference's CPU backend:
//   leaf addressing    src/backend/cpu/dispatch.c:88-117  (single view)
//                      src/backend/cpu/dispatch.c:26-85   (stacked views)
//   op evaluation      src/backend/cpu/dispatch.c:188-199
//   reduce / store     src/backend/cpu/dispatch.c:148-151, 202-217
//   post-reduce phase  src/backend/cpu/dispatch.c:222-281
// Differences on purpose: indices are 64-bit (the CPU's u32 iteration count
// wraps at 2^32 points), every load is checked against the buffer's size
// (out of range reads give 0 and raise a status bit instead of faulting), and
// a SUM with more than 64 terms per output is accumulated by a warp or a CTA
// in tree order instead of strictly left to right.
#include "device_common.cuh"
#include "gen_desc.h"
#include "state.h"

namespace thc {

__device__ __forceinline__ float checked_load(const void *buf, uint32_t dt, int64_t idx, uint64_t cap, int *status) {
    if (idx < 0) return 0.0f;
    if ((uint64_t)idx >= cap) { atomicOr(status, ERR_LOAD_OOB); return 0.0f; }
    return load_as_f32(buf, dt, (uint64_t)idx);
}

// one view: masks, then broadcast-by-modulo strided address
__device__ float read_view(const void *buf, uint64_t cap, uint32_t dt, const DView &v,
                           const uint32_t *c, uint32_t rank, int *status) {
    const uint32_t n = rank < v.rank ? rank : v.rank;
    if (v.has_mask) {
        for (uint32_t d = 0; d < n; d++)
            if (c[d] < v.mb[d] || c[d] >= v.me[d]) return 0.0f;
        for (uint32_t k = 0; k < v.n_cm; k++) {
            int32_t t = (int32_t)c[v.cm[k].da & 7u] * v.cm[k].sa + (int32_t)c[v.cm[k].db & 7u];
            if (t < (int32_t)v.cm[k].begin || t >= (int32_t)v.cm[k].end) return 0.0f;
        }
    }
    int64_t idx = v.offset;
    for (uint32_t d = 0; d < n; d++) {
        uint32_t dim = v.dims[d];
        uint32_t cc = dim > 1 ? c[d] % dim : 0u;
        idx += (int64_t)cc * v.strides[d];
    }
    return checked_load(buf, dt, idx, cap, status);
}

// stacked views: the flat position in the iteration space is pushed through
// each (outer, inner) pair, innermost view last.  `fdims` are the dims the
// flat position is taken over (all zero in the post-reduce phase, as the CPU
// backend passes a zeroed shape there).
__device__ float read_tracker(const void *buf, uint64_t cap, uint32_t dt, const DTracker &t,
                              const uint32_t *c, uint32_t rank, const uint32_t *fdims, int *status) {
    uint32_t si = 0;
    {
        uint32_t s = 1;
        for (int d = (int)rank - 1; d >= 0; d--) { si += c[d] * s; s *= fdims[d]; }
    }
    for (int vi = (int)t.n_views - 2; vi >= 0; vi--) {
        const DView &in = t.views[vi];
        const DView &ou = t.views[vi + 1];
        uint32_t oflat = 0;
        {
            uint32_t run = 1, ostride = 1;
            for (int d = (int)ou.rank - 1; d >= 0; d--) {
                uint32_t dim = ou.dims[d];
                if (dim > 1) {
                    uint32_t cc = run ? (si / run) % dim : 0u;
                    oflat += cc * ostride;
                }
                run *= dim;           // a zero dim zeroes the divisor (guarded above)
                ostride *= dim;
            }
        }
        int32_t idx = in.offset;
        uint32_t rem = oflat;
        uint32_t istr[THC_MAX_DIM];
        {
            uint32_t s = 1;
            for (int d = (int)in.rank - 1; d >= 0; d--) { istr[d] = s; s *= in.dims[d]; }
        }
        for (uint32_t d = 0; d < in.rank; d++) {
            uint32_t cc = istr[d] ? rem / istr[d] : 0u;
            rem = istr[d] ? rem % istr[d] : rem;
            if (in.has_mask && (cc < in.mb[d] || cc >= in.me[d])) return 0.0f;
            if (in.strides[d] != 0) idx += (int32_t)cc * in.strides[d];
        }
        if (idx < 0) return 0.0f;
        si = (uint32_t)idx;
    }
    return checked_load(buf, dt, (int64_t)si, cap, status);
}

__device__ __forceinline__ float read_leaf(const GenDesc *D, const GenArgs &A, uint32_t i,
                                           const uint32_t *c, const uint32_t *fdims) {
    const DLeaf &L = D->leaves[i];
    if (L.tracker >= 0)
        return read_tracker(A.leaf[i], A.cap[i], L.dtype, D->trackers[L.tracker], c, D->rank, fdims, A.status);
    return read_view(A.leaf[i], A.cap[i], L.dtype, L.v, c, D->rank, A.status);
}

// leaves -> SSA ops [0, n_eval) -> value of the last one (or leaf 0)
__device__ float eval_point(const GenDesc *D, const GenArgs &A, const uint32_t *c, float *vals, uint32_t n_eval) {
    const uint32_t nl = D->n_leaves;
    for (uint32_t i = 0; i < nl; i++) vals[i] = read_leaf(D, A, i, c, D->full_dims);
    for (uint32_t i = 0; i < n_eval; i++) {
        const thc_fused_op_t op = D->ops[i];
        vals[nl + i] = alu(op.uop, op.aux, vals[op.arg_a], vals[op.arg_b]);
    }
    return n_eval ? vals[nl + n_eval - 1] : vals[0];
}

__global__ void __launch_bounds__(256) k_generic_ew(const GenDesc *__restrict__ D, const GenArgs A) {
    float vals[THC_MAX_LEAVES + THC_MAX_OPS];
    const uint64_t total = D->full_numel;
    const uint32_t rank = D->rank;
    for (uint64_t flat = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; flat < total;
         flat += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t c[THC_MAX_DIM] = {0, 0, 0, 0, 0, 0, 0, 0};
        uint64_t rem = flat;
        for (int d = (int)rank - 1; d >= 0; d--) { uint32_t dim = D->full_dims[d]; c[d] = (uint32_t)(rem % dim); rem /= dim; }
        float r = eval_point(D, A, c, vals, D->n_ops);
        if (flat < A.out_cap) store_from_f32(A.out, D->out_dtype, flat, r);
        else atomicOr(A.status, ERR_STORE_OOB);
    }
}

// post-reduce phase for one output element (legacy provenance path)
__device__ float post_reduce(const GenDesc *D, const GenArgs &A, const uint32_t *c, float *vals, float reduced) {
    const uint32_t nl = D->n_leaves, npre = nl - D->n_post_leaves;
    const uint32_t zero_dims[THC_MAX_DIM] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (uint32_t i = 0; i < nl; i++) vals[i] = i < npre ? 0.0f : read_leaf(D, A, i, c, zero_dims);
    vals[nl + D->post_start - 1] = reduced;
    for (uint32_t i = D->post_start; i < D->n_ops; i++) {
        const thc_fused_op_t op = D->ops[i];
        vals[nl + i] = alu(op.uop, op.aux, vals[op.arg_a], vals[op.arg_b]);
    }
    return vals[nl + D->n_ops - 1];
}

// G threads cooperate on each output element: 1 (serial, exact left-to-right
// order, also the only mode that can mimic accumulation in a non-f32 output
// dtype), 32 (a warp) or 256 (the CTA).
template <int G>
__global__ void __launch_bounds__(256) k_generic_reduce(const GenDesc *__restrict__ D, const GenArgs A) {
    float vals[THC_MAX_LEAVES + THC_MAX_OPS];
    __shared__ float part[8];
    const uint32_t rank = D->rank, rtype = D->reduce_type, odt = D->out_dtype;
    const uint64_t n_out = D->out_numel, n_red = D->reduce_numel;
    const uint32_t n_eval = D->post_start ? D->post_start : D->n_ops;
    const uint32_t lane = G == 1 ? 0 : (threadIdx.x % G);
    const uint64_t groups = ((uint64_t)gridDim.x * blockDim.x) / G;
    const uint64_t gi0 = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
    // every thread of a group runs the same trip count (the shuffles below need it)
    for (uint64_t oi = gi0; oi < n_out; oi += groups) {
        uint32_t c[THC_MAX_DIM] = {0, 0, 0, 0, 0, 0, 0, 0};
        {
            uint64_t rem = oi;
            for (int k = (int)D->n_kdims - 1; k >= 0; k--) {
                uint32_t d = D->kdim[k], dim = D->full_dims[d];
                c[d] = (uint32_t)(rem % dim); rem /= dim;
            }
        }
        float acc = red_init(rtype);
        if (G == 1 && odt != THC_F32) {
            // accumulate in the stored representation, as the CPU backend does by
            // loading and storing the output element at every step
            uint32_t bits = encode_bits(acc, odt);
            for (uint64_t r = 0; r < n_red; r++) {
                uint64_t rem = r;
                for (int k = (int)D->n_rdims - 1; k >= 0; k--) {
                    uint32_t d = D->rdim[k], dim = D->full_dims[d];
                    c[d] = (uint32_t)(rem % dim); rem /= dim;
                }
                float v = eval_point(D, A, c, vals, n_eval);
                bits = encode_bits(red_combine(rtype, decode_bits(bits, odt), v), odt);
            }
            for (uint32_t k = 0; k < D->n_rdims; k++) c[D->rdim[k]] = 0;
            if (D->post_start && D->post_start < D->n_ops)
                bits = encode_bits(post_reduce(D, A, c, vals, decode_bits(bits, odt)), odt);
            if (oi < A.out_cap) store_bits(A.out, odt, oi, bits);
            else atomicOr(A.status, ERR_STORE_OOB);
            continue;
        }
        for (uint64_t r = lane; r < n_red; r += G) {
            uint64_t rem = r;
            for (int k = (int)D->n_rdims - 1; k >= 0; k--) {
                uint32_t d = D->rdim[k], dim = D->full_dims[d];
                c[d] = (uint32_t)(rem % dim); rem /= dim;
            }
            float v = eval_point(D, A, c, vals, n_eval);
            acc = red_combine(rtype, acc, v);
        }
        if (G > 1) {
            for (int o = 16; o > 0; o >>= 1) acc = red_combine(rtype, acc, __shfl_down_sync(0xffffffffu, acc, o));
        }
        if (G == 256) {
            __syncthreads();                       // part[] free from the previous output
            if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
            __syncthreads();
            if (threadIdx.x == 0) { acc = part[0]; for (int w = 1; w < 8; w++) acc = red_combine(rtype, acc, part[w]); }
        }
        if (lane == 0) {
            for (uint32_t k = 0; k < D->n_rdims; k++) c[D->rdim[k]] = 0;
            if (D->post_start && D->post_start < D->n_ops) acc = post_reduce(D, A, c, vals, acc);
            if (oi < A.out_cap) store_from_f32(A.out, odt, oi, acc);
            else atomicOr(A.status, ERR_STORE_OOB);
        }
    }
}

// host: launch the right generic kernel for a prepared descriptor
void launch_generic(const GenDesc &H, const GenDesc *dev_desc, const GenArgs &args) {
    profile_begin();
    if (!H.has_reduce) {
        if (H.full_numel == 0) return;
        unsigned grid = grid_for(H.full_numel, 256, 8);
        k_generic_ew<<<grid, 256, 0, g.stream>>>(dev_desc, args);
        after_launch("generic_ew");
        return;
    }
    if (H.out_numel == 0) return;
    int G = 1;
    if (H.out_dtype == THC_F32) {
        if (H.reduce_numel >= 2048) G = 256;
        else if (H.reduce_numel > 64) G = 32;
    }
    if (G == 1) {
        k_generic_reduce<1><<<grid_for(H.out_numel, 256, 8), 256, 0, g.stream>>>(dev_desc, args);
        after_launch("generic_reduce_serial");
    } else if (G == 32) {
        k_generic_reduce<32><<<grid_for(H.out_numel, 8, 8), 256, 0, g.stream>>>(dev_desc, args);
        after_launch("generic_reduce_warp");
    } else {
        k_generic_reduce<256><<<grid_for(H.out_numel, 1, 8), 256, 0, g.stream>>>(dev_desc, args);
        after_launch("generic_reduce_cta");
    }
}

}  // namespace thc
