// uop.cu — executes a lowered KOP program (`UOpKernel`), the second dispatch
// form of the vtable.
//
// Semantics restated from src/backend/cpu/uop.c:29-155: one program run per
// `gid` (grid[0] runs when local_size > 0, else grid0*grid1*grid2), values are
// u32 or f32 depending on the producing op (uop.c:3-27), RANGE/ENDRANGE are
// counted loops, ACC folds into its ACC_INIT register, STORE writes the
// output buffer.  The lowered program loads before it masks
// (src/lower/_.c:303-307), which walks off the buffer for padded views; here
// every LOAD is checked against the buffer size and yields 0 out of range, so
// the following MASK selects the right value without a fault.
//
// adam_step follows the arithmetic of the reference's Metal kernel
// (src/shaders.metal:406-420), the only definition of that vtable slot.
#include "device_common.cuh"
#include "plans.h"
#include "state.h"

namespace thc {

struct KProg {
    uint32_t n_ops, n_leaves, out_dtype;
    uint32_t leaf_dtypes[THC_MAX_LEAVES];
    uint32_t range_end[THC_KOP_MAX];     // RANGE -> its ENDRANGE
    uint32_t range_start[THC_KOP_MAX];   // ENDRANGE -> its RANGE
    thc_kop_t ops[THC_KOP_MAX];
};

struct KArgs {
    void *out; uint64_t out_cap;
    const void *leaf[THC_MAX_LEAVES]; uint64_t cap[THC_MAX_LEAVES];
    uint64_t total; int *status;
    uint64_t fuel;                       // op executions one gid may take: the host's count for this program, doubled
};

__device__ __forceinline__ bool k_is_float(uint32_t type) {
    return type == THC_KOP_CONST_F || type == THC_KOP_LOAD || type == THC_KOP_ALU ||
           type == THC_KOP_ACC_INIT || type == THC_KOP_MASK;
}

__global__ void __launch_bounds__(128) k_uop(const KProg *__restrict__ P, const KArgs A) {
    uint32_t reg[THC_KOP_MAX];           // bit patterns; typed by the producing op
    const uint32_t n = P->n_ops;
    auto as_u = [&](uint32_t id) -> uint32_t {
        if (id >= n) return 0u;
        return k_is_float(P->ops[id].type) ? cast_u32(__uint_as_float(reg[id])) : reg[id];
    };
    auto as_f = [&](uint32_t id) -> float {
        if (id >= n) return 0.0f;
        return k_is_float(P->ops[id].type) ? __uint_as_float(reg[id]) : (float)reg[id];
    };
    for (uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; gid < A.total;
         gid += (uint64_t)gridDim.x * blockDim.x) {
        for (uint32_t i = 0; i < n; i++) reg[i] = 0u;
        uint32_t pc = 0;
        uint64_t fuel = A.fuel;           // the host counted what a well-formed run needs; running out is reported, not spun on
        while (pc < n) {
            if (fuel-- == 0) { atomicOr(A.status, ERR_BAD_PROGRAM); break; }
            const thc_kop_t op = P->ops[pc];
            switch (op.type) {
                case THC_KOP_GID:      reg[pc] = (uint32_t)gid; break;
                case THC_KOP_CONST_U:  reg[pc] = op.imm.u; break;
                case THC_KOP_CONST_F:
                case THC_KOP_ACC_INIT: reg[pc] = __float_as_uint(op.imm.f); break;
                case THC_KOP_MOD:      reg[pc] = op.imm.u ? as_u(op.arg[0]) % op.imm.u : 0u; break;
                case THC_KOP_DIV:      reg[pc] = op.imm.u ? as_u(op.arg[0]) / op.imm.u : 0u; break;
                case THC_KOP_IDX:      reg[pc] = as_u(op.arg[0]) * op.imm.u + as_u(op.arg[1]); break;
                case THC_KOP_LOAD: {
                    const uint32_t b = op.imm.u;
                    const uint32_t idx = as_u(op.arg[0]);
                    float v = 0.0f;
                    if (b == 0) {
                        if (idx < A.out_cap) v = load_as_f32(A.out, P->out_dtype, idx);
                    } else if (b - 1 < P->n_leaves) {
                        if (idx < A.cap[b - 1]) v = load_as_f32(A.leaf[b - 1], P->leaf_dtypes[b - 1], idx);
                    }
                    reg[pc] = __float_as_uint(v);
                    break;
                }
                case THC_KOP_MASK:
                    reg[pc] = __float_as_uint(as_f(op.arg[0]) != 0.0f ? as_f(op.arg[1]) : 0.0f);
                    break;
                case THC_KOP_ALU:
                    reg[pc] = __float_as_uint(alu(op.imm.u, op.arg[2], as_f(op.arg[0]), as_f(op.arg[1])));
                    break;
                case THC_KOP_ACC: {
                    const uint32_t a = op.arg[0];
                    if (a < n) reg[a] = __float_as_uint(red_combine(op.imm.u == THC_RMAX ? THC_RMAX : THC_SUM,
                                                                    __uint_as_float(reg[a]), as_f(op.arg[1])));
                    break;
                }
                case THC_KOP_RANGE:
                    reg[pc] = 0u;
                    if (op.imm.u == 0) pc = P->range_end[pc];      // empty loop: skip the body
                    break;
                case THC_KOP_ENDRANGE: {
                    const uint32_t s = P->range_start[pc];
                    if (reg[s] + 1 < P->ops[s].imm.u) { reg[s] += 1; pc = s; }   // next trip: resume after RANGE
                    break;
                }
                case THC_KOP_STORE: {
                    const uint32_t idx = as_u(op.arg[0]);
                    if (idx < A.out_cap) store_from_f32(A.out, P->out_dtype, idx, as_f(op.arg[1]));
                    else atomicOr(A.status, ERR_STORE_OOB);
                    break;
                }
                case THC_KOP_NOOP: break;
                default: atomicOr(A.status, ERR_BAD_PROGRAM); pc = n; break;
            }
            pc++;
        }
    }
}

__global__ void __launch_bounds__(256) k_adam(float *__restrict__ p, const float *__restrict__ gr,
                                              float *__restrict__ m, float *__restrict__ v,
                                              float lr, float b1, float b2, float eps, float bc1, float bc2, uint32_t n) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float gi = gr[i];
        const float mi = __fadd_rn(__fmul_rn(b1, m[i]), __fmul_rn(1.0f - b1, gi));
        const float vi = __fadd_rn(__fmul_rn(b2, v[i]), __fmul_rn(__fmul_rn(1.0f - b2, gi), gi));
        m[i] = mi; v[i] = vi;
        const float mh = __fdiv_rn(mi, bc1), vh = __fdiv_rn(vi, bc2);
        p[i] = __fsub_rn(p[i], __fdiv_rn(__fmul_rn(lr, mh), __fadd_rn(__fsqrt_rn(vh), eps)));
    }
}

// 2x2 stride-2 max-pool that also records which element of the window won: scan order
// (0,0),(0,1),(1,0),(1,1), strict '>' so the first maximum wins, index stored as u8 0..3
// (the arithmetic of the reference's max-pool shader, src/shaders.metal:427-458).
// One thread per pair of neighbouring outputs: two 16-byte loads (one per input row).
// (value, index) of a window scanned in order w0..w3 with strict '>'.  `floor`: start from the RMAX identity
// -1e30f instead of from w0, which is what a reduce dispatch computes (src/backend/cpu/dispatch.c:148-151, 202-217).
__device__ __forceinline__ void pick4(float w0, float w1, float w2, float w3, bool floor, float &best, uint8_t &bi) {
    best = floor ? -1e30f : w0; bi = 0;
    if (floor && w0 > best) best = w0;
    if (w1 > best) { best = w1; bi = 1; }
    if (w2 > best) { best = w2; bi = 2; }
    if (w3 > best) { best = w3; bi = 3; }
}
__global__ void __launch_bounds__(256) k_maxpool2x2_index(const float *__restrict__ x, float *__restrict__ y, uint8_t *__restrict__ idx,
                                                          unsigned long long planes, unsigned H, unsigned W, unsigned vec, unsigned floor) {
    const unsigned OH = H / 2, OW = W / 2;
    const unsigned per_row = vec ? OW / 2 : OW;                      // work items per output row
    const unsigned long long items = planes * OH * per_row;
    for (unsigned long long it = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; it < items;
         it += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned c = (unsigned)(it % per_row);
        const unsigned long long rowi = it / per_row;                // plane * OH + oy
        const unsigned oy = (unsigned)(rowi % OH);
        const unsigned long long plane = rowi / OH;
        const float *r0 = x + (plane * H + 2ull * oy) * W;
        const float *r1 = r0 + W;
        const unsigned long long o = rowi * OW;
        if (vec) {
            const float4 a = *reinterpret_cast<const float4 *>(r0 + 4u * c), b = *reinterpret_cast<const float4 *>(r1 + 4u * c);
            float b0, b1; uint8_t i0, i1;
            pick4(a.x, a.y, b.x, b.y, floor != 0, b0, i0);
            pick4(a.z, a.w, b.z, b.w, floor != 0, b1, i1);
            *reinterpret_cast<float2 *>(y + o + 2u * c) = make_float2(b0, b1);
            if (idx) { idx[o + 2u * c] = i0; idx[o + 2u * c + 1] = i1; }
        } else {
            float best; uint8_t bi;
            pick4(r0[2u * c], r0[2u * c + 1], r1[2u * c], r1[2u * c + 1], floor != 0, best, bi);
            y[o + c] = best;
            if (idx) idx[o + c] = bi;
        }
    }
}

// first index of the row maximum (strictly greater wins, so ties keep the earlier index): one warp per row.
// The reference computes this on the host after a full read-back (src/ops/_.c:502-524).
__global__ void __launch_bounds__(256) k_argmax_rows(const float *__restrict__ x, uint32_t *__restrict__ out, unsigned rows, unsigned cols) {
    const unsigned lane = threadIdx.x & 31;
    for (unsigned long long r = ((unsigned long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows;
         r += ((unsigned long long)gridDim.x * blockDim.x) >> 5) {
        const float *row = x + r * cols;
        // per-lane candidate over its strided columns, seeded like the host loop: best = column 0
        float bv = row[0]; unsigned bi = 0;
        for (unsigned c = lane; c < cols; c += 32) {
            const float v = row[c];
            if (c != 0 && (v > bv)) { bv = v; bi = c; }
        }
        // a candidate replaces another only if strictly greater, or equal with a smaller index;
        // a NaN never wins a '>' test, exactly as in the sequential scan
#pragma unroll
        for (int w = 16; w > 0; w >>= 1) {
            const float ov = __shfl_down_sync(0xffffffffu, bv, w);
            const unsigned oi = __shfl_down_sync(0xffffffffu, bi, w);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) out[r] = bi;
    }
}

// ---- the RMAX dispatch of a 2x2 stride-2 pool (thvm_maxpool2d, src/nn/conv.c:484-513) on the pooling kernel ----
// Recognised shape: one unmasked f32 leaf, no ops, RMAX over the last two dims (2, 2), the leaf a window view of
// contiguous [planes, H, W] memory: strides (..., 2W, 2, W, 1) over (..., OH, OW, 2, 2) with H = 2 OH, W = 2 OW.
bool try_pool2x2(Plan *p) {
    const GenDesc &H = p->host;
    if (!H.has_reduce || H.reduce_type != THC_RMAX || H.n_leaves != 1 || H.n_ops != 0 || H.post_start || H.out_dtype != THC_F32) return false;
    const DLeaf &L = H.leaves[0];
    const int r = (int)H.rank;
    if (L.dtype != THC_F32 || L.tracker >= 0 || L.v.has_mask || L.v.n_cm || r < 4 || (int)L.v.rank != r) return false;
    if (H.n_rdims != 2 || (int)H.rdim[0] != r - 2 || (int)H.rdim[1] != r - 1) return false;
    for (int d = 0; d < r; d++) if (L.v.dims[d] != H.full_dims[d]) return false;
    if (H.full_dims[r - 1] != 2 || H.full_dims[r - 2] != 2) return false;
    const unsigned long long OW = H.full_dims[r - 3], OH = H.full_dims[r - 4], W = 2 * OW, Hh = 2 * OH;
    if (L.v.strides[r - 1] != 1 || L.v.strides[r - 2] != (long long)W || L.v.strides[r - 3] != 2 || L.v.strides[r - 4] != (long long)(2 * W)) return false;
    unsigned long long planes = 1, want = Hh * W;
    for (int d = r - 5; d >= 0; d--) {
        if (H.full_dims[d] != 1 && (unsigned long long)L.v.strides[d] != want) return false;
        planes *= H.full_dims[d]; want *= H.full_dims[d];
    }
    if (L.v.offset < 0 || Hh > 0xFFFFFFFFull || W > 0xFFFFFFFFull) return false;
    p->pool_planes = planes; p->pool_h = (uint32_t)Hh; p->pool_w = (uint32_t)W; p->pool_off = L.v.offset;
    p->kind = PLAN_POOL;
    return true;
}

// ---- the max-pool backward dispatch, out[.., oy, ox, i, j] = g[.., oy, ox] * (one - (max[.., oy, ox] > x[.., 2oy+i, 2ox+j])) ----
// (the mask form of the reference's RMAX gradient rule, src/interact/grad.c:406-425: every element equal to the
// maximum passes the gradient).  Output in window layout [planes, OH, OW, 2, 2], contiguous.
__global__ void __launch_bounds__(256) k_maxpool2x2_bwd(const float *__restrict__ g, const float *__restrict__ one, const float *__restrict__ mx,
                                                        const float *__restrict__ x, float *__restrict__ out,
                                                        unsigned long long planes, unsigned H, unsigned W, unsigned vec) {
    const unsigned OH = H / 2, OW = W / 2;
    const unsigned per_row = vec ? OW / 2 : OW;
    const unsigned long long items = planes * OH * per_row;
    const float o1 = one[0];
    for (unsigned long long it = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; it < items;
         it += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned c = (unsigned)(it % per_row);
        const unsigned long long rowi = it / per_row;                // plane * OH + oy
        const unsigned oy = (unsigned)(rowi % OH);
        const unsigned long long plane = rowi / OH;
        const float *r0 = x + (plane * H + 2ull * oy) * W;
        const float *r1 = r0 + W;
        const unsigned long long o = rowi * OW;
        auto f = [&](float gg, float m, float v) { return __fmul_rn(gg, __fsub_rn(o1, m > v ? 1.0f : 0.0f)); };
        if (vec) {
            const float4 a = *reinterpret_cast<const float4 *>(r0 + 4u * c), b = *reinterpret_cast<const float4 *>(r1 + 4u * c);
            const float2 gg = *reinterpret_cast<const float2 *>(g + o + 2u * c), mm = *reinterpret_cast<const float2 *>(mx + o + 2u * c);
            float4 *dst = reinterpret_cast<float4 *>(out + (o + 2u * c) * 4ull);
            dst[0] = make_float4(f(gg.x, mm.x, a.x), f(gg.x, mm.x, a.y), f(gg.x, mm.x, b.x), f(gg.x, mm.x, b.y));
            dst[1] = make_float4(f(gg.y, mm.y, a.z), f(gg.y, mm.y, a.w), f(gg.y, mm.y, b.z), f(gg.y, mm.y, b.w));
        } else {
            const float gg = g[o + c], m = mx[o + c];
            float4 *dst = reinterpret_cast<float4 *>(out + (o + c) * 4ull);
            dst[0] = make_float4(f(gg, m, r0[2u * c]), f(gg, m, r0[2u * c + 1]), f(gg, m, r1[2u * c]), f(gg, m, r1[2u * c + 1]));
        }
    }
}

static bool window_view(const GenDesc &H, const DLeaf &L, unsigned long long &planes, unsigned long long &Hh, unsigned long long &W) {
    const int r = (int)H.rank;
    if (L.dtype != THC_F32 || L.tracker >= 0 || L.v.has_mask || L.v.n_cm || r < 4 || (int)L.v.rank != r) return false;
    for (int d = 0; d < r; d++) if (L.v.dims[d] != H.full_dims[d]) return false;
    if (H.full_dims[r - 1] != 2 || H.full_dims[r - 2] != 2) return false;
    const unsigned long long OW = H.full_dims[r - 3], OH = H.full_dims[r - 4];
    W = 2 * OW; Hh = 2 * OH;
    if (L.v.strides[r - 1] != 1 || L.v.strides[r - 2] != (long long)W || L.v.strides[r - 3] != 2 || L.v.strides[r - 4] != (long long)(2 * W)) return false;
    planes = 1;
    unsigned long long want = Hh * W;
    for (int d = r - 5; d >= 0; d--) {
        if (H.full_dims[d] != 1 && (unsigned long long)L.v.strides[d] != want) return false;
        planes *= H.full_dims[d]; want *= H.full_dims[d];
    }
    return L.v.offset >= 0 && Hh <= 0xFFFFFFFFull && W <= 0xFFFFFFFFull;
}
// a [planes, OH, OW] tensor broadcast over the 2x2 window dims
static bool pooled_view(const GenDesc &H, const DLeaf &L) {
    const int r = (int)H.rank;
    if (L.dtype != THC_F32 || L.tracker >= 0 || L.v.has_mask || L.v.n_cm || (int)L.v.rank != r) return false;
    for (int d = 0; d < r; d++) if (L.v.dims[d] != H.full_dims[d]) return false;
    const unsigned long long OW = H.full_dims[r - 3], OH = H.full_dims[r - 4];
    if (L.v.strides[r - 1] != 0 || L.v.strides[r - 2] != 0 || L.v.strides[r - 3] != 1 || L.v.strides[r - 4] != (long long)OW) return false;
    unsigned long long want = OH * OW;
    for (int d = r - 5; d >= 0; d--) {
        if (H.full_dims[d] != 1 && (unsigned long long)L.v.strides[d] != want) return false;
        want *= H.full_dims[d];
    }
    return L.v.offset >= 0;
}

bool try_pool2x2_bwd(Plan *p) {
    const GenDesc &H = p->host;
    if (H.has_reduce || H.n_leaves != 4 || H.n_ops != 3 || H.post_start || H.out_dtype != THC_F32) return false;
    const thc_fused_op_t *o = H.ops;
    if (!(o[0].uop == THC_CMP && o[0].arg_a == 2 && o[0].arg_b == 3 && o[1].uop == THC_SUB && o[1].arg_a == 1 && o[1].arg_b == 4 &&
          o[2].uop == THC_MUL && o[2].arg_a == 0 && o[2].arg_b == 5)) return false;
    unsigned long long planes, Hh, W;
    if (!window_view(H, H.leaves[3], planes, Hh, W) || !pooled_view(H, H.leaves[0]) || !pooled_view(H, H.leaves[2])) return false;
    const DLeaf &S1 = H.leaves[1];
    if (S1.dtype != THC_F32 || S1.tracker >= 0 || S1.v.has_mask || S1.v.offset < 0) return false;
    for (unsigned d = 0; d < S1.v.rank; d++) if (S1.v.dims[d] != 1 && S1.v.strides[d] != 0) return false;
    p->pool_planes = planes; p->pool_h = (uint32_t)Hh; p->pool_w = (uint32_t)W; p->pool_off = H.leaves[3].v.offset;
    p->pool_g_off = H.leaves[0].v.offset; p->pool_one_off = S1.v.offset; p->pool_m_off = H.leaves[2].v.offset;
    p->kind = PLAN_POOL_BWD;
    return true;
}

bool launch_pool2x2_bwd(Plan *p, const GenArgs &args) {
    const unsigned long long in_n = p->pool_planes * p->pool_h * p->pool_w, out_n = in_n / 4;
    if ((unsigned long long)p->pool_off + in_n > args.cap[3] || (unsigned long long)p->pool_g_off + out_n > args.cap[0] ||
        (unsigned long long)p->pool_m_off + out_n > args.cap[2] || (unsigned long long)p->pool_one_off >= args.cap[1])
        return false;
    const float *gr = (const float *)args.leaf[0] + p->pool_g_off, *one = (const float *)args.leaf[1] + p->pool_one_off;
    const float *mx = (const float *)args.leaf[2] + p->pool_m_off, *x = (const float *)args.leaf[3] + p->pool_off;
    if (reinterpret_cast<uintptr_t>(args.out) & 15u) return false;
    const unsigned vec = (p->pool_w % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(gr) & 7u) == 0 &&
                          (reinterpret_cast<uintptr_t>(mx) & 7u) == 0) ? 1u : 0u;
    const uint64_t items = p->pool_planes * (p->pool_h / 2) * (vec ? p->pool_w / 4 : p->pool_w / 2);
    if (g.profile_level >= 2) snprintf(g.last_shape, sizeof g.last_shape, "planes=%llu H=%u W=%u vec=%u", p->pool_planes, p->pool_h, p->pool_w, vec);
    profile_begin();
    k_maxpool2x2_bwd<<<grid_for(items, 256, 8), 256, 0, g.stream>>>(gr, one, mx, x, (float *)args.out, p->pool_planes, p->pool_h, p->pool_w, vec);
    after_launch("pool2x2_backward");
    return true;
}

bool launch_pool2x2(Plan *p, const GenArgs &args) {
    const unsigned long long in_n = p->pool_planes * p->pool_h * p->pool_w;
    if ((unsigned long long)p->pool_off + in_n > args.cap[0]) return false;         // would leave the buffer: the checked generic kernel runs
    const float *x = (const float *)args.leaf[0] + p->pool_off;
    const unsigned vec = (p->pool_w % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(args.out) & 7u) == 0) ? 1u : 0u;
    const uint64_t items = p->pool_planes * (p->pool_h / 2) * (vec ? p->pool_w / 4 : p->pool_w / 2);
    if (g.profile_level >= 2) snprintf(g.last_shape, sizeof g.last_shape, "planes=%llu H=%u W=%u vec=%u", p->pool_planes, p->pool_h, p->pool_w, vec);
    profile_begin();
    k_maxpool2x2_index<<<grid_for(items, 256, 8), 256, 0, g.stream>>>(x, (float *)args.out, nullptr, p->pool_planes, p->pool_h, p->pool_w, vec, 1u);
    after_launch("pool2x2_rmax");
    return true;
}

}  // namespace thc

using namespace thc;

extern "C" {

void thvm_cuda_dispatch_uop_kernel(uint32_t out_buf, const uint32_t *leaf_bufs, uint32_t n_leaves,
                                   const thc_uop_kernel_t *kernel, uint64_t cache_key) {
    (void)cache_key;
    if (!g.ready) fatal("dispatch_uop_kernel: backend not initialised (no CUDA device?)");
    if (!kernel) return;
    if (kernel->n_ops > THC_KOP_MAX || n_leaves > THC_MAX_LEAVES) { set_error("uop kernel: %u ops / %u leaves out of range", kernel->n_ops, n_leaves); return; }
    static KProg hp;                          // ~20 KB, reused per call
    memset(&hp, 0, sizeof hp);
    hp.n_ops = kernel->n_ops; hp.n_leaves = n_leaves; hp.out_dtype = kernel->out_dtype;
    for (uint32_t i = 0; i < n_leaves; i++) hp.leaf_dtypes[i] = kernel->leaf_dtypes[i];
    // Loop structure, and the number of op executions one gid performs: every op runs once per trip of the loops
    // around it.  A program whose nested trip counts multiply out beyond UOP_MAX_STEPS per gid is refused here
    // instead of being left to occupy the GPU (the largest reduce range a reference kernel carries is 2^32).
    constexpr double UOP_MAX_STEPS = 34359738368.0;   // 2^35
    uint32_t stack[THC_KOP_MAX], sp = 0;
    double trips = 1.0, steps = 0.0;
    for (uint32_t i = 0; i < kernel->n_ops; i++) {
        hp.ops[i] = kernel->ops[i];
        if (kernel->ops[i].type == THC_KOP_RANGE) {
            steps += trips;
            stack[sp++] = i;
            trips *= (double)(kernel->ops[i].imm.u ? kernel->ops[i].imm.u : 1u);
            continue;
        }
        if (kernel->ops[i].type == THC_KOP_ENDRANGE) {
            if (sp == 0) { set_error("uop kernel: ENDRANGE without RANGE at %u", i); return; }
            uint32_t s = stack[--sp];
            hp.range_end[s] = i; hp.range_start[i] = s;
            steps += trips;
            trips /= (double)(kernel->ops[s].imm.u ? kernel->ops[s].imm.u : 1u);
            continue;
        }
        steps += trips;
    }
    if (sp != 0) { set_error("uop kernel: unclosed RANGE"); return; }
    if (steps > UOP_MAX_STEPS) { set_error("uop kernel: %.3g op executions per output exceed the limit of %.3g", steps, UOP_MAX_STEPS); return; }

    Buf &ob = buf_checked(out_buf, "dispatch_uop(out)");
    KArgs a; memset(&a, 0, sizeof a);
    a.out = ob.ptr; a.out_cap = ob.bytes / dtype_bytes(kernel->out_dtype);
    for (uint32_t i = 0; i < n_leaves; i++) {
        Buf &lb = buf_checked(leaf_bufs[i], "dispatch_uop(leaf)");
        a.leaf[i] = lb.ptr; a.cap[i] = lb.bytes / dtype_bytes(kernel->leaf_dtypes[i]);
    }
    a.total = kernel->local_size > 0 ? kernel->grid[0]
                                     : (uint64_t)kernel->grid[0] * kernel->grid[1] * kernel->grid[2];
    a.status = g.dev_status;
    a.fuel = 2ull * (uint64_t)steps + 16;
    if (a.total == 0) return;
    mark_device_written(out_buf);

    KProg *dp = (KProg *)scratch_reserve(sizeof(KProg));
    // the program is staged through the ring in <= 1 MiB pieces (it is ~20 KB)
    upload_small(dp, &hp, sizeof(KProg));
    profile_begin();
    k_uop<<<grid_for(a.total, 128, 8), 128, 0, g.stream>>>(dp, a);
    after_launch("uop_program");
}

void thvm_cuda_adam_step(uint32_t param, uint32_t grad, uint32_t m, uint32_t v, float lr, float beta1, float beta2,
                         float eps, float bc1, float bc2, uint32_t n) {
    Buf &bp = buf_checked(param, "adam(param)"), &bg = buf_checked(grad, "adam(grad)");
    Buf &bm = buf_checked(m, "adam(m)"), &bv = buf_checked(v, "adam(v)");
    uint64_t need = (uint64_t)n * 4;
    if (bp.bytes < need || bg.bytes < need || bm.bytes < need || bv.bytes < need) { set_error("adam_step: n=%u exceeds a buffer", n); return; }
    if (n == 0) return;
    mark_device_written(param); mark_device_written(m); mark_device_written(v);
    profile_begin();
    k_adam<<<grid_for(n, 256, 8), 256, 0, g.stream>>>((float *)bp.ptr, (const float *)bg.ptr, (float *)bm.ptr,
                                                      (float *)bv.ptr, lr, beta1, beta2, eps, bc1, bc2, n);
    after_launch("adam_step");
}

int thvm_cuda_maxpool2x2_index(uint32_t out_val, uint32_t out_idx, uint32_t x, uint32_t planes, uint32_t H, uint32_t W) {
    if (H < 2 || W < 2 || planes == 0) { set_error("maxpool2x2_index: empty shape"); return 1; }
    const uint64_t in_n = (uint64_t)planes * H * W, out_n = (uint64_t)planes * (H / 2) * (W / 2);
    Buf &bx = buf_checked(x, "maxpool2x2_index(x)");
    Buf &by = buf_for_output(out_val, "maxpool2x2_index(y)", out_n * 4);
    Buf *bi = out_idx ? &buf_for_output(out_idx, "maxpool2x2_index(idx)", out_n) : nullptr;
    if (bx.bytes < in_n * 4 || by.bytes < out_n * 4 || (bi && bi->bytes < out_n)) { set_error("maxpool2x2_index: a buffer is too small"); return 1; }
    mark_device_written(out_val);
    if (out_idx) mark_device_written(out_idx);
    const unsigned vec = (W % 4 == 0) ? 1u : 0u;                   // rows start 16-byte aligned, outputs 8-byte aligned
    const uint64_t items = (uint64_t)planes * (H / 2) * (vec ? W / 4 : W / 2);
    profile_begin();
    k_maxpool2x2_index<<<grid_for(items, 256, 8), 256, 0, g.stream>>>((const float *)bx.ptr, (float *)by.ptr, bi ? (uint8_t *)bi->ptr : nullptr,
                                                                     planes, H, W, vec, 0u);
    after_launch("maxpool2x2_index");
    return 0;
}

int thvm_cuda_argmax_rows(uint32_t out_u32, uint32_t x, uint32_t rows, uint32_t cols) {
    if (rows == 0 || cols == 0) { set_error("argmax_rows: empty shape"); return 1; }
    Buf &bx = buf_checked(x, "argmax_rows(x)");
    Buf &bo = buf_for_output(out_u32, "argmax_rows(out)", (uint64_t)rows * 4);
    if (bx.bytes < (uint64_t)rows * cols * 4 || bo.bytes < (uint64_t)rows * 4) { set_error("argmax_rows: a buffer is too small"); return 1; }
    mark_device_written(out_u32);
    profile_begin();
    k_argmax_rows<<<grid_for(rows, 8, 8), 256, 0, g.stream>>>((const float *)bx.ptr, (uint32_t *)bo.ptr, rows, cols);
    after_launch("argmax_rows");
    return 0;
}

}  // extern "C"
