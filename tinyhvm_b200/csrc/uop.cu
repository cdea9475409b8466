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
        uint64_t fuel = 1ull << 40;       // a malformed program cannot spin forever
        while (pc < n && fuel--) {
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
    uint32_t stack[THC_KOP_MAX], sp = 0;
    for (uint32_t i = 0; i < kernel->n_ops; i++) {
        hp.ops[i] = kernel->ops[i];
        if (kernel->ops[i].type == THC_KOP_RANGE) stack[sp++] = i;
        else if (kernel->ops[i].type == THC_KOP_ENDRANGE) {
            if (sp == 0) { set_error("uop kernel: ENDRANGE without RANGE at %u", i); return; }
            uint32_t s = stack[--sp];
            hp.range_end[s] = i; hp.range_start[i] = s;
        }
    }
    if (sp != 0) { set_error("uop kernel: unclosed RANGE"); return; }

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

}  // extern "C"
