/* thvm_oracle.c — CPU restatement of the reference's realized-kernel path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product (tinyhvm_b200/, the CUDA
 * library) links, loads or calls this file; it exists so the tests, the smoke
 * check and the CPU-baseline leg of the benchmark have an independent,
 * sequential answer to compare the CUDA kernels with.
 *
 * Parity status: PINNED.  tests/test_oracle_pins.py checks this file against
 * (a) the golden vectors the reference itself carries for this path and
 * (b) the reference's own CPU backend compiled from its sources
 * (oracle/_ref/libthvm_cpu_ref.so, built by oracle/Makefile), on randomised
 * dispatches, bit for bit; fixtures generated from that library are committed
 * under tests/golden/.
 *
 * Every function names the reference code it restates.  Arithmetic is done in
 * the same order as the reference (one element at a time, row-major over the
 * iteration shape, left-to-right accumulation) so f32 results are bit-equal.
 * One deliberate difference: iteration counts are 64-bit, where the reference
 * uses u32 and wraps at 2^32 points (src/backend/cpu/dispatch.c:132-138).
 *
 * Build: gcc -O2 -ffp-contract=off -shared -fPIC (see oracle/Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include "../include/thvm_cuda.h"

typedef uint32_t u32; typedef int32_t i32; typedef uint64_t u64; typedef uint16_t u16; typedef float f32;

/* ---- dtype conversion: src/tinyhvm.h:433-526 ---- */

/* f32 -> f16 bits: src/tinyhvm.h:433-457.  Rounds half up on bit 12 of the
 * mantissa; finite overflow with a non-zero mantissa yields 0x7E00-style bits. */
u16 oracle_f32_to_f16(f32 f) {
    u32 x; memcpy(&x, &f, 4);
    u32 s = (x >> 16) & 0x8000u, m = x & 0x7FFFFFu;
    i32 e = (i32)((x >> 23) & 0xFFu) - 127 + 15;
    if (e >= 31) return (u16)(s | 0x7C00u | (m ? 0x0200u : 0u));
    if (e <= 0) {
        if (e < -10) return (u16)s;
        m = (m | 0x800000u) >> (1 - e);
        if (m & 0x1000u) m += 0x2000u;
        return (u16)(s | (m >> 13));
    }
    if (m & 0x1000u) {
        m += 0x2000u;
        if (m & 0x800000u) { m = 0; e++; if (e >= 31) return (u16)(s | 0x7C00u); }
    }
    return (u16)(s | ((u32)e << 10) | (m >> 13));
}

/* f16 bits -> f32: src/tinyhvm.h:459-486 */
f32 oracle_f16_to_f32(u16 h) {
    u32 s = ((u32)h & 0x8000u) << 16, e = ((u32)h >> 10) & 0x1Fu, m = (u32)h & 0x3FFu, b;
    if (e == 0x1Fu) b = s | 0x7F800000u | (m << 13);
    else if (e) b = s | ((e + 112u) << 23) | (m << 13);
    else if (!m) b = s;
    else { e = 1; while (!(m & 0x400u)) { m <<= 1; e--; } b = s | ((e + 112u) << 23) | ((m & 0x3FFu) << 13); }
    f32 o; memcpy(&o, &b, 4); return o;
}

/* src/tinyhvm.h:488-496 */
static f32 ld(const void *p, u32 dt, u64 i) {
    switch (dt) {
        case THC_F32: return ((const f32 *)p)[i];
        case THC_F16: return oracle_f16_to_f32(((const u16 *)p)[i]);
        case THC_I32: return (f32)((const i32 *)p)[i];
        case THC_U32: return (f32)((const u32 *)p)[i];
    }
    return 0.0f;
}
/* src/tinyhvm.h:508-516 (the C casts are the platform's: cvttss2si on x86-64) */
static void st(void *p, u32 dt, u64 i, f32 v) {
    switch (dt) {
        case THC_F32: ((f32 *)p)[i] = v; break;
        case THC_F16: ((u16 *)p)[i] = oracle_f32_to_f16(v); break;
        case THC_I32: ((i32 *)p)[i] = (i32)v; break;
        case THC_U32: ((u32 *)p)[i] = (u32)v; break;
    }
}
/* src/tinyhvm.h:518-526 */
static f32 cast_via(f32 v, u32 dt) {
    switch (dt) {
        case THC_F16: return oracle_f16_to_f32(oracle_f32_to_f16(v));
        case THC_I32: return (f32)(i32)v;
        case THC_U32: return (f32)(u32)v;
    }
    return v;
}

/* ---- scalar op: src/backend/cpu/dispatch.c:5-21 ---- */
static f32 apply(u32 uop, u32 aux, f32 a, f32 b) {
    switch (uop) {
        case THC_ADD:  return a + b;
        case THC_MUL:  return a * b;
        case THC_SUB:  return a - b;
        case THC_DIV:  return b != 0.0f ? a / b : 0.0f;
        case THC_MAX:  return a > b ? a : b;
        case THC_CMP:  return a > b ? 1.0f : 0.0f;
        case THC_NEG:  return -a;
        case THC_RELU: return a > 0.0f ? a : 0.0f;
        case THC_EXP:  return expf(a);
        case THC_LOG:  return logf(a);
        case THC_SQRT: return sqrtf(a);
        case THC_CAST: return cast_via(a, aux);
    }
    return a;
}

/* ---- leaf addressing ---- */

/* single view: src/backend/cpu/dispatch.c:88-117 */
static f32 leaf_value(const void *buf, u32 dt, const thc_view_t *v, const u32 *c, u32 rank) {
    u32 n = rank < v->shape.rank ? rank : v->shape.rank;
    if (v->has_mask) {
        for (u32 d = 0; d < n; d++)
            if (c[d] < v->mask_begin[d] || c[d] >= v->mask_end[d]) return 0.0f;
        for (u32 k = 0; k < v->n_compound_masks; k++) {
            i32 t = (i32)c[v->compound_masks[k].dim_a] * v->compound_masks[k].stride_a
                  + (i32)c[v->compound_masks[k].dim_b];
            if (t < (i32)v->compound_masks[k].begin || t >= (i32)v->compound_masks[k].end) return 0.0f;
        }
    }
    i32 at = v->offset;
    for (u32 d = 0; d < n; d++) at += (i32)(c[d] % v->shape.dims[d]) * v->strides[d];
    return at < 0 ? 0.0f : ld(buf, dt, (u32)at);
}

/* stacked views: src/backend/cpu/dispatch.c:26-85.  All index math is u32. */
static f32 leaf_value_stacked(const void *buf, u32 dt, const thc_tracker_t *t, const u32 *c, u32 rank, const u32 *fdims) {
    u32 pos = 0, w = 1;
    for (i32 d = (i32)rank - 1; d >= 0; d--) { pos += c[d] * w; w *= fdims[d]; }
    for (i32 vi = (i32)t->n_views - 2; vi >= 0; vi--) {
        const thc_view_t *in = &t->views[vi], *ou = &t->views[vi + 1];
        u32 oflat = 0, run = 1, ow = 1;
        for (i32 d = (i32)ou->shape.rank - 1; d >= 0; d--) {
            u32 dim = ou->shape.dims[d];
            if (dim > 1) oflat += ((pos / run) % dim) * ow;
            run *= dim; ow *= dim;
        }
        u32 iw[THC_MAX_DIM], acc = 1;
        for (i32 d = (i32)in->shape.rank - 1; d >= 0; d--) { iw[d] = acc; acc *= in->shape.dims[d]; }
        i32 at = in->offset; u32 rem = oflat;
        for (u32 d = 0; d < in->shape.rank; d++) {
            u32 cc = rem / iw[d]; rem %= iw[d];
            if (in->has_mask && (cc < in->mask_begin[d] || cc >= in->mask_end[d])) return 0.0f;
            if (in->strides[d]) at += (i32)cc * in->strides[d];
        }
        if (at < 0) return 0.0f;
        pos = (u32)at;
    }
    return ld(buf, dt, pos);
}

static f32 read_any(const void *buf, u32 dt, const thc_view_t *v, const thc_tracker_t *t,
                    const u32 *c, u32 rank, const u32 *fdims) {
    if (t && t->n_views >= 2) return leaf_value_stacked(buf, dt, t, c, rank, fdims);
    return leaf_value(buf, dt, v, c, rank);
}

/* Optional side channel for the tests: when non-NULL during a SUM dispatch, the
 * f32 terms are also added in double precision into this array (one entry per
 * output), giving the exactly-rounded sum the f32 orders can be measured
 * against.  Not part of the reference's algorithm. */
static double *wide_sums = NULL;
void oracle_set_wide_sums(double *buf) { wide_sums = buf; }

/* ---- the fused kernel: src/backend/cpu/dispatch.c:119-282 ---- */
void oracle_dispatch_kernel_rs(void *out, const void *const *leaf_ptrs, const thc_view_t *const *leaf_views,
                               const thc_tracker_t *const *leaf_sts, u32 n_leaves,
                               const thc_fused_op_t *ops, u32 n_ops, const thc_shape_t *full,
                               const thc_reduce_spec_t *reduce, const u32 *leaf_dtypes, u32 out_dtype) {
    u32 rank = full->rank ? full->rank : 1;
    int red = reduce && reduce->reduce_type;
    u32 keepw[THC_MAX_DIM];              /* output stride of each kept dim, 0 for reduced dims */
    u64 total = 1, n_out = 1;
    for (u32 d = 0; d < rank; d++) total *= full->dims[d];
    for (i32 d = (i32)rank - 1; d >= 0; d--) {
        if (red && reduce->is_reduce[d]) keepw[d] = 0;
        else { keepw[d] = (u32)n_out; n_out *= full->dims[d]; }
    }
    if (red) {                            /* dispatch.c:148-151 */
        f32 init = reduce->reduce_type == THC_RMAX ? -1e30f : 0.0f;
        for (u64 i = 0; i < n_out; i++) st(out, out_dtype, i, init);
        if (wide_sums) for (u64 i = 0; i < n_out; i++) wide_sums[i] = 0.0;
    }
    u32 n_eval = (red && reduce->post_reduce_start) ? reduce->post_reduce_start : n_ops;
    f32 val[THC_MAX_LEAVES + THC_MAX_OPS];
    u32 c[THC_MAX_DIM] = {0};
    for (u64 flat = 0; flat < total; flat++) {
        for (u32 i = 0; i < n_leaves; i++)
            val[i] = read_any(leaf_ptrs[i], leaf_dtypes ? leaf_dtypes[i] : THC_F32, leaf_views ? leaf_views[i] : NULL,
                              leaf_sts ? leaf_sts[i] : NULL, c, rank, full->dims);
        for (u32 i = 0; i < n_eval; i++) val[n_leaves + i] = apply(ops[i].uop, ops[i].aux, val[ops[i].arg_a], val[ops[i].arg_b]);
        f32 r = n_eval ? val[n_leaves + n_eval - 1] : val[0];
        if (!red) st(out, out_dtype, flat, r);
        else {
            u64 oi = 0;
            for (u32 d = 0; d < rank; d++) oi += (u64)c[d] * keepw[d];
            f32 cur = ld(out, out_dtype, oi);
            if (wide_sums && reduce->reduce_type == THC_SUM) wide_sums[oi] += (double)r;
            st(out, out_dtype, oi, reduce->reduce_type == THC_SUM ? cur + r : (r > cur ? r : cur));
        }
        for (i32 d = (i32)rank - 1; d >= 0; d--) {           /* row-major odometer */
            if (++c[d] < full->dims[d]) break;
            c[d] = 0;
        }
    }
    /* post-reduce phase: dispatch.c:222-281 */
    if (red && reduce->post_reduce_start && reduce->post_reduce_start < n_ops) {
        u32 ps = reduce->post_reduce_start, npre = n_leaves - reduce->n_post_leaves;
        u32 zero[THC_MAX_DIM] = {0};
        memset(c, 0, sizeof c);
        for (u64 oi = 0; oi < n_out; oi++) {
            f32 rv = ld(out, out_dtype, oi);
            for (u32 i = 0; i < n_leaves; i++)
                val[i] = i < npre ? 0.0f
                       : read_any(leaf_ptrs[i], leaf_dtypes ? leaf_dtypes[i] : THC_F32, leaf_views[i],
                                  leaf_sts ? leaf_sts[i] : NULL, c, rank, zero);
            val[n_leaves + ps - 1] = rv;
            for (u32 i = ps; i < n_ops; i++) val[n_leaves + i] = apply(ops[i].uop, ops[i].aux, val[ops[i].arg_a], val[ops[i].arg_b]);
            st(out, out_dtype, oi, val[n_leaves + n_ops - 1]);
            for (i32 d = (i32)rank - 1; d >= 0; d--) {       /* odometer over the kept dims */
                if (red && reduce->is_reduce[d]) continue;
                if (++c[d] < full->dims[d]) break;
                c[d] = 0;
            }
        }
    }
}

/* ---- lowered KOP program: src/backend/cpu/uop.c:3-155 ---- */
static int kf(const thc_uop_kernel_t *k, u32 id) {
    switch (k->ops[id].type) {
        case THC_KOP_CONST_F: case THC_KOP_LOAD: case THC_KOP_ALU: case THC_KOP_ACC_INIT: case THC_KOP_MASK: return 1;
        default: return 0;
    }
}
static u32 ku(const thc_uop_kernel_t *k, u32 id, const u32 *uv, const f32 *fv) { return id >= k->n_ops ? 0 : (kf(k, id) ? (u32)fv[id] : uv[id]); }
static f32 kv(const thc_uop_kernel_t *k, u32 id, const u32 *uv, const f32 *fv) { return id >= k->n_ops ? 0.0f : (kf(k, id) ? fv[id] : (f32)uv[id]); }

static int run_span(const thc_uop_kernel_t *k, const u32 *closes, u32 from, u32 to, u32 gid,
                    void *out, const void *const *leaf, const u64 *cap, u64 out_cap, u32 *uv, f32 *fv) {
    for (u32 i = from; i < to; i++) {
        const thc_kop_t *op = &k->ops[i];
        switch (op->type) {
            case THC_KOP_NOOP: return 0;                       /* uop.c:112-113: unknown op aborts */
            case THC_KOP_GID: uv[i] = gid; break;
            case THC_KOP_CONST_U: uv[i] = op->imm.u; break;
            case THC_KOP_CONST_F: case THC_KOP_ACC_INIT: fv[i] = op->imm.f; break;
            case THC_KOP_MOD: uv[i] = op->imm.u ? ku(k, op->arg[0], uv, fv) % op->imm.u : 0; break;
            case THC_KOP_DIV: uv[i] = op->imm.u ? ku(k, op->arg[0], uv, fv) / op->imm.u : 0; break;
            case THC_KOP_IDX: uv[i] = ku(k, op->arg[0], uv, fv) * op->imm.u + ku(k, op->arg[1], uv, fv); break;
            case THC_KOP_LOAD: {
                u32 b = op->imm.u, idx = ku(k, op->arg[0], uv, fv);
                /* The reference loads unconditionally (uop.c:55-69) and faults on
                 * padded views; `cap` lets the caller state the buffer sizes so an
                 * out-of-range load reads 0, which the following MASK discards. */
                if (b == 0) fv[i] = (!cap || idx < out_cap) ? ld(out, k->out_dtype, idx) : 0.0f;
                else if (b - 1 < k->n_leaves) fv[i] = (!cap || idx < cap[b - 1]) ? ld(leaf[b - 1], k->leaf_dtypes[b - 1], idx) : 0.0f;
                else fv[i] = 0.0f;
                break;
            }
            case THC_KOP_MASK: fv[i] = kv(k, op->arg[0], uv, fv) != 0.0f ? kv(k, op->arg[1], uv, fv) : 0.0f; break;
            case THC_KOP_ALU: fv[i] = apply(op->imm.u, op->arg[2], kv(k, op->arg[0], uv, fv), kv(k, op->arg[1], uv, fv)); break;
            case THC_KOP_ACC: {
                u32 a = op->arg[0]; f32 v = kv(k, op->arg[1], uv, fv);
                fv[a] = op->imm.u == THC_RMAX ? (fv[a] > v ? fv[a] : v) : fv[a] + v;
                break;
            }
            case THC_KOP_RANGE: {
                u32 end = closes[i];
                if (end == 0xFFFFFFFFu || end <= i) return 0;
                for (u32 r = 0; r < op->imm.u; r++) {
                    uv[i] = r;
                    if (!run_span(k, closes, i + 1, end, gid, out, leaf, cap, out_cap, uv, fv)) return 0;
                }
                i = end;
                break;
            }
            case THC_KOP_ENDRANGE: break;
            case THC_KOP_STORE: st(out, k->out_dtype, ku(k, op->arg[0], uv, fv), kv(k, op->arg[1], uv, fv)); break;
            default: return 0;
        }
    }
    return 1;
}

/* `cap`/`out_cap` (elements) may be NULL/0 to load unchecked like the reference. */
void oracle_dispatch_uop_kernel(void *out, u64 out_cap, const void *const *leaf_ptrs, const u64 *cap,
                                u32 n_leaves, const thc_uop_kernel_t *k) {
    (void)n_leaves;
    static u32 closes[THC_KOP_MAX], stack[THC_KOP_MAX];
    u32 sp = 0;
    for (u32 i = 0; i < THC_KOP_MAX; i++) closes[i] = 0xFFFFFFFFu;
    for (u32 i = 0; i < k->n_ops; i++) {
        if (k->ops[i].type == THC_KOP_RANGE) stack[sp++] = i;
        else if (k->ops[i].type == THC_KOP_ENDRANGE) { if (!sp) return; closes[stack[--sp]] = i; }
    }
    if (sp) return;
    u64 total = k->local_size > 0 ? k->grid[0] : (u64)k->grid[0] * k->grid[1] * k->grid[2];
    static u32 uv[THC_KOP_MAX]; static f32 fv[THC_KOP_MAX];
    for (u64 gid = 0; gid < total; gid++) {
        memset(uv, 0, sizeof uv); memset(fv, 0, sizeof fv);
        if (!run_span(k, closes, 0, k->n_ops, (u32)gid, out, leaf_ptrs, cap, out_cap, uv, fv)) return;
    }
}

/* ---- single-op forms: src/backend/cpu/ops.c ---- */

/* flat index -> element index through a view's own shape: ops.c:4-13 (u32 math, masks ignored) */
static u32 through(u32 flat, const thc_view_t *v) {
    u32 at = (u32)v->offset;
    for (i32 d = (i32)v->shape.rank - 1; d >= 0; d--) {
        at += (flat % v->shape.dims[d]) * (u32)v->strides[d];
        flat /= v->shape.dims[d];
    }
    return at;
}

/* ops.c:15-35 */
void oracle_op_unary(u32 uop, void *dst, const thc_view_t *dv, u32 ddt, const void *src, const thc_view_t *sv, u32 sdt) {
    for (u32 i = 0; i < dv->numel; i++) {
        f32 x = ld(src, sdt, through(i, sv));
        if (uop == THC_NEG || uop == THC_RELU || uop == THC_EXP || uop == THC_LOG || uop == THC_SQRT) x = apply(uop, 0, x, 0.0f);
        st(dst, ddt, i, x);
    }
}
/* ops.c:37-61 */
void oracle_op_binary(u32 uop, void *dst, const thc_view_t *dv, u32 ddt, const void *a, const thc_view_t *av, u32 adt,
                      const void *b, const thc_view_t *bv, u32 bdt) {
    for (u32 i = 0; i < dv->numel; i++) {
        f32 x = ld(a, adt, through(i, av)), y = ld(b, bdt, through(i, bv));
        int known = uop == THC_ADD || uop == THC_MUL || uop == THC_DIV || uop == THC_SUB || uop == THC_MAX || uop == THC_CMP;
        st(dst, ddt, i, known ? apply(uop, 0, x, y) : x);
    }
}
/* ops.c:99-112 (the non-BLAS branch, which is the one Linux builds) */
void oracle_op_mm(void *dst, u32 ddt, const void *a, const thc_view_t *av, u32 adt, const void *b, const thc_view_t *bv, u32 bdt,
                  u32 M, u32 K, u32 N) {
    for (u32 i = 0; i < M; i++)
        for (u32 j = 0; j < N; j++) {
            f32 s = 0;
            for (u32 k = 0; k < K; k++) s += ld(a, adt, through(i * K + k, av)) * ld(b, bdt, through(k * N + j, bv));
            st(dst, ddt, (u64)i * N + j, s);
        }
}
/* ops.c:114-130 */
void oracle_op_reduce(u32 uop, void *dst, u32 dst_numel, u32 ddt, const void *src, u32 sdt, u32 reduce_dim) {
    for (u32 o = 0; o < dst_numel; o++) {
        f32 acc = uop == THC_RMAX ? -1e30f : 0.0f;
        for (u32 r = 0; r < reduce_dim; r++) {
            f32 v = ld(src, sdt, (u64)o * reduce_dim + r);
            if (uop == THC_SUM) acc += v; else if (uop == THC_RMAX) acc = v > acc ? v : acc;
        }
        st(dst, ddt, o, acc);
    }
}

/* ---- behaviours only an MSL shader defines ---- */

/* Adam: src/shaders.metal:406-420 */
void oracle_adam_step(f32 *p, const f32 *g, f32 *m, f32 *v, f32 lr, f32 b1, f32 b2, f32 eps, f32 bc1, f32 bc2, u32 n) {
    for (u32 i = 0; i < n; i++) {
        f32 gi = g[i];
        f32 mi = b1 * m[i] + (1.0f - b1) * gi;
        f32 vi = b2 * v[i] + (1.0f - b2) * gi * gi;
        m[i] = mi; v[i] = vi;
        p[i] -= lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    }
}

/* 2x2/2 max-pool with window index: src/shaders.metal:427-458.  Scan order
 * (0,0),(0,1),(1,0),(1,1); strict '>' so the first maximum wins; index u8 0..3. */
void oracle_maxpool2x2_index(const f32 *x, f32 *y, uint8_t *idx, u32 BC, u32 H, u32 W) {
    u32 OH = H / 2, OW = W / 2;
    for (u32 p = 0; p < BC; p++)
        for (u32 oy = 0; oy < OH; oy++)
            for (u32 ox = 0; ox < OW; ox++) {
                const f32 *w = x + (u64)p * H * W + (u64)(2 * oy) * W + 2 * ox;
                f32 best = w[0]; uint8_t bi = 0;
                if (w[1] > best) { best = w[1]; bi = 1; }
                if (w[W] > best) { best = w[W]; bi = 2; }
                if (w[W + 1] > best) { best = w[W + 1]; bi = 3; }
                u64 o = ((u64)p * OH + oy) * OW + ox;
                y[o] = best; if (idx) idx[o] = bi;
            }
}

/* argmax per row, first strictly greater wins: src/ops/_.c:502-524 */
void oracle_argmax_rows(const f32 *x, u32 rows, u32 cols, u32 *out) {
    for (u32 r = 0; r < rows; r++) {
        u32 best = 0;
        for (u32 c = 1; c < cols; c++) if (x[(u64)r * cols + c] > x[(u64)r * cols + best]) best = c;
        out[r] = best;
    }
}

/* ---- signature: src/tinyhvm.h:766-856 ---- */
static u64 mixin(u64 h, u64 v) { return (h ^ v) * 0x100000001b3ULL; }
static u64 hash_view(u64 h, const thc_view_t *v) {
    if (!v) return mixin(h, 0);
    h = mixin(h, v->shape.rank); h = mixin(h, v->numel); h = mixin(h, (u64)(u32)v->offset); h = mixin(h, v->has_mask);
    for (u32 d = 0; d < v->shape.rank && d < THC_MAX_DIM; d++) {
        h = mixin(h, v->shape.dims[d]); h = mixin(h, (u64)(u32)v->strides[d]);
        if (v->has_mask) { h = mixin(h, v->mask_begin[d]); h = mixin(h, v->mask_end[d]); }
        h = mixin(h, v->mod_size[d]);
    }
    h = mixin(h, v->n_compound_masks);
    for (u32 i = 0; i < v->n_compound_masks && i < 2; i++) {
        h = mixin(h, v->compound_masks[i].dim_a); h = mixin(h, v->compound_masks[i].dim_b);
        h = mixin(h, (u64)(u32)v->compound_masks[i].stride_a);
        h = mixin(h, v->compound_masks[i].begin); h = mixin(h, v->compound_masks[i].end);
    }
    return h;
}
u64 oracle_signature(const thc_fused_op_t *ops, u32 n_ops, const thc_view_t *const *views, const thc_tracker_t *const *sts,
                     u32 n_leaves, const thc_shape_t *full, const thc_reduce_spec_t *red) {
    u64 h = 0x5448564d4b45524eULL;
    h = mixin(h, n_ops); h = mixin(h, n_leaves);
    for (u32 i = 0; i < n_ops; i++) { h = mixin(h, ops[i].uop); h = mixin(h, ops[i].arg_a); h = mixin(h, ops[i].arg_b); h = mixin(h, ops[i].aux); }
    if (!full) h = mixin(h, 0);
    else { h = mixin(h, full->rank); for (u32 d = 0; d < full->rank && d < THC_MAX_DIM; d++) h = mixin(h, full->dims[d]); }
    if (!red) h = mixin(h, 0);
    else {
        h = mixin(h, red->reduce_type); h = mixin(h, red->post_reduce_start); h = mixin(h, red->n_post_leaves);
        h = mixin(h, red->reduce2_type); h = mixin(h, red->reduce2_start);
        for (u32 d = 0; d < THC_MAX_DIM; d++) { h = mixin(h, red->is_reduce[d]); h = mixin(h, red->is_reduce2[d]); }
    }
    for (u32 i = 0; i < n_leaves; i++) {
        const thc_tracker_t *t = sts ? sts[i] : NULL;
        if (!t || !t->n_views) h = hash_view(h, views ? views[i] : NULL);
        else { h = mixin(h, t->n_views); for (u32 k = 0; k < t->n_views && k < THC_MAX_VIEWS; k++) h = hash_view(h, &t->views[k]); }
    }
    return mixin(h, 0);
}
