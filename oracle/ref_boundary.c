/* ref_boundary.c — exports the reference's own CPU backend at the vtable
 * boundary, so tests can run identical dispatches through the real reference
 * code and through the restatement in thvm_oracle.c.
 *
 * TEST INFRASTRUCTURE ONLY.  This file contains no reference code: it
 * `#include`s the reference's CPU backend hub from the reference checkout
 * (include path given by oracle/Makefile) and forwards to the `cpu_backend`
 * vtable it defines (src/backend/cpu/_.c:21-35).  The resulting library lands
 * in oracle/_ref/, which is not version-controlled.
 */
#include "backend/cpu/_.c"
#include "../include/thvm_cuda.h"

/* layout checks: the mirrors in include/thvm_cuda.h against the reference */
_Static_assert(sizeof(thc_shape_t) == sizeof(Shape), "Shape");
_Static_assert(sizeof(thc_view_t) == sizeof(View), "View");
_Static_assert(offsetof(thc_view_t, mask_begin) == offsetof(View, mask_begin), "View.mask_begin");
_Static_assert(offsetof(thc_view_t, compound_masks) == offsetof(View, compound_masks), "View.compound_masks");
_Static_assert(offsetof(thc_view_t, mod_size) == offsetof(View, mod_size), "View.mod_size");
_Static_assert(sizeof(thc_tracker_t) == sizeof(ShapeTracker), "ShapeTracker");
_Static_assert(sizeof(thc_fused_op_t) == sizeof(FusedOp), "FusedOp");
_Static_assert(sizeof(thc_reduce_spec_t) == sizeof(ReduceSpec), "ReduceSpec");
_Static_assert(offsetof(thc_reduce_spec_t, is_reduce2) == offsetof(ReduceSpec, is_reduce2), "ReduceSpec.is_reduce2");
_Static_assert(sizeof(thc_kop_t) == sizeof(KOp), "KOp");
_Static_assert(sizeof(thc_uop_kernel_t) == sizeof(UOpKernel), "UOpKernel");
_Static_assert(offsetof(thc_uop_kernel_t, leaf_views) == offsetof(UOpKernel, leaf_views), "UOpKernel.leaf_views");
_Static_assert(offsetof(thc_uop_kernel_t, out_dtype) == offsetof(UOpKernel, out_dtype), "UOpKernel.out_dtype");
_Static_assert(THC_MAX_BUFS == MAX_BUFS, "MAX_BUFS");

int   ref_init(void)                       { return cpu_backend.init(); }
void  ref_shutdown(void)                   { cpu_backend.shutdown(); }
u32   ref_buf_alloc(u64 bytes)             { return cpu_backend.buf_alloc(bytes); }
void  ref_buf_write(u32 id, const void *d, u64 b) { cpu_backend.buf_write(id, d, b); }
void  ref_buf_read(u32 id, void *o, u64 b) { cpu_backend.buf_read(id, o, b); }
void  ref_pool_reset(u32 keep)             { cpu_backend.pool_reset(keep); }
void  ref_op_unary(u32 uop, u32 dst, const View *dv, u32 ddt, u32 src, const View *sv, u32 sdt)
      { cpu_backend.op_unary(uop, dst, dv, ddt, src, sv, sdt); }
void  ref_op_binary(u32 uop, u32 dst, const View *dv, u32 ddt, u32 a, const View *av, u32 adt, u32 b, const View *bv, u32 bdt)
      { cpu_backend.op_binary(uop, dst, dv, ddt, a, av, adt, b, bv, bdt); }
void  ref_op_mm(u32 dst, u32 ddt, u32 a, const View *av, u32 adt, u32 b, const View *bv, u32 bdt, u32 M, u32 K, u32 N)
      { cpu_backend.op_mm(dst, ddt, a, av, adt, b, bv, bdt, M, K, N); }
void  ref_op_reduce(u32 uop, u32 dst, u32 dn, u32 ddt, u32 src, u32 sn, u32 sdt, u32 rd)
      { cpu_backend.op_reduce(uop, dst, dn, ddt, src, sn, sdt, rd); }
void  ref_dispatch_kernel_rs(u32 out_buf, u32 *leaf_bufs, const View **leaf_views, const ShapeTracker *const *leaf_sts,
                             u32 n_leaves, FusedOp *ops, u32 n_ops, const Shape *full_shape, const ReduceSpec *reduce,
                             const u32 *leaf_dtypes, u32 out_dtype)
      { cpu_backend.dispatch_kernel_rs(out_buf, leaf_bufs, leaf_views, leaf_sts, n_leaves, ops, n_ops, full_shape,
                                       reduce, NULL, NULL, 0, leaf_dtypes, out_dtype); }
void  ref_dispatch_uop_kernel(u32 out_buf, const u32 *leaf_bufs, u32 n_leaves, const UOpKernel *k)
      { cpu_backend.dispatch_uop_kernel(out_buf, leaf_bufs, n_leaves, k, 0); }
u64   ref_signature(const FusedOp *ops, u32 n_ops, const View *const *views, const ShapeTracker *const *sts, u32 n_leaves,
                    const Shape *full, const ReduceSpec *red)
      { return thvm_kernel_signature_from_ptrs(ops, n_ops, views, sts, n_leaves, full, red, NULL, 0); }
u16   ref_f32_to_f16(f32 f) { return f32_to_f16_bits(f); }
f32   ref_f16_to_f32(u16 h) { return f16_bits_to_f32(h); }
