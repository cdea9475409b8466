/* ref_host.c — the reference's whole host runtime (interaction-net reducer,
 * fuser, scheduler, lowerer, nn library) compiled from its own sources,
 * together with its CPU backend and the CUDA backend hub, plus staged driver
 * programs for the benchmark configs.
 *
 * TEST INFRASTRUCTURE ONLY.  No reference code is copied here: the reference's
 * translation units are `#include`d from the reference checkout (include path
 * from oracle/Makefile), the same way its own tests include them
 * (test/test_mm_dup_2arm.m:14-18).  The library lands in oracle/_ref/.
 *
 * What it is for: the SAME driver program is run with thvm_init("cpu") and
 * thvm_init("cuda"); every realised tensor is kept, and the tests compare the
 * two runs tensor by tensor.  With "cuda" the reference's scheduler calls
 * libthvm_cuda.so through the vtable hub, which is the drop-in path end to end.
 *
 * The drivers are "staged" (explicit realise points, tree-shaped expressions,
 * hand-written VJPs from forward UOps following the rule bodies of
 * src/interact/grad.c) because the reference's own autograd, padded conv2d and
 * batchnorm_forward do not run on Linux at this snapshot.
 */
#define thvm_init thvm_init_base
#include "tinyhvm.c"
#undef thvm_init
#include "backend/cpu/_.c"
#include "nn/_.c"
#include "../tinyhvm_b200/backend_cuda/_.c"
#include <time.h>

#include "ref_trace.c"

TinyHVM *thvm_init(const char *device) {
    TinyHVM *ctx = thvm_init_device(thvm_init_base, device);
    if (device && strncmp(device, "record", 6) == 0) {            /* "record" or "record-dry" */
        tr_dry = strcmp(device, "record-dry") == 0;
        ctx->backends[THVM_DEV_CUDA] = &rec_backend;
        ctx->n_backends = THVM_DEV_CUDA + 1;
        ctx->default_device = THVM_DEV_CUDA;
    }
    return ctx;
}

/* ------------------------------------------------------------------ the reference's lowerer at the vtable boundary
 * A dispatch in the form dispatch_kernel_rs receives (views, trackers, ops, iteration shape, reduce spec, dtypes) is put
 * into a KernelEntry and lowered by the reference's own thvm_lower_kernel_uop (src/lower/_.c:765-973), the way
 * thvm_sched_dispatch_kernel does before it calls dispatch_uop_kernel (src/schedule/_.c:2343-2378).  Returns 1 when a
 * program was produced.  The output dtype is f32 (the scheduler takes it from the output tensor). */
int drv_lower_dispatch(const View *const *views, const ShapeTracker *const *sts, u32 n_leaves, const FusedOp *ops, u32 n_ops,
                       const Shape *full, const ReduceSpec *red, const u32 *leaf_dtypes, UOpKernel *out) {
    static TinyHVM *lctx = NULL;
    static KernelEntry ke;
    if (!lctx) lctx = thvm_init_base("cpu");
    if (!lctx || n_leaves > FUSE_MAX_LEAVES || n_ops > FUSE_MAX_OPS) return 0;
    memset(&ke, 0, sizeof ke);
    for (u32 i = 0; i < n_ops; i++) ke.ops[i] = ops[i];
    ke.n_ops = n_ops;
    for (u32 i = 0; i < n_leaves; i++) {
        ke.leaf_ids[i] = 0xFFFFFFFFu; ke.leaf_kinds[i] = KERNEL_LEAF_TENSOR;
        ke.leaf_dtypes[i] = leaf_dtypes ? leaf_dtypes[i] : DTYPE_F32;
        ke.leaf_views[i] = *views[i];
        if (sts && sts[i]) ke.leaf_sts[i] = *sts[i];
        else { ke.leaf_sts[i].views[0] = *views[i]; ke.leaf_sts[i].n_views = 1; }
    }
    ke.n_leaves = n_leaves;
    ke.full_shape = *full; ke.raw_out_shape = *full; ke.out_shape = *full;
    if (red && red->reduce_type) { ke.reduce = *red; ke.has_reduce = red->reduce_type; }
    ke.output_tid = 0xFFFFFFFFu; ke.raw_output_tid = 0xFFFFFFFFu;
    return thvm_lower_kernel_uop(lctx, &ke, out, NULL);
}

/* ------------------------------------------------------------------ results */
#define DRV_MAX 512
static struct { char name[64]; f32 *data; u32 n; } drv_res[DRV_MAX];
static u32 drv_n = 0;
static double drv_secs = 0.0;

void drv_clear(void) { for (u32 i = 0; i < drv_n; i++) free(drv_res[i].data); drv_n = 0; }
u32 drv_count(void) { return drv_n; }
const char *drv_name(u32 i) { return i < drv_n ? drv_res[i].name : ""; }
u32 drv_numel(u32 i) { return i < drv_n ? drv_res[i].n : 0; }
const f32 *drv_data(u32 i) { return i < drv_n ? drv_res[i].data : NULL; }
double drv_seconds(void) { return drv_secs; }

static double now_s(void) { struct timespec t; clock_gettime(CLOCK_MONOTONIC, &t); return t.tv_sec + 1e-9 * t.tv_nsec; }

/* realise a term: thvm_eval + force, as tensor_realize does (src/nn/tensor_api.c:18-24) */
static Term realize(TinyHVM *ctx, Term t) { Tensor x = tensor_realize(tensor_from_term(ctx, t)); return x.term; }

/* keep a host copy of a realised tensor under `name` */
static void keep(TinyHVM *ctx, const char *name, Term t) {
    if (drv_n >= DRV_MAX) return;
    u32 n = 1, dt = DTYPE_F32;
    Shape sh = {0};
    f32 *h = (f32 *)thvm_to_host_raw(ctx, t, &dt, &sh);          /* forces lazy views of realised tensors too */
    for (u32 d = 0; d < sh.rank; d++) n *= sh.dims[d];
    if (dt != DTYPE_F32) h = NULL;
    snprintf(drv_res[drv_n].name, sizeof drv_res[drv_n].name, "%s", name);
    drv_res[drv_n].n = h ? n : 0;
    drv_res[drv_n].data = h ? malloc((size_t)n * 4) : NULL;
    if (h) memcpy(drv_res[drv_n].data, h, (size_t)n * 4);
    drv_n++;
}

static Term scalar(TinyHVM *ctx, f32 v) { return thvm_scalar(ctx, v); }
static Term op2(TinyHVM *ctx, u32 uop, Term a, Term b) { return thvm_op(ctx, uop, a, b); }
static Term op1(TinyHVM *ctx, u32 uop, Term a) { return thvm_op(ctx, uop, a, term_era()); }
static Term transpose2(TinyHVM *ctx, Term t) { return thvm_permute(ctx, t, (u32[]){1, 0}, 2); }
/* A realised bare reduce keeps its un-reshaped view ([M,1,N] for a matmul).  The
 * realised TAG_TEN may be shared freely, but a lazy view of it is a linear term:
 * every consumer gets its own fresh reshape from as2()/as1(). */
static Term mm_raw(TinyHVM *ctx, Term a, Term b) { return realize(ctx, thvm_mm(ctx, a, b)); }
static Term as2(TinyHVM *ctx, Term raw, u32 M, u32 N) { return thvm_reshape(ctx, raw, SHAPE(M, N)); }
static Term as1(TinyHVM *ctx, Term raw, u32 N) { return thvm_reshape(ctx, raw, SHAPE(N)); }

/* ------------------------------------------------------------------ config 2 */
/* y = sum_last(relu(a*b+c)) and its VJP w.r.t. a for a ones seed, g = b*(a*b+c > 0) */
int drv_chain(const char *dev, u32 R, u32 C, const f32 *a, const f32 *b, const f32 *c) {
    TinyHVM *ctx = thvm_init(dev);
    Term ta = thvm_tensor(ctx, a, SHAPE(R, C)), tb = thvm_tensor(ctx, b, SHAPE(R, C)), tc = thvm_tensor(ctx, c, SHAPE(R, C));
    double t0 = now_s();
    Term u = op2(ctx, UOP_ADD, op2(ctx, UOP_MUL, ta, tb), tc);
    Term y = realize(ctx, thvm_sum_axes(ctx, op1(ctx, UOP_RELU, u), (u32[]){1}, 1));
    Term u2 = op2(ctx, UOP_ADD, op2(ctx, UOP_MUL, ta, tb), tc);               /* rebuilt: tree-shaped */
    Term g = realize(ctx, op2(ctx, UOP_MUL, tb, op2(ctx, UOP_CMP, u2, scalar(ctx, 0.f))));
    f32 *hy = thvm_to_host(ctx, y); (void)hy;
    drv_secs = now_s() - t0;
    keep(ctx, "y", y); keep(ctx, "g", g);
    thvm_free(ctx);
    return 0;
}

/* ------------------------------------------------------------------ config 3 */
/* C = A@B, L = sum(C*C), dC = 2C, dA = dC@B^T, dB = A^T@dC  (n x n) */
int drv_gemm(const char *dev, u32 n, const f32 *A, const f32 *B) {
    TinyHVM *ctx = thvm_init(dev);
    Term tA = thvm_tensor(ctx, A, SHAPE(n, n)), tB = thvm_tensor(ctx, B, SHAPE(n, n));
    double t0 = now_s();
    Term C = mm_raw(ctx, tA, tB);
    Term L = realize(ctx, thvm_sum_axes(ctx, op2(ctx, UOP_MUL, as2(ctx, C, n, n), as2(ctx, C, n, n)), (u32[]){0, 1}, 2));
    Term dC = realize(ctx, op2(ctx, UOP_MUL, as2(ctx, C, n, n), scalar(ctx, 2.f)));
    Term dA = mm_raw(ctx, dC, transpose2(ctx, tB));
    Term dB = mm_raw(ctx, transpose2(ctx, tA), dC);
    f32 *h = thvm_to_host(ctx, L); (void)h;
    drv_secs = now_s() - t0;
    keep(ctx, "C", C); keep(ctx, "L", L); keep(ctx, "dA", dA); keep(ctx, "dB", dB);
    thvm_free(ctx);
    return 0;
}

/* ------------------------------------------------------------------ shared pieces */
/* softmax cross-entropy backward: dlogits = (softmax(l) - onehot) / B, staged */
static Term ce_backward(TinyHVM *ctx, Term logits, const u8 *labels, u32 B, u32 C) {
    Term m = realize(ctx, thvm_rmax_axes(ctx, logits, (u32[]){1}, 1));                       /* [B,1] */
    Term e = realize(ctx, op1(ctx, UOP_EXP, op2(ctx, UOP_SUB, logits, thvm_expand(ctx, m, SHAPE(B, C)))));
    Term s = realize(ctx, thvm_sum_axes(ctx, e, (u32[]){1}, 1));                             /* [B,1] */
    f32 *oh = calloc((size_t)B * C, 4);
    for (u32 i = 0; i < B; i++) oh[i * C + labels[i]] = 1.0f;
    rec_note("onehot", 0);
    Term onehot = thvm_tensor(ctx, oh, SHAPE(B, C));
    free(oh);
    Term p = op2(ctx, UOP_DIV, e, thvm_expand(ctx, s, SHAPE(B, C)));
    return realize(ctx, op2(ctx, UOP_MUL, op2(ctx, UOP_SUB, p, onehot), scalar(ctx, 1.0f / (f32)B)));
}

/* y = x@W + b, realised, as [B,N] */
static Term linear_fwd(TinyHVM *ctx, Term x, Term W, Term b, u32 B, u32 N) {
    /* same composition as thvm_tg_linear (src/nn/tg_tensor.c:34-88), which insists
     * on a realised x; here x may be a lazy view of a realised tensor */
    Term bc = thvm_expand(ctx, thvm_reshape(ctx, b, SHAPE(1, N)), SHAPE(B, N));
    return realize(ctx, op2(ctx, UOP_ADD, thvm_mm(ctx, x, W), bc));
}

/* ------------------------------------------------------------------ config 1 */
/* 2-layer MLP: loss and the four gradients */
int drv_mlp(const char *dev, u32 B, u32 I, u32 H, u32 O, const f32 *x, const f32 *W1, const f32 *b1,
            const f32 *W2, const f32 *b2, const u8 *labels) {
    TinyHVM *ctx = thvm_init(dev);
    Term tx = thvm_tensor(ctx, x, SHAPE(B, I));
    Term tW1 = thvm_tensor(ctx, W1, SHAPE(I, H)), tb1 = thvm_tensor(ctx, b1, SHAPE(H));
    Term tW2 = thvm_tensor(ctx, W2, SHAPE(H, O)), tb2 = thvm_tensor(ctx, b2, SHAPE(O));
    double t0 = now_s();
    Term u = linear_fwd(ctx, tx, tW1, tb1, B, H);                                            /* pre-activation */
    Term h = realize(ctx, op1(ctx, UOP_RELU, u));
    Term logits = linear_fwd(ctx, h, tW2, tb2, B, O);
    Term loss = realize(ctx, cross_entropy_loss(ctx, logits, (u8 *)labels, B, O));
    Term dl = ce_backward(ctx, logits, labels, B, O);
    Term dW2 = mm_raw(ctx, transpose2(ctx, h), dl);
    Term db2 = realize(ctx, thvm_sum_axes(ctx, dl, (u32[]){0}, 1));
    Term dh = mm_raw(ctx, dl, transpose2(ctx, tW2));
    Term du = realize(ctx, op2(ctx, UOP_MUL, as2(ctx, dh, B, H), op2(ctx, UOP_CMP, u, scalar(ctx, 0.f))));
    Term dW1 = mm_raw(ctx, transpose2(ctx, tx), du);
    Term db1 = realize(ctx, thvm_sum_axes(ctx, du, (u32[]){0}, 1));
    f32 *hl = thvm_to_host(ctx, loss); (void)hl;
    drv_secs = now_s() - t0;
    keep(ctx, "loss", loss); keep(ctx, "dW1", dW1); keep(ctx, "db1", db1); keep(ctx, "dW2", dW2); keep(ctx, "db2", db2);
    keep(ctx, "logits", logits);
    thvm_free(ctx);
    return 0;
}

#include "ref_host_cnn.c"
