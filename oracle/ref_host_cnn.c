/* ref_host_cnn.c — staged CNN training steps (LeNet-5, VGG-style) written with
 * the reference's own lazy-tensor API; included by ref_host.c.
 *
 * TEST INFRASTRUCTURE ONLY (see ref_host.c).  Every backward expression follows
 * the rule body of the reference's autograd it stands in for:
 *   RELU   da * CMP(a,0)                         src/interact/grad.c:194-202
 *   MM     gy @ b^T,  a^T @ gy                   src/interact/grad.c:483-496
 *   RMAX   da * (1 - CMP(expand(rmax(a)), a))    src/interact/grad.c:406-425 (ties all get the gradient)
 *   EXPAND sum to the source shape               src/interact/grad.c:379-404
 *   PAD <-> SHRINK                               src/interact/grad.c:317-373
 * Staging rules: a realised TAG_TEN may be shared; every lazy view is rebuilt
 * per consumer; padding is materialised (ADD(pad(x),0)) before a convolution;
 * a permute is materialised before a rank-changing reshape.
 */

/* The reference's lowered CPU path loads before it masks and walks off the buffer
 * on padded views (src/lower/_.c:303-307, src/backend/cpu/uop.c:55-69); its
 * FusedOp interpreter handles them, so CPU runs of programs with padding use it. */
static void cpu_masked_leaf_workaround(const char *dev) {
    if (strcmp(dev, "cpu") == 0) setenv("THVM_NO_LOWER", "1", 1); else unsetenv("THVM_NO_LOWER");
}

static Term as4(TinyHVM *ctx, Term raw, u32 a, u32 b, u32 c, u32 d) { return thvm_reshape(ctx, raw, SHAPE(a, b, c, d)); }
static Term sum023(TinyHVM *ctx, Term t) { return thvm_sum_axes(ctx, t, (u32[]){0, 2, 3}, 3); }

/* zero padding of H and W by p, materialised */
static Term pad_hw(TinyHVM *ctx, Term x, u32 p) {
    if (!p) return x;
    u32 pairs[8] = {0, 0, 0, 0, p, p, p, p};
    return realize(ctx, op2(ctx, UOP_ADD, thvm_pad(ctx, x, pairs, 4), scalar(ctx, 0.f)));
}

/* conv (stride 1, input already padded) + optional bias; returns the realised pre-activation */
static Term conv_fwd(TinyHVM *ctx, Term xp, Term W, Term bias) {
    return realize(ctx, thvm_conv2d(ctx, xp, W, bias, 1, (u32[]){1, 1}, (u32[]){0, 0, 0, 0}));
}

/* dW[Co,Ci,K,K] = sum over B,OH,OW of window(xp) * g : a 7-D MUL + SUM{0,3,4}; raw result */
static Term conv_wgrad(TinyHVM *ctx, Term xp, Term g4, u32 B, u32 Ci, u32 Co, u32 OH, u32 OW, u32 K) {
    Term P = thvm_pool(ctx, xp, (u32[]){K, K}, (u32[]){1, 1}, 2);                       /* [B,Ci,OH,OW,K,K] */
    Term xr = thvm_expand(ctx, thvm_reshape(ctx, P, SHAPE(B, 1, Ci, OH, OW, K, K)), SHAPE(B, Co, Ci, OH, OW, K, K));
    Term gr = thvm_expand(ctx, thvm_reshape(ctx, g4, SHAPE(B, Co, 1, OH, OW, 1, 1)), SHAPE(B, Co, Ci, OH, OW, K, K));
    return realize(ctx, thvm_sum_axes(ctx, op2(ctx, UOP_MUL, xr, gr), (u32[]){0, 3, 4}, 3));
}

/* gradient w.r.t. the (padded) conv input: full correlation of the K-1 padded
 * upstream gradient with the spatially flipped, channel-transposed weight.  A flip is
 * not expressible as a view (the lowerer rejects negative strides,
 * src/lower/_.c:452-455), so it is computed on the device as a contraction with a
 * constant 0/1 tensor, Wf[c,o,p',q'] = sum_{p,q} W[o,c,p,q] * J[p,q,p',q'] with
 * J = 1 where p+p' = q+q' = K-1 (exact: one product per output is W*1, the rest W*0),
 * then permuted and materialised.  Raw result, logical shape [B,Ci,OH+K-1,OW+K-1]. */
static Term conv_dgrad(TinyHVM *ctx, Term g4, Term W, u32 Ci, u32 Co, u32 K) {
    f32 *J = calloc((size_t)K * K * K * K, 4);
    for (u32 p = 0; p < K; p++) for (u32 q = 0; q < K; q++) J[((p * K + q) * K + (K - 1 - p)) * K + (K - 1 - q)] = 1.0f;
    Term tJ = thvm_tensor(ctx, J, SHAPE(1, 1, K, K, K, K));
    free(J);
    Term Wr = thvm_expand(ctx, thvm_reshape(ctx, W, SHAPE(Co, Ci, K, K, 1, 1)), SHAPE(Co, Ci, K, K, K, K));
    Term Jr = thvm_expand(ctx, tJ, SHAPE(Co, Ci, K, K, K, K));
    Term flipped = realize(ctx, thvm_sum_axes(ctx, op2(ctx, UOP_MUL, Wr, Jr), (u32[]){2, 3}, 2));     /* raw [Co,Ci,1,1,K,K] */
    Term Wf = realize(ctx, op2(ctx, UOP_ADD, thvm_permute(ctx, as4(ctx, flipped, Co, Ci, K, K), (u32[]){1, 0, 2, 3}, 4), scalar(ctx, 0.f)));
    Term gp = pad_hw(ctx, g4, K - 1);
    return realize(ctx, thvm_conv2d(ctx, gp, Wf, term_era(), 1, (u32[]){1, 1}, (u32[]){0, 0, 0, 0}));
}

/* 2x2/2 max-pool forward; raw result [B,C,OH,OW,1,1] */
static Term pool_fwd(TinyHVM *ctx, Term a4) { return realize(ctx, thvm_maxpool2d(ctx, a4, (u32[]){2, 2}, (u32[]){2, 2})); }

static Term pool_window(TinyHVM *ctx, Term a4, u32 B, u32 C, u32 OH, u32 OW) {
    return thvm_permute(ctx, thvm_reshape(ctx, a4, SHAPE(B, C, OH, 2, OW, 2)), (u32[]){0, 1, 2, 4, 3, 5}, 6);
}

/* max-pool backward, mask form; returns a realised contiguous [B,C,OH,2,OW,2] buffer (= [B,C,H,W]) */
static Term pool_bwd(TinyHVM *ctx, Term a4, Term m_raw, Term g_raw, u32 B, u32 C, u32 OH, u32 OW) {
    Term m6 = thvm_expand(ctx, thvm_reshape(ctx, m_raw, SHAPE(B, C, OH, OW, 1, 1)), SHAPE(B, C, OH, OW, 2, 2));
    Term mask = op2(ctx, UOP_SUB, scalar(ctx, 1.f), op2(ctx, UOP_CMP, m6, pool_window(ctx, a4, B, C, OH, OW)));
    Term g6 = thvm_expand(ctx, thvm_reshape(ctx, g_raw, SHAPE(B, C, OH, OW, 1, 1)), SHAPE(B, C, OH, OW, 2, 2));
    Term dwin = realize(ctx, op2(ctx, UOP_MUL, g6, mask));
    return realize(ctx, op2(ctx, UOP_ADD, thvm_permute(ctx, dwin, (u32[]){0, 1, 2, 4, 3, 5}, 6), scalar(ctx, 0.f)));
}

/* relu backward: g * (u > 0), realised */
static Term relu_bwd(TinyHVM *ctx, Term g, Term u) { return realize(ctx, op2(ctx, UOP_MUL, g, op2(ctx, UOP_CMP, u, scalar(ctx, 0.f)))); }

/* SGD write-back: w <- w - lr * g  (ASSIGN rule, src/interact/tensor_ops.c:3-160) */
static void sgd(TinyHVM *ctx, Term w, Term g_view, f32 lr) {
    rec_note("lr", 0);
    thvm_eval(ctx, thvm_assign(ctx, w, op2(ctx, UOP_SUB, w, op2(ctx, UOP_MUL, g_view, scalar(ctx, lr)))));
}

/* ---- data parallelism: the driver runs on one shard of the batch per process; after
 * the backward pass it hands the gradient buffers to a hook that sums them across
 * the processes (NCCL inside libthvm_cuda.so for "cuda"; the CPU tests plug in a
 * gloo exchange), and the update uses lr / world. ---- */
typedef int (*DrvDpHook)(const u32 *buf_ids, const u64 *counts, u32 n);
typedef void (*DrvAfterInit)(void);
static DrvDpHook drv_dp_hook = NULL;
static DrvAfterInit drv_after_init = NULL;
static u32 drv_dp_world = 1;
void drv_set_dp(u32 world, DrvDpHook hook, DrvAfterInit after_init) { drv_dp_world = world ? world : 1; drv_dp_hook = hook; drv_after_init = after_init; }
/* host access to a buffer of the default backend, for hooks that exchange through the host */
void drv_buf_read(TinyHVM *ctx, u32 buf_id, void *out, u64 bytes) { ctx_default_backend(ctx)->buf_read(buf_id, out, bytes); }
void drv_buf_write(TinyHVM *ctx, u32 buf_id, const void *src, u64 bytes) { ctx_default_backend(ctx)->buf_write(buf_id, src, bytes); }
static TinyHVM *drv_ctx = NULL;
TinyHVM *drv_current_ctx(void) { return drv_ctx; }

static void dp_sum_grads(TinyHVM *ctx, const Term *grads, u32 n) {
    if (!drv_dp_hook) return;
    u32 ids[32]; u64 counts[32];
    for (u32 i = 0; i < n && i < 32; i++) {
        TensorMeta *m = &ctx->tensors[(u32)term_val(grads[i])];
        ids[i] = m->buf_id; counts[i] = m->view.numel;
    }
    if (drv_dp_hook(ids, counts, n) != 0) { fprintf(stderr, "drv: gradient all-reduce failed\n"); exit(1); }
}

static void keepf(TinyHVM *ctx, const char *fmt, u32 step, Term t) { char nm[64]; snprintf(nm, sizeof nm, fmt, step); keep(ctx, nm, t); }

/* ------------------------------------------------------------------ config 4: LeNet-5 */
/* params (flat, in this order): W1[6,1,5,5] b1[6] W2[16,6,5,5] b2[16] W3[400,120] b3[120] W4[120,84] b4[84] W5[84,10] b5[10]
 * x[steps][B,1,28,28], labels[steps][B].  Keeps the loss of every step, the
 * gradients of step 0 and the parameters after the last step. */
/* replace the kept tensor `name` by host values (the loss of a captured step is known only after its replay) */
static void keep_host(const char *name, const f32 *v, u32 n) {
    for (u32 i = 0; i < drv_n; i++)
        if (strcmp(drv_res[i].name, name) == 0) { free(drv_res[i].data); drv_res[i].data = malloc((size_t)n * 4); memcpy(drv_res[i].data, v, (size_t)n * 4); drv_res[i].n = n; return; }
    if (drv_n >= DRV_MAX) return;
    snprintf(drv_res[drv_n].name, sizeof drv_res[drv_n].name, "%s", name);
    drv_res[drv_n].data = malloc((size_t)n * 4); memcpy(drv_res[drv_n].data, v, (size_t)n * 4); drv_res[drv_n].n = n; drv_n++;
}

/* capture_at < steps: step `capture_at` is issued between jit_begin_capture and jit_end_capture (the reference's own
 * capture / replay entry points, bound by the CUDA hub) and every step from there on is a jit_replay with that step's
 * batch and one-hot labels set as inputs: the live reference host (reducer, fuser, scheduler) records the step once and
 * is out of the loop afterwards. */
static int drv_lenet_impl(const char *dev, u32 B, u32 steps, f32 lr, const f32 *x, const u8 *labels, const f32 *params, u32 keep_grads, u32 capture_at);
int drv_lenet(const char *dev, u32 B, u32 steps, f32 lr, const f32 *x, const u8 *labels, const f32 *params, u32 keep_grads) {
    return drv_lenet_impl(dev, B, steps, lr, x, labels, params, keep_grads, 0xFFFFFFFFu);
}
int drv_lenet_captured(const char *dev, u32 B, u32 steps, f32 lr, const f32 *x, const u8 *labels, const f32 *params, u32 capture_at) {
    return drv_lenet_impl(dev, B, steps, lr, x, labels, params, 0, capture_at);
}

/* point the captured step's inputs at step s's data: the batch by its size, the one-hot label matrices by theirs */
static void lenet_set_inputs(u32 B, const f32 *xs, const f32 *oh) {
    for (u32 k = 0; k < jit_input_count(); k++) {
        const u64 nb = jit_input_bytes(k);
        if (nb == (u64)B * 784 * 4) jit_set_input(k, xs);
        else if (nb == (u64)B * 10 * 4) jit_set_input(k, oh);
        else { fprintf(stderr, "drv_lenet_captured: input %u of %llu bytes is neither the batch nor the labels\n", k, (unsigned long long)nb); exit(1); }
    }
}

static int drv_lenet_impl(const char *dev, u32 B, u32 steps, f32 lr, const f32 *x, const u8 *labels, const f32 *params, u32 keep_grads, u32 capture_at) {
    cpu_masked_leaf_workaround(dev);
    TinyHVM *ctx = thvm_init(dev);
    drv_ctx = ctx;
    if (drv_after_init) drv_after_init();
    lr = lr / (f32)drv_dp_world;                     /* gradients are summed over the ranks */
    const f32 *p = params;
#define PARAM(name, n, ...) (rec_note(name, 0), p += (n), thvm_tensor(ctx, p - (n), SHAPE(__VA_ARGS__)))
    Term W1 = PARAM("W1", 150, 6, 1, 5, 5),    b1 = PARAM("b1", 6, 6);
    Term W2 = PARAM("W2", 2400, 16, 6, 5, 5),  b2 = PARAM("b2", 16, 16);
    Term W3 = PARAM("W3", 48000, 400, 120),    b3 = PARAM("b3", 120, 120);
    Term W4 = PARAM("W4", 10080, 120, 84),     b4 = PARAM("b4", 84, 84);
    Term W5 = PARAM("W5", 840, 84, 10),        b5 = PARAM("b5", 10, 10);
    u32 keep_id = ctx->tensor_count;
    double t0 = now_s();
    f32 *oh_host = calloc((size_t)B * 10, 4);
    for (u32 s = 0; s < steps; s++) {
        const u8 *lab = labels + (size_t)s * B;
        if (s > capture_at) {                                                /* replay of the captured step on this step's data */
            char nm[32]; f32 lv = 0;
            memset(oh_host, 0, (size_t)B * 10 * 4);
            for (u32 i = 0; i < B; i++) oh_host[i * 10 + lab[i]] = 1.0f;
            lenet_set_inputs(B, x + (size_t)s * B * 784, oh_host);
            jit_replay();
            jit_result(0, &lv, 4);                                           /* waits for the step */
            snprintf(nm, sizeof nm, "loss%u", s); keep_host(nm, &lv, 1);
            continue;
        }
        if (s == capture_at) { jit_declare_input((u64)B * 784 * 4); jit_declare_input((u64)B * 10 * 4); jit_begin_capture(keep_id); }
        rec_mark("step_begin");
        rec_note("x", 0);
        Term tx = thvm_tensor(ctx, x + (size_t)s * B * 784, SHAPE(B, 1, 28, 28));
        /* forward */
        Term xp = pad_hw(ctx, tx, 2);                                        /* [B,1,32,32] */
        Term u1 = conv_fwd(ctx, xp, W1, b1);                                 /* [B,6,28,28] */
        Term a1 = realize(ctx, op1(ctx, UOP_RELU, u1));
        Term p1 = pool_fwd(ctx, a1);                                         /* raw [B,6,14,14,1,1] */
        Term u2 = conv_fwd(ctx, as4(ctx, p1, B, 6, 14, 14), W2, b2);         /* [B,16,10,10] */
        Term a2 = realize(ctx, op1(ctx, UOP_RELU, u2));
        Term p2 = pool_fwd(ctx, a2);                                         /* raw [B,16,5,5,1,1] */
        Term u3 = linear_fwd(ctx, as2(ctx, p2, B, 400), W3, b3, B, 120);
        Term a3 = realize(ctx, op1(ctx, UOP_RELU, u3));
        Term u4 = linear_fwd(ctx, a3, W4, b4, B, 84);
        Term a4 = realize(ctx, op1(ctx, UOP_RELU, u4));
        Term logits = linear_fwd(ctx, a4, W5, b5, B, 10);
        rec_note("onehot", 257);                                             /* the one-hot labels built inside the loss */
        Term loss = realize(ctx, cross_entropy_loss(ctx, logits, (u8 *)lab, B, 10));
        /* backward */
        Term dl = ce_backward(ctx, logits, lab, B, 10);
        Term dW5 = mm_raw(ctx, transpose2(ctx, a4), dl);
        Term db5 = realize(ctx, thvm_sum_axes(ctx, dl, (u32[]){0}, 1));
        Term da4 = mm_raw(ctx, dl, transpose2(ctx, W5));
        Term du4 = relu_bwd(ctx, as2(ctx, da4, B, 84), u4);
        Term dW4 = mm_raw(ctx, transpose2(ctx, a3), du4);
        Term db4 = realize(ctx, thvm_sum_axes(ctx, du4, (u32[]){0}, 1));
        Term da3 = mm_raw(ctx, du4, transpose2(ctx, W4));
        Term du3 = relu_bwd(ctx, as2(ctx, da3, B, 120), u3);
        Term dW3 = mm_raw(ctx, transpose2(ctx, as2(ctx, p2, B, 400)), du3);
        Term db3 = realize(ctx, thvm_sum_axes(ctx, du3, (u32[]){0}, 1));
        Term dp2 = mm_raw(ctx, du3, transpose2(ctx, W3));                    /* raw [B,1,400] */
        Term da2 = pool_bwd(ctx, a2, p2, dp2, B, 16, 5, 5);                  /* [B,16,10,10] */
        Term du2 = relu_bwd(ctx, as4(ctx, da2, B, 16, 10, 10), u2);
        Term dW2 = conv_wgrad(ctx, as4(ctx, p1, B, 6, 14, 14), du2, B, 6, 16, 10, 10, 5);
        Term db2 = realize(ctx, sum023(ctx, du2));
        Term dp1 = conv_dgrad(ctx, du2, W2, 6, 16, 5);                       /* raw [B,6,14,14] */
        Term da1 = pool_bwd(ctx, a1, p1, dp1, B, 6, 14, 14);                 /* [B,6,28,28] */
        Term du1 = relu_bwd(ctx, as4(ctx, da1, B, 6, 28, 28), u1);
        Term dW1 = conv_wgrad(ctx, xp, du1, B, 1, 6, 28, 28, 5);
        Term db1 = realize(ctx, sum023(ctx, du1));
        { Term gr[10] = {dW1, db1, dW2, db2, dW3, db3, dW4, db4, dW5, db5}; dp_sum_grads(ctx, gr, 10); }
        rec_mark("read:loss");
        keepf(ctx, "loss%u", s, loss);
        if (s == 0 && keep_grads) {
            keep(ctx, "logits", logits);
            keep(ctx, "dW1", dW1); keep(ctx, "db1", db1); keep(ctx, "dW2", dW2); keep(ctx, "db2", db2);
            keep(ctx, "dW3", dW3); keep(ctx, "db3", db3); keep(ctx, "dW4", dW4); keep(ctx, "db4", db4);
            keep(ctx, "dW5", dW5); keep(ctx, "db5", db5);
        }
        /* update */
        sgd(ctx, W1, as4(ctx, dW1, 6, 1, 5, 5), lr);   sgd(ctx, b1, as1(ctx, db1, 6), lr);
        sgd(ctx, W2, as4(ctx, dW2, 16, 6, 5, 5), lr);  sgd(ctx, b2, as1(ctx, db2, 16), lr);
        sgd(ctx, W3, as2(ctx, dW3, 400, 120), lr);     sgd(ctx, b3, as1(ctx, db3, 120), lr);
        sgd(ctx, W4, as2(ctx, dW4, 120, 84), lr);      sgd(ctx, b4, as1(ctx, db4, 84), lr);
        sgd(ctx, W5, as2(ctx, dW5, 84, 10), lr);       sgd(ctx, b5, as1(ctx, db5, 10), lr);
        rec_mark("read:b5");
        f32 *sync = thvm_to_host(ctx, b5); (void)sync;                       /* drain the device queue before the clock stops */
        rec_mark("step_end");
        if (s + 1 < steps || s == capture_at) { thvm_reset(ctx, keep_id); thvm_sched_reset_runtime(); }
        if (s == capture_at) {                                               /* nothing of the step has run yet: run it now */
            char nm[32]; f32 lv = 0;
            jit_end_capture();
            memset(oh_host, 0, (size_t)B * 10 * 4);
            for (u32 i = 0; i < B; i++) oh_host[i * 10 + lab[i]] = 1.0f;
            lenet_set_inputs(B, x + (size_t)s * B * 784, oh_host);
            jit_replay();
            jit_result(0, &lv, 4);
            snprintf(nm, sizeof nm, "loss%u", s); keep_host(nm, &lv, 1);
        }
    }
    free(oh_host);
    drv_secs = now_s() - t0;
    keep(ctx, "W1", W1); keep(ctx, "b1", b1); keep(ctx, "W2", W2); keep(ctx, "b2", b2); keep(ctx, "W3", W3);
    keep(ctx, "b3", b3); keep(ctx, "W4", W4); keep(ctx, "b4", b4); keep(ctx, "W5", W5); keep(ctx, "b5", b5);
    drv_ctx = NULL;
    thvm_free(ctx);
    return 0;
}

/* record `steps` LeNet training steps as a vtable trace (see ref_trace.c); dry = log only */
int drv_record_lenet(const char *path, u32 dry, u32 B, u32 steps, f32 lr, const f32 *x, const u8 *labels, const f32 *params) {
    if (rec_open(path)) return 1;
    drv_set_dp(1, rec_dp_hook, NULL);
    int rc = drv_lenet(dry ? "record-dry" : "record", B, steps, lr, x, labels, params, 0);
    drv_set_dp(1, NULL, NULL);
    rec_close();
    return rc;
}

/* ------------------------------------------------------------------ config 5: VGG-style CNN */
/* Three blocks of two [conv3x3 pad1 (no bias) + batchnorm(training) + relu] layers, a 2x2 max-pool after
 * each block, flatten, linear, softmax cross-entropy, SGD.  chan[0..6] = input channels and the six conv
 * widths (3,64,64,128,128,256,256 in the config); H = W = input size (64).  Batchnorm follows
 * src/nn/batchnorm.c:7-112 (biased variance, eps 1e-5), staged: every [1,C,1,1] statistic is realised and
 * x - mean is rebuilt per consumer; the running statistics, which the loss does not depend on, are not kept.
 * params (flat): per conv layer W[Co,Ci,3,3], gamma[Co], beta[Co]; then Wl[F,classes], bl[classes]. */
typedef struct { Term W, gamma, beta, xp, xhat, invstd, u, a; u32 Ci, Co, h; } VggLayer;

static Term bc4(TinyHVM *ctx, Term stat_raw, u32 B, u32 C, u32 h) {       /* [1,C,1,1] statistic broadcast to [B,C,h,h] */
    return thvm_expand(ctx, thvm_reshape(ctx, stat_raw, SHAPE(1, C, 1, 1)), SHAPE(B, C, h, h));
}

int drv_vgg(const char *dev, u32 B, u32 H, u32 classes, const u32 *chan, u32 steps, f32 lr, const f32 *x, const u8 *labels,
            const f32 *params, u32 keep_grads) {
    cpu_masked_leaf_workaround(dev);
    TinyHVM *ctx = thvm_init(dev);
    drv_ctx = ctx;
    if (drv_after_init) drv_after_init();
    lr = lr / (f32)drv_dp_world;
    VggLayer L[6];
    const f32 *p = params;
    char nm[32];
    for (u32 l = 0; l < 6; l++) {
        u32 Ci = chan[l], Co = chan[l + 1];
        L[l].Ci = Ci; L[l].Co = Co; L[l].h = H >> (l / 2);
        snprintf(nm, sizeof nm, "W%u", l); rec_note(nm, 0);     L[l].W = thvm_tensor(ctx, p, SHAPE(Co, Ci, 3, 3)); p += (size_t)Co * Ci * 9;
        snprintf(nm, sizeof nm, "gamma%u", l); rec_note(nm, 0); L[l].gamma = thvm_tensor(ctx, p, SHAPE(Co)); p += Co;
        snprintf(nm, sizeof nm, "beta%u", l); rec_note(nm, 0);  L[l].beta = thvm_tensor(ctx, p, SHAPE(Co)); p += Co;
    }
    const u32 hf = H >> 3, F = chan[6] * hf * hf;
    rec_note("Wl", 0); Term Wl = thvm_tensor(ctx, p, SHAPE(F, classes)); p += (size_t)F * classes;
    rec_note("bl", 0); Term bl = thvm_tensor(ctx, p, SHAPE(classes)); p += classes;
    u32 keep_id = ctx->tensor_count;
    double t0 = now_s();
    for (u32 s = 0; s < steps; s++) {
        rec_mark("step_begin");
        rec_note("x", 0);
        Term act = thvm_tensor(ctx, x + (size_t)s * B * chan[0] * H * H, SHAPE(B, chan[0], H, H));
        const u8 *lab = labels + (size_t)s * B;
        Term pooled[3];
        /* ---------------- forward ---------------- */
        for (u32 l = 0; l < 6; l++) {
            VggLayer *y = &L[l];
            const u32 h = y->h, Co = y->Co;
            const f32 inv = 1.0f / (f32)((u64)B * h * h);
            y->xp = pad_hw(ctx, as4(ctx, act, B, y->Ci, h, h), 1);
            Term z = conv_fwd(ctx, y->xp, y->W, term_era());                                             /* raw */
            Term mean = realize(ctx, op2(ctx, UOP_MUL, sum023(ctx, as4(ctx, z, B, Co, h, h)), scalar(ctx, inv)));
            Term d1 = op2(ctx, UOP_SUB, as4(ctx, z, B, Co, h, h), bc4(ctx, mean, B, Co, h));
            Term d2 = op2(ctx, UOP_SUB, as4(ctx, z, B, Co, h, h), bc4(ctx, mean, B, Co, h));
            Term var = realize(ctx, op2(ctx, UOP_MUL, sum023(ctx, op2(ctx, UOP_MUL, d1, d2)), scalar(ctx, inv)));
            y->invstd = realize(ctx, op2(ctx, UOP_DIV, scalar(ctx, 1.f), op1(ctx, UOP_SQRT, op2(ctx, UOP_ADD, var, scalar(ctx, 1e-5f)))));
            y->xhat = realize(ctx, op2(ctx, UOP_MUL, op2(ctx, UOP_SUB, as4(ctx, z, B, Co, h, h), bc4(ctx, mean, B, Co, h)), bc4(ctx, y->invstd, B, Co, h)));
            y->u = realize(ctx, op2(ctx, UOP_ADD, op2(ctx, UOP_MUL, y->xhat, bc4(ctx, y->gamma, B, Co, h)), bc4(ctx, y->beta, B, Co, h)));
            y->a = realize(ctx, op1(ctx, UOP_RELU, y->u));
            act = y->a;
            if (l & 1) { pooled[l / 2] = pool_fwd(ctx, y->a); act = pooled[l / 2]; }                     /* raw [B,Co,h/2,h/2,1,1] */
        }
        Term logits = linear_fwd(ctx, as2(ctx, act, B, F), Wl, bl, B, classes);
        rec_note("onehot", 257);
        Term loss = realize(ctx, cross_entropy_loss(ctx, logits, (u8 *)lab, B, classes));
        /* ---------------- backward ---------------- */
        Term dl = ce_backward(ctx, logits, lab, B, classes);
        Term dWl = mm_raw(ctx, transpose2(ctx, as2(ctx, act, B, F)), dl);
        Term dbl = realize(ctx, thvm_sum_axes(ctx, dl, (u32[]){0}, 1));
        Term g = mm_raw(ctx, dl, transpose2(ctx, Wl));                                                   /* raw [B,1,F]: grad of the last pool */
        Term dW[6], dgamma[6], dbeta[6];
        for (i32 l = 5; l >= 0; l--) {
            VggLayer *y = &L[l];
            const u32 h = y->h, Co = y->Co, Ci = y->Ci;
            const f32 N = (f32)((u64)B * h * h);
            if (l & 1) g = pool_bwd(ctx, y->a, pooled[l / 2], g, B, Co, h / 2, h / 2);                   /* -> [B,Co,h,h] */
            Term du = relu_bwd(ctx, as4(ctx, g, B, Co, h, h), y->u);
            dbeta[l] = realize(ctx, sum023(ctx, du));
            dgamma[l] = realize(ctx, sum023(ctx, op2(ctx, UOP_MUL, du, y->xhat)));
            Term scale = op2(ctx, UOP_MUL, op2(ctx, UOP_MUL, bc4(ctx, y->gamma, B, Co, h), bc4(ctx, y->invstd, B, Co, h)), scalar(ctx, 1.0f / N));
            Term inner = op2(ctx, UOP_SUB, op2(ctx, UOP_SUB, op2(ctx, UOP_MUL, du, scalar(ctx, N)), bc4(ctx, dbeta[l], B, Co, h)),
                             op2(ctx, UOP_MUL, y->xhat, bc4(ctx, dgamma[l], B, Co, h)));
            Term dz = realize(ctx, op2(ctx, UOP_MUL, scale, inner));
            dW[l] = conv_wgrad(ctx, y->xp, dz, B, Ci, Co, h, h, 3);
            if (l > 0) {
                Term dxp = conv_dgrad(ctx, dz, y->W, Ci, Co, 3);                                         /* raw [B,Ci,h+2,h+2] */
                u32 pairs[8] = {0, B, 0, Ci, 1, h + 1, 1, h + 1};
                g = realize(ctx, op2(ctx, UOP_ADD, thvm_shrink(ctx, as4(ctx, dxp, B, Ci, h + 2, h + 2), pairs, 4), scalar(ctx, 0.f)));
            }
        }
        { Term gr[20]; u32 n = 0; for (u32 l = 0; l < 6; l++) { gr[n++] = dW[l]; gr[n++] = dgamma[l]; gr[n++] = dbeta[l]; } gr[n++] = dWl; gr[n++] = dbl; dp_sum_grads(ctx, gr, n); }
        rec_mark("read:loss");
        keepf(ctx, "loss%u", s, loss);
        if (s == 0 && keep_grads) {
            keep(ctx, "logits", logits);
            for (u32 l = 0; l < 6; l++) {
                snprintf(nm, sizeof nm, "dW%u", l); keep(ctx, nm, dW[l]);
                snprintf(nm, sizeof nm, "dgamma%u", l); keep(ctx, nm, dgamma[l]);
                snprintf(nm, sizeof nm, "dbeta%u", l); keep(ctx, nm, dbeta[l]);
            }
            keep(ctx, "dWl", dWl); keep(ctx, "dbl", dbl);
        }
        /* ---------------- update ---------------- */
        for (u32 l = 0; l < 6; l++) {
            sgd(ctx, L[l].W, as4(ctx, dW[l], L[l].Co, L[l].Ci, 3, 3), lr);
            sgd(ctx, L[l].gamma, as1(ctx, dgamma[l], L[l].Co), lr);
            sgd(ctx, L[l].beta, as1(ctx, dbeta[l], L[l].Co), lr);
        }
        sgd(ctx, Wl, as2(ctx, dWl, F, classes), lr);
        sgd(ctx, bl, as1(ctx, dbl, classes), lr);
        rec_mark("read:bl");
        f32 *sync = thvm_to_host(ctx, bl); (void)sync;
        rec_mark("step_end");
        if (s + 1 < steps) { thvm_reset(ctx, keep_id); thvm_sched_reset_runtime(); }
    }
    drv_secs = now_s() - t0;
    for (u32 l = 0; l < 6; l++) {
        snprintf(nm, sizeof nm, "W%u", l); keep(ctx, nm, L[l].W);
        snprintf(nm, sizeof nm, "gamma%u", l); keep(ctx, nm, L[l].gamma);
        snprintf(nm, sizeof nm, "beta%u", l); keep(ctx, nm, L[l].beta);
    }
    keep(ctx, "Wl", Wl); keep(ctx, "bl", bl);
    drv_ctx = NULL;
    thvm_free(ctx);
    return 0;
}

int drv_record_vgg(const char *path, u32 dry, u32 B, u32 H, u32 classes, const u32 *chan, u32 steps, f32 lr, const f32 *x,
                   const u8 *labels, const f32 *params) {
    if (rec_open(path)) return 1;
    drv_set_dp(1, rec_dp_hook, NULL);
    int rc = drv_vgg(dry ? "record-dry" : "record", B, H, classes, chan, steps, lr, x, labels, params, 0);
    drv_set_dp(1, NULL, NULL);
    rec_close();
    return rc;
}
