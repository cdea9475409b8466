// fast.cu — the specialised bandwidth kernels and their selection.
//
// A dispatch (see plan.cu) qualifies when every leaf and the output are f32,
// every leaf is a single view without compound masks, and each leaf dim equals
// the iteration dim or is 1 (no modulo wrap).  Its iteration space is then
// collapsed (fast_desc.h) and one of three skeletons runs it:
//   k_ew         no reduce; each thread produces 4 consecutive outputs with
//                128-bit loads/stores where the leaf layout allows it;
//   k_red_inner  the innermost collapsed dim is reduced: 1, 32 or 256 threads
//                cooperate on one output (warp shuffles, then shared memory);
//                if there are too few outputs to fill 148 SMs the reduce range
//                is split across CTAs and a second pass adds the partials
//                (deterministic order, scratch from the library's pool);
//   k_red_outer  the innermost collapsed dim is kept: threads run along it
//                (coalesced) and walk the reduce range, same split scheme.
// The fused op list is either interpreted per vector of 4 elements, or — for
// the chains the training configs produce over and over (CHAINS below) —
// compiled in, selected by matching the dispatch's op list, which is the part
// of the reference's kernel-cache signature (src/tinyhvm.h:828-856) that does
// not depend on shapes.
//
// Accumulation order differs from the CPU backend's left-to-right loop
// (src/backend/cpu/dispatch.c:169-218): per-thread strided partial sums, then
// a tree.  Elementwise results are bit-identical.
#include <string.h>
#include "device_common.cuh"
#include "fast_desc.h"
#include "plans.h"
#include "state.h"

namespace thc {

// ------------------------------------------------------------------ static chains
struct ChainDef { int nl, no; unsigned char uop[8], a[8], b[8]; };
// unary ops carry b == a (the dispatcher canonicalises them the same way)
constexpr ChainDef CHAINS[] = {
    {0, 0, {}, {}, {}},                                                            // 0: interpreted
    {3, 3, {THC_MUL, THC_ADD, THC_RELU}, {0, 3, 4}, {1, 2, 4}},                    // 1: relu(a*b+c)
    {4, 4, {THC_MUL, THC_ADD, THC_CMP, THC_MUL}, {0, 4, 5, 1}, {1, 2, 3, 6}},      // 2: b*(a*b+c > z)
    {2, 2, {THC_ADD, THC_RELU}, {0, 2}, {1, 2}},                                   // 3: relu(y+bias)
    {2, 1, {THC_ADD}, {0}, {1}},                                                   // 4: a+b (pad / bias)
    {2, 1, {THC_MUL}, {0}, {1}},                                                   // 5: a*b
    {1, 0, {}, {}, {}},                                                            // 6: copy / plain reduce
    {2, 1, {THC_SUB}, {0}, {1}},                                                   // 7: a-b
    {2, 2, {THC_SUB, THC_EXP}, {0, 2}, {1, 2}},                                    // 8: exp(a-b)
    // the batch-norm / pooling / SGD chains of the CNN training steps
    {4, 3, {THC_SUB, THC_SUB, THC_MUL}, {0, 2, 4}, {1, 3, 5}},                     // 9: (a-b)*(c-d)      variance terms
    {3, 2, {THC_SUB, THC_MUL}, {0, 3}, {1, 2}},                                    // 10: (a-b)*c         normalise
    {3, 2, {THC_MUL, THC_ADD}, {0, 3}, {1, 2}},                                    // 11: a*b+c           scale and shift
    {1, 1, {THC_RELU}, {0}, {0}},                                                  // 12: relu(a)
    {3, 2, {THC_CMP, THC_MUL}, {1, 0}, {2, 3}},                                    // 13: a*(b>c)         relu backward
    {8, 7, {THC_MUL, THC_MUL, THC_MUL, THC_SUB, THC_MUL, THC_SUB, THC_MUL}, {0, 8, 3, 10, 6, 11, 9}, {1, 2, 4, 5, 7, 12, 13}},
                                                                                   // 14: a*b*c * ((d*e - f) - g*h)   batch-norm backward
    {4, 3, {THC_CMP, THC_SUB, THC_MUL}, {2, 1, 0}, {3, 4, 5}},                     // 15: a*(b-(c>d))     max-pool backward (ties all pass)
    {3, 2, {THC_MUL, THC_SUB}, {1, 0}, {2, 3}},                                    // 16: a-b*c           SGD update
};
constexpr int N_CHAINS = sizeof(CHAINS) / sizeof(CHAINS[0]);

struct InterpEval {
    static constexpr int MAXL = FL, NV = FL + FO;
    __device__ static __forceinline__ int nleaves(const FProg &P) { return (int)P.n_leaves; }
    __device__ static __forceinline__ int result(const FProg &P) { return P.n_ops ? (int)(P.n_leaves + P.n_ops - 1) : 0; }
    template <int V>
    __device__ static __forceinline__ void run(const FProg &P, float (&v)[NV][V]) {
        const int nl = (int)P.n_leaves;
        for (int i = 0; i < (int)P.n_ops; i++) {
            const unsigned u = P.uop[i], x = P.aux[i];
            const int a = P.a[i], b = P.b[i];
#pragma unroll
            for (int k = 0; k < V; k++) v[nl + i][k] = alu(u, x, v[a][k], v[b][k]);
        }
    }
};

template <int CI, int I, int V, int NV>
struct ChainStep {
    __device__ static __forceinline__ void run(float (&v)[NV][V]) {
        constexpr ChainDef C = CHAINS[CI];
        if constexpr (I < C.no) {
            constexpr unsigned u = C.uop[I];
            constexpr int a = C.a[I], b = C.b[I];
#pragma unroll
            for (int k = 0; k < V; k++) v[C.nl + I][k] = alu(u, 0u, v[a][k], v[b][k]);
            ChainStep<CI, I + 1, V, NV>::run(v);
        }
    }
};
template <int CI>
struct StaticEval {
    static constexpr int MAXL = CHAINS[CI].nl, NV = CHAINS[CI].nl + CHAINS[CI].no;
    __device__ static __forceinline__ int nleaves(const FProg &) { return CHAINS[CI].nl; }
    __device__ static __forceinline__ int result(const FProg &) { return CHAINS[CI].no ? NV - 1 : 0; }
    template <int V>
    __device__ static __forceinline__ void run(const FProg &, float (&v)[NV][V]) { ChainStep<CI, 0, V, NV>::run(v); }
};

// ------------------------------------------------------------------ leaf access
// V consecutive elements along the innermost collapsed dim, starting at coords c.
template <int V>
__device__ __forceinline__ void load_leaf(const FLeaf &L, const unsigned *c, int rank, unsigned long long flat, float (&dst)[V]) {
    if (L.mode == 2) {                       // a single element, broadcast
        const float s = L.ptr[L.off];
#pragma unroll
        for (int k = 0; k < V; k++) dst[k] = s;
        return;
    }
    if (L.mode == 1) {                       // laid out exactly like the iteration space
        const float *p = L.ptr + (L.off + (long long)flat);
        if (V == 4 && L.vec) {
            const float4 q = *reinterpret_cast<const float4 *>(p);
            dst[0] = q.x; dst[1] = q.y; dst[2] = q.z; dst[3] = q.w;
        } else {
#pragma unroll
            for (int k = 0; k < V; k++) dst[k] = p[k];
        }
        return;
    }
    long long off = L.off;
    bool dead = false;
#pragma unroll
    for (int d = 0; d < FR; d++)
        if (d < rank) {
            off += (long long)c[d] * L.stride[d];
            if (d < rank - 1 && ((L.masked >> d) & 1u) && (c[d] < L.mlo[d] || c[d] >= L.mhi[d])) dead = true;
        }
    if (dead) {
#pragma unroll
        for (int k = 0; k < V; k++) dst[k] = 0.0f;
        return;
    }
    const int in = rank - 1;
    const bool inner_masked = (L.masked >> in) & 1u;
    if (V == 4 && L.vec && !inner_masked) {
        if (L.stride[in] == 1) {
            const float4 q = *reinterpret_cast<const float4 *>(L.ptr + off);
            dst[0] = q.x; dst[1] = q.y; dst[2] = q.z; dst[3] = q.w;
        } else {
            const float s = L.ptr[off];
#pragma unroll
            for (int k = 0; k < V; k++) dst[k] = s;
        }
        return;
    }
    const int si = L.stride[in];
#pragma unroll
    for (int k = 0; k < V; k++) {
        const unsigned ci = c[in] + k;
        dst[k] = (inner_masked && (ci < L.mlo[in] || ci >= L.mhi[in])) ? 0.0f : L.ptr[off + (long long)k * si];
    }
}

template <class EV, int V>
__device__ __forceinline__ void eval_at(const FDesc &D, const unsigned *c, unsigned long long flat, float (&res)[V]) {
    float v[EV::NV][V];
    const int nl = EV::nleaves(D.prog);
#pragma unroll
    for (int i = 0; i < EV::MAXL; i++)
        if (i < nl) load_leaf<V>(D.leaf[i], c, (int)D.rank, flat, v[i]);
    EV::template run<V>(D.prog, v);
    const int r = EV::result(D.prog);
#pragma unroll
    for (int k = 0; k < V; k++) res[k] = v[r][k];
}

// ------------------------------------------------------------------ index decode
// idx -> coordinates of the listed collapsed dims (outermost first).  The
// outermost dim needs no division, and indices below 2^32 use 32-bit division.
__device__ __forceinline__ void decode_dims(unsigned long long idx, const unsigned *list, int n,
                                            const unsigned *dims, unsigned *c) {
    if (n <= 0) return;
    if (idx <= 0xFFFFFFFFull) {
        unsigned rem = (unsigned)idx;
        for (int k = n - 1; k > 0; k--) { const unsigned d = list[k]; const unsigned q = rem / dims[d]; c[d] = rem - q * dims[d]; rem = q; }
        c[list[0]] = rem;
    } else {
        unsigned long long rem = idx;
        for (int k = n - 1; k > 0; k--) { const unsigned d = list[k]; const unsigned long long q = rem / dims[d]; c[d] = (unsigned)(rem - q * dims[d]); rem = q; }
        c[list[0]] = (unsigned)rem;
    }
}

// ------------------------------------------------------------------ elementwise
template <class EV, int V>
__global__ void __launch_bounds__(256) k_ew(const __grid_constant__ FDesc D, float *__restrict__ out) {
    const unsigned long long items = D.numel / V;
    const int rank = (int)D.rank;
    for (unsigned long long it = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; it < items;
         it += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned long long flat = it * V;
        unsigned c[FR];
        if (flat <= 0xFFFFFFFFull) {
            unsigned rem = (unsigned)flat;
            for (int d = rank - 1; d > 0; d--) { const unsigned q = rem / D.dims[d]; c[d] = rem - q * D.dims[d]; rem = q; }
            c[0] = rem;
        } else {
            unsigned long long rem = flat;
            for (int d = rank - 1; d > 0; d--) { c[d] = (unsigned)(rem % D.dims[d]); rem /= D.dims[d]; }
            c[0] = (unsigned)rem;
        }
        float res[V];
        eval_at<EV, V>(D, c, flat, res);
        if (V == 4) *reinterpret_cast<float4 *>(out + flat) = make_float4(res[0], res[1], res[2], res[3]);
        else if (V == 2) *reinterpret_cast<float2 *>(out + flat) = make_float2(res[0], res[1]);
        else out[flat] = res[0];
    }
}

// coordinates (into c) and flat position of reduce index r for an output whose
// kept coordinates are already in c and whose kept flat position is kflat
__device__ __forceinline__ unsigned long long red_position(const FDesc &D, unsigned long long r, bool one_r,
                                                           unsigned long long kflat, unsigned *c) {
    if (one_r) { c[D.rd[0]] = (unsigned)r; return kflat + r * D.fstride[D.rd[0]]; }
    decode_dims(r, D.rd, (int)D.n_r, D.dims, c);
    unsigned long long f = kflat;
    for (int k = 0; k < (int)D.n_r; k++) f += (unsigned long long)c[D.rd[k]] * D.fstride[D.rd[k]];
    return f;
}

// ------------------------------------------------------------------ reduce, innermost dim reduced
template <class EV, int G, int V>
__global__ void __launch_bounds__(256) k_red_inner(const __grid_constant__ FDesc D, float *__restrict__ out) {
    __shared__ float part[8];
    const int rank = (int)D.rank;
    const unsigned rtype = D.rtype;
    const unsigned long long items = D.n_red / V;
    const unsigned long long chunk = (items + D.split - 1) / D.split;
    const unsigned long long n_groups = D.n_out * D.split;
    const unsigned lane = G == 1 ? 0u : threadIdx.x % G;
    const unsigned long long stride_groups = ((unsigned long long)gridDim.x * blockDim.x) / G;
    for (unsigned long long gi = ((unsigned long long)blockIdx.x * blockDim.x + threadIdx.x) / G; gi < n_groups;
         gi += stride_groups) {
        const unsigned long long o = gi / D.split;
        const unsigned s = (unsigned)(gi % D.split);
        unsigned c[FR];
        decode_dims(o, D.kd, (int)D.n_k, D.dims, c);
        unsigned long long kflat = 0;           // flat position of the kept coordinates
        for (int k = 0; k < (int)D.n_k; k++) kflat += (unsigned long long)c[D.kd[k]] * D.fstride[D.kd[k]];
        const bool one_r = D.n_r == 1;          // a single reduced dim: the innermost one, stride 1 in flat space
        const unsigned long long lo = (unsigned long long)s * chunk;
        const unsigned long long hi = lo + chunk < items ? lo + chunk : items;
        float acc = red_init(rtype);
        unsigned long long it = lo + lane;
        if (G > 1) {
            // two vectors per trip: twice the loads in flight per thread, two
            // independent accumulation chains
            float acc2 = red_init(rtype);
            unsigned c2[FR];
#pragma unroll
            for (int d = 0; d < FR; d++) c2[d] = c[d];
            for (; it + G < hi; it += 2 * G) {
                const unsigned long long f1 = red_position(D, it * V, one_r, kflat, c);
                const unsigned long long f2 = red_position(D, (it + G) * V, one_r, kflat, c2);
                float r1[V], r2[V];
                eval_at<EV, V>(D, c, f1, r1);
                eval_at<EV, V>(D, c2, f2, r2);
#pragma unroll
                for (int k = 0; k < V; k++) { acc = red_combine(rtype, acc, r1[k]); acc2 = red_combine(rtype, acc2, r2[k]); }
            }
            acc = red_combine(rtype, acc, acc2);
        }
        for (; it < hi; it += G) {
            const unsigned long long f1 = red_position(D, it * V, one_r, kflat, c);
            float res[V];
            eval_at<EV, V>(D, c, f1, res);
#pragma unroll
            for (int k = 0; k < V; k++) acc = red_combine(rtype, acc, res[k]);
        }
        if (G > 1) {
#pragma unroll
            for (int w = 16; w > 0; w >>= 1) acc = red_combine(rtype, acc, __shfl_down_sync(0xffffffffu, acc, w));
        }
        if (G == 256) {
            __syncthreads();
            if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
            __syncthreads();
            if (threadIdx.x == 0) { acc = part[0]; for (int w = 1; w < 8; w++) acc = red_combine(rtype, acc, part[w]); }
        }
        if (lane == 0) out[gi] = acc;       // gi == o when split == 1
    }
}

// ------------------------------------------------------------------ streamlined forms: every leaf flat or a single element
// When every leaf is laid out exactly like the iteration space (or is one broadcast
// element) no coordinates are needed at all: the loads of a trip are issued back to
// back, branch-free, from per-leaf base pointers.  These forms carry the big
// contiguous chains (y = sum_last(relu(a*b+c)) and its VJP) at the HBM rate.
template <class EV>
struct FlatLeaves {
    static constexpr int NL = EV::MAXL;
    const float4 *p[NL];
    float sc[NL];
    bool fl[NL];
    __device__ __forceinline__ void init(const FDesc &D) {
        const int nl = EV::nleaves(D.prog);
#pragma unroll
        for (int i = 0; i < NL; i++) {
            fl[i] = false; sc[i] = 0.0f; p[i] = nullptr;
            if (i < nl) {
                const FLeaf &L = D.leaf[i];
                fl[i] = L.mode == 1;
                if (fl[i]) p[i] = reinterpret_cast<const float4 *>(L.ptr + L.off);
                else sc[i] = L.ptr[L.off];
            }
        }
    }
    // the chain's result for the 4 elements of vector `idx`
    __device__ __forceinline__ float4 eval(const FDesc &D, unsigned long long idx) const {
        float v[EV::NV][4];
#pragma unroll
        for (int i = 0; i < NL; i++) {
            float4 q = make_float4(sc[i], sc[i], sc[i], sc[i]);
            if (fl[i]) q = __ldg(p[i] + idx);
            v[i][0] = q.x; v[i][1] = q.y; v[i][2] = q.z; v[i][3] = q.w;
        }
        EV::template run<4>(D.prog, v);
        const int r = EV::result(D.prog);
        return make_float4(v[r][0], v[r][1], v[r][2], v[r][3]);
    }
};
template <class EV> constexpr int flat_unroll() { return EV::MAXL <= 4 ? 2 : 1; }

// out[o] = reduce over one contiguous row of n_red elements; G = 256: one CTA per row, G = 32: one warp per row
template <class EV, int G>
__global__ void __launch_bounds__(256) k_rows(const __grid_constant__ FDesc D, float *__restrict__ out) {
    constexpr int U = flat_unroll<EV>();
    __shared__ float part[8];
    FlatLeaves<EV> LV;
    LV.init(D);
    const unsigned rtype = D.rtype;
    const unsigned cols4 = (unsigned)(D.n_red / 4);
    const unsigned lane = threadIdx.x % G;
    const unsigned long long per_cta = 256 / G;
    for (unsigned long long row = (unsigned long long)blockIdx.x * per_cta + threadIdx.x / G; row < D.n_out;
         row += (unsigned long long)gridDim.x * per_cta) {
        const unsigned long long base = row * cols4;
        float acc[U];
#pragma unroll
        for (int u = 0; u < U; u++) acc[u] = red_init(rtype);
        unsigned i = lane;
        for (; i + (U - 1) * G < cols4; i += U * G) {
            float4 r[U];
#pragma unroll
            for (int u = 0; u < U; u++) r[u] = LV.eval(D, base + i + u * G);
#pragma unroll
            for (int u = 0; u < U; u++)
                acc[u] = red_combine(rtype, acc[u], red_combine(rtype, red_combine(rtype, r[u].x, r[u].y), red_combine(rtype, r[u].z, r[u].w)));
        }
        for (; i < cols4; i += G) {
            const float4 r = LV.eval(D, base + i);
            acc[0] = red_combine(rtype, acc[0], red_combine(rtype, red_combine(rtype, r.x, r.y), red_combine(rtype, r.z, r.w)));
        }
        float a = acc[0];
#pragma unroll
        for (int u = 1; u < U; u++) a = red_combine(rtype, a, acc[u]);
#pragma unroll
        for (int w = 16; w > 0; w >>= 1) a = red_combine(rtype, a, __shfl_down_sync(0xffffffffu, a, w));
        if (G == 256) {                       // rows are uniform per CTA here, so the barriers are too
            __syncthreads();
            if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = a;
            __syncthreads();
            if (threadIdx.x == 0) {
                a = part[0];
                for (int w = 1; w < 8; w++) a = red_combine(rtype, a, part[w]);
                out[row] = a;
            }
        } else if (lane == 0) {
            out[row] = a;
        }
    }
}

// out = chain(leaves) over one flat run of numel elements; each CTA takes a contiguous slab
template <class EV>
__global__ void __launch_bounds__(256) k_ew_flat(const __grid_constant__ FDesc D, float *__restrict__ out) {
    constexpr int U = flat_unroll<EV>();
    FlatLeaves<EV> LV;
    LV.init(D);
    const unsigned long long n4 = D.numel / 4;
    float4 *o4 = reinterpret_cast<float4 *>(out);
    for (unsigned long long i = (unsigned long long)blockIdx.x * (256 * U) + threadIdx.x; i < n4; i += (unsigned long long)gridDim.x * (256 * U)) {
        float4 r[U];
#pragma unroll
        for (int u = 0; u < U; u++)
            if (i + u * 256 < n4) r[u] = LV.eval(D, i + u * 256);
#pragma unroll
        for (int u = 0; u < U; u++)
            if (i + u * 256 < n4) o4[i + u * 256] = r[u];
    }
}

// ------------------------------------------------------------------ row kernels: contiguous rows with per-row constants
// The iteration space seen as R rows of dims[in] elements, every leaf either walking the row with stride 1
// (16-byte loads) or constant along it (a per-channel statistic, a scalar): coordinates are decoded once per
// row, not per vector, and a row's loads are issued back to back.  Elementwise: the output row is contiguous.
// Reduce (the innermost dim and any outer dims reduced): each row yields one partial sum, written to slot
// o * row_split + s (o = index over the kept outer dims, s = index over the reduced outer dims); k_red_final
// adds the row_split partials of an output in fixed order.  This is the shape of every batch-norm kernel:
// [B, C, H*W] with [1, C, 1] statistics.
template <class EV, int G, bool RED>
__global__ void __launch_bounds__(256) k_rowsx(const __grid_constant__ FDesc D, float *__restrict__ out) {
    constexpr int U = flat_unroll<EV>();
    constexpr int NL = EV::MAXL;
    __shared__ float part[8];
    const int nl = EV::nleaves(D.prog);
    const int in = (int)D.rank - 1;
    const unsigned rtype = D.rtype;
    const unsigned cols4 = D.dims[in] / 4;
    const unsigned lane = threadIdx.x % G;
    const unsigned long long R = D.numel / D.dims[in];
    const unsigned long long per_cta = 256 / G;
    float4 *o4 = reinterpret_cast<float4 *>(out);
    for (unsigned long long row = (unsigned long long)blockIdx.x * per_cta + threadIdx.x / G; row < R;
         row += (unsigned long long)gridDim.x * per_cta) {
        unsigned c[FR];
        {
            unsigned long long rem = row;
            for (int d = in - 1; d > 0; d--) { const unsigned long long q = rem / D.dims[d]; c[d] = (unsigned)(rem - q * D.dims[d]); rem = q; }
            c[0] = (unsigned)rem;
        }
        FlatLeaves<EV> LV;
#pragma unroll
        for (int i = 0; i < NL; i++) {
            LV.fl[i] = false; LV.sc[i] = 0.0f; LV.p[i] = nullptr;
            if (i < nl) {
                const FLeaf &L = D.leaf[i];
                long long off = L.off;
                for (int d = 0; d < in; d++) off += (long long)c[d] * L.stride[d];
                LV.fl[i] = L.stride[in] == 1;
                if (LV.fl[i]) LV.p[i] = reinterpret_cast<const float4 *>(L.ptr + off);
                else LV.sc[i] = L.ptr[off];
            }
        }
        float acc[U];
#pragma unroll
        for (int u = 0; u < U; u++) acc[u] = red_init(rtype);
        unsigned i = lane;
        for (; i + (U - 1) * G < cols4; i += U * G) {
            float4 r[U];
#pragma unroll
            for (int u = 0; u < U; u++) r[u] = LV.eval(D, i + u * G);
#pragma unroll
            for (int u = 0; u < U; u++) {
                if (RED) acc[u] = red_combine(rtype, acc[u], red_combine(rtype, red_combine(rtype, r[u].x, r[u].y), red_combine(rtype, r[u].z, r[u].w)));
                else o4[row * cols4 + i + u * G] = r[u];
            }
        }
        for (; i < cols4; i += G) {
            const float4 r = LV.eval(D, i);
            if (RED) acc[0] = red_combine(rtype, acc[0], red_combine(rtype, red_combine(rtype, r.x, r.y), red_combine(rtype, r.z, r.w)));
            else o4[row * cols4 + i] = r;
        }
        if (RED) {
            float a = acc[0];
#pragma unroll
            for (int u = 1; u < U; u++) a = red_combine(rtype, a, acc[u]);
#pragma unroll
            for (int w = 16; w > 0; w >>= 1) a = red_combine(rtype, a, __shfl_down_sync(0xffffffffu, a, w));
            unsigned long long slot = 0;
            for (int d = 0; d < in; d++) slot += (unsigned long long)c[d] * (D.omul[d] * D.row_split + D.smul[d]);
            if (G == 256) {                   // one row per CTA: the barriers are uniform
                __syncthreads();
                if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = a;
                __syncthreads();
                if (threadIdx.x == 0) {
                    a = part[0];
                    for (int w = 1; w < 8; w++) a = red_combine(rtype, a, part[w]);
                    out[slot] = a;
                }
            } else if (lane == 0) {
                out[slot] = a;
            }
        }
    }
}

// ------------------------------------------------------------------ reduce, innermost dim kept
template <class EV>
__global__ void __launch_bounds__(256) k_red_outer(const __grid_constant__ FDesc D, float *__restrict__ out) {
    __shared__ float part[8][33];
    const int rank = (int)D.rank;
    (void)rank;
    const unsigned rtype = D.rtype;
    const unsigned tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const unsigned long long o = (unsigned long long)blockIdx.x * 32 + tx;
    const bool live = o < D.n_out;
    unsigned c[FR];
#pragma unroll
    for (int d = 0; d < FR; d++) c[d] = 0;
    if (live) {
        decode_dims(o, D.kd, (int)D.n_k, D.dims, c);
    }
    unsigned long long kflat = 0;
    for (int k = 0; k < (int)D.n_k; k++) kflat += (unsigned long long)c[D.kd[k]] * D.fstride[D.kd[k]];
    float acc = red_init(rtype);
    if (live)
        for (unsigned long long r = (unsigned long long)blockIdx.y * 8 + ty; r < D.n_red; r += 8ull * gridDim.y) {
            const unsigned long long f1 = red_position(D, r, D.n_r == 1, kflat, c);
            float res[1];
            eval_at<EV, 1>(D, c, f1, res);
            acc = red_combine(rtype, acc, res[0]);
        }
    part[ty][tx] = acc;
    __syncthreads();
    if (ty == 0 && live) {
        for (int w = 1; w < 8; w++) acc = red_combine(rtype, acc, part[w][tx]);
        out[o * gridDim.y + blockIdx.y] = acc;
    }
}

// second pass with many partials per output: one warp per output, lanes stride over the partials, fixed tree
__global__ void __launch_bounds__(256) k_red_final_warp(const float *__restrict__ partial, float *__restrict__ out,
                                                        unsigned long long n_out, unsigned split, unsigned rtype) {
    const unsigned lane = threadIdx.x & 31;
    for (unsigned long long o = ((unsigned long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; o < n_out;
         o += ((unsigned long long)gridDim.x * blockDim.x) >> 5) {
        float acc = red_init(rtype);
        for (unsigned s = lane; s < split; s += 32) acc = red_combine(rtype, acc, partial[o * split + s]);
#pragma unroll
        for (int w = 16; w > 0; w >>= 1) acc = red_combine(rtype, acc, __shfl_down_sync(0xffffffffu, acc, w));
        if (lane == 0) out[o] = acc;
    }
}

// second pass: out[o] = fold of partial[o*split .. o*split+split)
__global__ void __launch_bounds__(256) k_red_final(const float *__restrict__ partial, float *__restrict__ out,
                                                   unsigned long long n_out, unsigned split, unsigned rtype) {
    for (unsigned long long o = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; o < n_out;
         o += (unsigned long long)gridDim.x * blockDim.x) {
        float acc = partial[o * split];
        for (unsigned s = 1; s < split; s++) acc = red_combine(rtype, acc, partial[o * split + s]);
        out[o] = acc;
    }
}

// ------------------------------------------------------------------ host: classify
struct FastDesc {
    FDesc d;
    int   strategy;                 // 0 ew, 1 reduce-inner, 2 reduce-outer
    int   group;                    // threads per output for reduce-inner
    long long min_off[FL], max_off[FL];
    const char *name, *flat_name;   // kernel family for the launch statistics: general form, streamlined form
    bool  flat_shape;               // every leaf flat or one element, shape fit for the streamlined kernels
    bool  flat;                     // decided per launch: flat_shape and all pointers 16-byte aligned
    bool  rows_shape, rows;         // same for the row kernels (contiguous rows, per-row constants)
    const char *rows_name;
};

static bool build_fast(const GenDesc &H, FastDesc &F) {
    if (H.post_start || H.n_leaves > FL || H.n_ops > FO || H.out_dtype != THC_F32 || H.full_numel == 0) return false;
    const int rank = (int)H.rank;
    long long st[FL][THC_MAX_DIM];
    unsigned lo[FL][THC_MAX_DIM], hi[FL][THC_MAX_DIM];
    bool part[FL][THC_MAX_DIM];
    for (unsigned i = 0; i < H.n_leaves; i++) {
        const DLeaf &L = H.leaves[i];
        if (L.tracker >= 0 || L.dtype != THC_F32) return false;
        if (L.v.has_mask && L.v.n_cm) return false;
        const int n = (int)L.v.rank < rank ? (int)L.v.rank : rank;
        for (int d = 0; d < rank; d++) {
            st[i][d] = 0; lo[i][d] = 0; hi[i][d] = H.full_dims[d]; part[i][d] = false;
            if (d >= n) continue;
            const unsigned ld = L.v.dims[d];
            if (ld == 0 || (ld != H.full_dims[d] && ld != 1)) return false;
            st[i][d] = ld > 1 ? L.v.strides[d] : 0;
            if (L.v.has_mask) {
                lo[i][d] = L.v.mb[d];
                hi[i][d] = L.v.me[d] < H.full_dims[d] ? L.v.me[d] : H.full_dims[d];
                part[i][d] = lo[i][d] > 0 || hi[i][d] < H.full_dims[d];
                if (hi[i][d] <= lo[i][d]) return false;            // leaf is zero everywhere: leave to the generic kernel
            }
        }
    }
    // collapse
    struct Dim { unsigned long long n; bool red; int src; };
    Dim dims[THC_MAX_DIM]; int nd = 0;
    long long cst[FL][THC_MAX_DIM]; unsigned clo[FL][THC_MAX_DIM], chi[FL][THC_MAX_DIM]; bool cpart[FL][THC_MAX_DIM];
    for (int d = 0; d < rank; d++) {
        if (H.full_dims[d] == 1) {
            for (unsigned i = 0; i < H.n_leaves; i++) if (part[i][d]) return false;
            continue;
        }
        const bool red = H.has_reduce && [&] { for (unsigned k = 0; k < H.n_rdims; k++) if ((int)H.rdim[k] == d) return true; return false; }();
        bool merge = nd > 0 && dims[nd - 1].red == red;
        if (merge)
            for (unsigned i = 0; i < H.n_leaves && merge; i++)
                if (cpart[i][nd - 1] || part[i][d] || cst[i][nd - 1] != st[i][d] * (long long)H.full_dims[d]) merge = false;
        if (merge && dims[nd - 1].n * H.full_dims[d] > 0xFFFFFFFFull) merge = false;
        if (merge) {
            dims[nd - 1].n *= H.full_dims[d];
            for (unsigned i = 0; i < H.n_leaves; i++) { cst[i][nd - 1] = st[i][d]; clo[i][nd - 1] = 0; chi[i][nd - 1] = (unsigned)dims[nd - 1].n; }
        } else {
            dims[nd] = {H.full_dims[d], red, d};
            for (unsigned i = 0; i < H.n_leaves; i++) { cst[i][nd] = st[i][d]; clo[i][nd] = lo[i][d]; chi[i][nd] = hi[i][d]; cpart[i][nd] = part[i][d]; }
            nd++;
        }
    }
    if (nd == 0) {                                                // every dim is 1
        dims[0] = {1, false, 0}; nd = 1;
        for (unsigned i = 0; i < H.n_leaves; i++) { cst[i][0] = 0; clo[i][0] = 0; chi[i][0] = 1; cpart[i][0] = false; }
    }
    if (nd > FR) return false;

    FDesc &D = F.d;
    memset(&D, 0, sizeof D);
    D.rank = nd; D.numel = 1; D.n_out = 1; D.n_red = 1;
    D.rtype = H.has_reduce ? H.reduce_type : 0;
    for (int d = 0; d < nd; d++) {
        D.dims[d] = (unsigned)dims[d].n; D.is_red[d] = dims[d].red;
        D.numel *= dims[d].n;
        if (dims[d].red) { D.rd[D.n_r++] = d; D.n_red *= dims[d].n; } else { D.kd[D.n_k++] = d; D.n_out *= dims[d].n; }
    }
    const int in = nd - 1;
    {
        unsigned long long w = 1;
        for (int d = nd - 1; d >= 0; d--) { D.fstride[d] = w; w *= D.dims[d]; }
    }
    bool vec_ok = D.dims[in] % 4 == 0;
    for (unsigned i = 0; i < H.n_leaves; i++) {
        FLeaf &L = D.leaf[i];
        L.off = H.leaves[i].v.offset;
        F.min_off[i] = F.max_off[i] = L.off;
        bool lv = true;
        for (int d = 0; d < nd; d++) {
            if (cst[i][d] > 0x7FFFFFFFll || cst[i][d] < -0x7FFFFFFFll) return false;
            L.stride[d] = (int)cst[i][d]; L.mlo[d] = clo[i][d]; L.mhi[d] = chi[i][d];
            if (cpart[i][d]) L.masked |= 1u << d;
            const long long a = cst[i][d] * (long long)(cpart[i][d] ? clo[i][d] : 0);
            const long long b = cst[i][d] * (long long)((cpart[i][d] ? chi[i][d] : D.dims[d]) - 1);
            F.min_off[i] += a < b ? a : b;
            F.max_off[i] += a < b ? b : a;
            if (d != in && (cst[i][d] % 4) != 0) lv = false;
        }
        if (!(cst[i][in] == 1 || cst[i][in] == 0)) lv = false;
        if (cst[i][in] == 1 && (L.off % 4) != 0) lv = false;
        L.vec = lv ? 1u : 0u;
        bool flat = L.masked == 0, single = L.masked == 0;
        for (int d = 0; d < nd; d++) {
            if ((unsigned long long)cst[i][d] != D.fstride[d] || cst[i][d] < 0) flat = false;
            if (cst[i][d] != 0) single = false;
        }
        L.mode = single ? 2u : (flat ? 1u : 0u);
    }
    // elementwise dispatches whose innermost dim is even but not a multiple of 4 (2x2 pooling windows, rows padded
    // to 66) still decode one coordinate set per pair of outputs
    D.vec = vec_ok ? 4u : ((!H.has_reduce && D.dims[in] % 2 == 0) ? 2u : 1u);
    D.split = 1;

    // program; unary ops get b = a so they match the static chain table
    D.prog.n_leaves = H.n_leaves; D.prog.n_ops = H.n_ops;
    for (unsigned i = 0; i < H.n_ops; i++) {
        const unsigned u = H.ops[i].uop;
        const bool unary = u == THC_NEG || u == THC_EXP || u == THC_LOG || u == THC_RELU || u == THC_CAST || u == THC_SQRT;
        D.prog.uop[i] = (unsigned char)u; D.prog.a[i] = (unsigned char)H.ops[i].arg_a;
        D.prog.b[i] = (unsigned char)(unary ? H.ops[i].arg_a : H.ops[i].arg_b);
        D.prog.aux[i] = (unsigned char)H.ops[i].aux;
        if (u > 255 || H.ops[i].aux > 255) return false;
    }
    D.chain = 0;
    for (int ci = 1; ci < N_CHAINS; ci++) {
        const ChainDef &C = CHAINS[ci];
        if (C.nl != (int)H.n_leaves || C.no != (int)H.n_ops) continue;
        bool eq = true;
        for (int k = 0; k < C.no && eq; k++)
            eq = C.uop[k] == D.prog.uop[k] && C.a[k] == D.prog.a[k] && C.b[k] == D.prog.b[k] && D.prog.uop[k] != THC_CAST;
        if (eq) { D.chain = ci; break; }
    }

    // strategy
    const unsigned sms = (unsigned)g.sm_count;
    bool all_flat = D.vec == 4;                    // every leaf flat (and 16-byte loadable) or one element
    for (unsigned i = 0; i < H.n_leaves; i++)
        if (!(D.leaf[i].mode == 2 || (D.leaf[i].mode == 1 && D.leaf[i].vec))) all_flat = false;
    F.flat_shape = false; F.flat = false;
    F.flat_name = ""; F.rows_name = ""; F.rows_shape = false; F.rows = false;
    D.row_split = 1;
    {   // row kernels: every leaf unmasked and either stride 1 (16-byte loadable) or stride 0 along the innermost dim
        bool ok = D.vec == 4 && nd >= 2 && D.dims[in] >= 128 && (!H.has_reduce || D.is_red[in]);
        for (unsigned i = 0; i < H.n_leaves && ok; i++) {
            const FLeaf &L = D.leaf[i];
            ok = L.masked == 0 && ((L.stride[in] == 1 && L.vec) || L.stride[in] == 0);
        }
        if (ok) {
            unsigned long long om = 1, sm = 1;
            for (int d = in - 1; d >= 0; d--) {
                D.omul[d] = D.smul[d] = 0;
                if (D.is_red[d]) { D.smul[d] = sm; sm *= D.dims[d]; } else { D.omul[d] = om; om *= D.dims[d]; }
            }
            if (sm <= 65535) { D.row_split = (unsigned)sm; F.rows_shape = true; }
        }
    }
    if (!H.has_reduce && D.vec == 2) { F.strategy = 0; F.name = D.chain ? "ew_vec2_static" : "ew_vec2_interp"; return true; }
    if (!H.has_reduce) { F.strategy = 0; F.flat_shape = all_flat; F.flat_name = D.chain ? "ew_flat_static" : "ew_flat_interp";
        F.rows_name = D.chain ? "ew_rows_static" : "ew_rows_interp"; F.name = D.chain ? (D.vec == 4 ? "ew_vec4_static" : "ew_scalar_static") : (D.vec == 4 ? "ew_vec4_interp" : "ew_scalar_interp"); return true; }
    if (D.is_red[in]) {
        F.strategy = 1;
        const unsigned long long items = D.n_red / D.vec;
        // A warp per output needs no block barrier; a CTA per output only pays off
        // when there are too few outputs for warps alone to keep HBM busy.
        F.group = items < 32 ? 1 : ((items < 1024 || D.n_out >= 16ull * sms) ? 32 : 256);
        if (F.group == 256 && D.n_out < 2ull * sms) {
            unsigned long long want = (4ull * sms + D.n_out - 1) / D.n_out;
            unsigned long long most = items / 1024;                 // keep >= 4 vectors per thread per slice
            if (want > most) want = most;
            if (want > 1) D.split = (unsigned)want;
        }
        if (all_flat && D.n_r == 1 && D.split == 1 && items >= 32 && items <= 0x7FFFFFFFull) {
            // contiguous rows: a CTA per row streams best once a row gives every thread two vectors
            F.flat_shape = true;
            if (items >= 512 && D.n_out >= 2ull * sms) F.group = 256;
            F.flat_shape = F.group != 1;
            F.flat_name = F.group == 256 ? "reduce_rows_cta" : "reduce_rows_warp";
        }
        F.name = F.group == 256 ? (D.split > 1 ? "reduce_inner_cta_split" : "reduce_inner_cta") : (F.group == 32 ? "reduce_inner_warp" : "reduce_inner_thread");
        F.rows_name = D.row_split > 1 ? "reduce_rows_split" : "reduce_rows";
        if (F.flat_shape) F.rows_shape = false;            // the all-flat form is the cheaper special case
        return true;
    }
    F.strategy = 2;
    F.rows_shape = false;
    D.vec = 1;
    const unsigned long long gx = (D.n_out + 31) / 32;
    if (gx > 0x7FFFFFFFull) return false;
    unsigned long long want = gx < 2ull * sms ? (2ull * sms + gx - 1) / gx : 1;
    unsigned long long most = (D.n_red + 31) / 32;
    if (want > most) want = most;
    if (want > 65535) want = 65535;
    D.split = want > 1 ? (unsigned)want : 1u;
    F.name = D.split > 1 ? "reduce_outer_split" : "reduce_outer";
    return true;
}

void classify_plan(Plan *p) {
    if (try_contraction(p)) return;
    if (try_pool2x2(p) || try_pool2x2_bwd(p) || try_pad2d(p) || try_window_to_plane(p) || try_crop2d(p)) return;
    FastDesc *F = new FastDesc();
    if (build_fast(p->host, *F)) { p->fast = (struct FastDesc *)F; p->kind = F->strategy == 0 ? PLAN_EW : PLAN_REDUCE; }
    else { delete F; p->fast = nullptr; p->kind = PLAN_GENERIC; }
}
void free_fast(Plan *p) { delete (FastDesc *)p->fast; p->fast = nullptr; free_contraction(p); }

// ------------------------------------------------------------------ host: launch
template <class EV>
static void launch_with(const FastDesc &F, const FDesc &D, float *out) {
    const unsigned long long items = D.numel / D.vec;
    if (F.flat && F.strategy == 0) {
        const unsigned long long ctas = (items + 256 * flat_unroll<EV>() - 1) / (256 * flat_unroll<EV>());
        k_ew_flat<EV><<<(unsigned)(ctas < 0x7FFFFFFFull ? ctas : 0x7FFFFFFFull), 256, 0, g.stream>>>(D, out);
        return;
    }
    if (F.flat && F.strategy == 1) {
        if (F.group == 256) k_rows<EV, 256><<<(unsigned)(D.n_out < 0x7FFFFFFFull ? D.n_out : 0x7FFFFFFFull), 256, 0, g.stream>>>(D, out);
        else                k_rows<EV, 32><<<grid_for(D.n_out, 8, 8), 256, 0, g.stream>>>(D, out);
        return;
    }
    if (F.rows) {
        const unsigned long long R = D.numel / D.dims[D.rank - 1];
        const bool cta = D.dims[D.rank - 1] / 4 >= 2048u;      // a CTA per row once a row gives every thread 8 vectors
        const unsigned grid = cta ? (unsigned)(R < 0x7FFFFFFFull ? R : 0x7FFFFFFFull) : grid_for(R, 8, 8);
        if (F.strategy == 0) {
            if (cta) k_rowsx<EV, 256, false><<<grid, 256, 0, g.stream>>>(D, out);
            else     k_rowsx<EV, 32, false><<<grid, 256, 0, g.stream>>>(D, out);
        } else {
            float *dst = D.split > 1 ? (float *)scratch_reserve(D.n_out * D.split * sizeof(float)) : out;
            if (cta) k_rowsx<EV, 256, true><<<grid, 256, 0, g.stream>>>(D, dst);
            else     k_rowsx<EV, 32, true><<<grid, 256, 0, g.stream>>>(D, dst);
        }
        return;
    }
    if (F.strategy == 0) {
        const unsigned grid = grid_for(items, 256, 8);
        if (D.vec == 4)      k_ew<EV, 4><<<grid, 256, 0, g.stream>>>(D, out);
        else if (D.vec == 2) k_ew<EV, 2><<<grid, 256, 0, g.stream>>>(D, out);
        else                 k_ew<EV, 1><<<grid, 256, 0, g.stream>>>(D, out);
        return;
    }
    float *dst = out;
    if (D.split > 1) dst = (float *)scratch_reserve(D.n_out * D.split * sizeof(float));
    if (F.strategy == 1) {
        const unsigned long long groups = D.n_out * D.split;
        if (F.group == 256) {
            const unsigned grid = grid_for(groups, 1, 8);
            if (D.vec == 4) k_red_inner<EV, 256, 4><<<grid, 256, 0, g.stream>>>(D, dst);
            else            k_red_inner<EV, 256, 1><<<grid, 256, 0, g.stream>>>(D, dst);
        } else if (F.group == 32) {
            const unsigned grid = grid_for(groups, 8, 8);
            if (D.vec == 4) k_red_inner<EV, 32, 4><<<grid, 256, 0, g.stream>>>(D, dst);
            else            k_red_inner<EV, 32, 1><<<grid, 256, 0, g.stream>>>(D, dst);
        } else {
            const unsigned grid = grid_for(groups, 256, 8);
            if (D.vec == 4) k_red_inner<EV, 1, 4><<<grid, 256, 0, g.stream>>>(D, dst);
            else            k_red_inner<EV, 1, 1><<<grid, 256, 0, g.stream>>>(D, dst);
        }
    } else {
        dim3 grid((unsigned)((D.n_out + 31) / 32), D.split);
        k_red_outer<EV><<<grid, 256, 0, g.stream>>>(D, dst);
    }
}

bool launch_fast(Plan *p, const GenArgs &args) {
    if (p->kind == PLAN_CONTRACT) return launch_contraction(p, args);
    if (p->kind == PLAN_POOL) return launch_pool2x2(p, args);
    if (p->kind == PLAN_POOL_BWD) return launch_pool2x2_bwd(p, args);
    if (p->kind == PLAN_PAD2D) return launch_pad2d(p, args);
    if (p->kind == PLAN_WIN2PLANE) return launch_window_to_plane(p, args);
    if (p->kind == PLAN_CROP2D) return launch_crop2d(p, args);
    FastDesc &F = *(FastDesc *)p->fast;
    FDesc D = F.d;
    for (unsigned i = 0; i < D.prog.n_leaves; i++) {
        // the leaf must stay inside its buffer; otherwise the checked generic kernel runs
        if (F.min_off[i] < 0 || (unsigned long long)F.max_off[i] >= args.cap[i]) return false;
        D.leaf[i].ptr = (const float *)args.leaf[i];
        if ((reinterpret_cast<uintptr_t>(args.leaf[i]) & 15u) != 0) D.leaf[i].vec = 0;
    }
    float *out = (float *)args.out;
    if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0) return false;
    F.flat = F.flat_shape;
    F.rows = F.rows_shape && !F.flat_shape;
    for (unsigned i = 0; i < D.prog.n_leaves; i++) {
        if (D.leaf[i].mode == 1 && !D.leaf[i].vec) F.flat = false;
        if (D.leaf[i].stride[D.rank - 1] == 1 && !D.leaf[i].vec) F.rows = false;
    }
    if (F.rows && F.strategy == 1) D.split = D.row_split;  // partial sums per output for the fold pass
    if (g.profile_level >= 2) {
        int w = snprintf(g.last_shape, sizeof g.last_shape, "dims=[");
        for (unsigned d = 0; d < D.rank; d++) w += snprintf(g.last_shape + w, sizeof g.last_shape - w, "%u%s%s", D.dims[d], D.is_red[d] ? "r" : "", d + 1 < D.rank ? "," : "");
        w += snprintf(g.last_shape + w, sizeof g.last_shape - w, "] vec=%u leaves:", D.vec);
        for (unsigned i = 0; i < D.prog.n_leaves; i++) {
            w += snprintf(g.last_shape + w, sizeof g.last_shape - w, " m%u(", D.leaf[i].mode);
            for (unsigned d = 0; d < D.rank; d++) w += snprintf(g.last_shape + w, sizeof g.last_shape - w, "%d%s", D.leaf[i].stride[d], d + 1 < D.rank ? "," : ")");
        }
    }
    profile_begin();
    switch (D.chain) {
        case 1: launch_with<StaticEval<1>>(F, D, out); break;
        case 2: launch_with<StaticEval<2>>(F, D, out); break;
        case 3: launch_with<StaticEval<3>>(F, D, out); break;
        case 4: launch_with<StaticEval<4>>(F, D, out); break;
        case 5: launch_with<StaticEval<5>>(F, D, out); break;
        case 6: launch_with<StaticEval<6>>(F, D, out); break;
        case 7: launch_with<StaticEval<7>>(F, D, out); break;
        case 8: launch_with<StaticEval<8>>(F, D, out); break;
        case 9: launch_with<StaticEval<9>>(F, D, out); break;
        case 10: launch_with<StaticEval<10>>(F, D, out); break;
        case 11: launch_with<StaticEval<11>>(F, D, out); break;
        case 12: launch_with<StaticEval<12>>(F, D, out); break;
        case 13: launch_with<StaticEval<13>>(F, D, out); break;
        case 14: launch_with<StaticEval<14>>(F, D, out); break;
        case 15: launch_with<StaticEval<15>>(F, D, out); break;
        case 16: launch_with<StaticEval<16>>(F, D, out); break;
        default: launch_with<InterpEval>(F, D, out); break;
    }
    after_launch(F.flat ? F.flat_name : (F.rows ? F.rows_name : F.name));
    if (F.strategy != 0 && D.split > 1) {
        if (D.split >= 64) k_red_final_warp<<<grid_for(D.n_out, 8, 4), 256, 0, g.stream>>>((const float *)g.scratch, out, D.n_out, D.split, D.rtype);
        else k_red_final<<<grid_for(D.n_out, 256, 4), 256, 0, g.stream>>>((const float *)g.scratch, out, D.n_out, D.split, D.rtype);
        after_launch("reduce_final");
    }
    return true;
}

}  // namespace thc

// ------------------------------------------------------------------ allocation-free entry point
// Per-channel sum of a contiguous [B, C, HW] f32 tensor (the batch-norm statistic,
// SUM over axes 0 and 2) for callers that must not allocate device memory while
// they run: a host that hands every byte of the GPU to its own arena up front, a
// step that is being recorded and therefore may not call the allocator, a
// latency-critical loop that cannot afford an allocator round trip.  The split
// reduce above normally takes its partial sums from pool scratch
// (cudaMallocAsync); here they live in a fixed array inside the library image,
// which every GPU that loads the library carries until the process exits.
namespace thc {

constexpr unsigned NOALLOC_MAX_PARTIALS = 65536;                 // floats: 256 KiB per GPU
static __device__ __align__(256) float noalloc_partials[NOALLOC_MAX_PARTIALS];

// `noalloc_partials` is only a host-side handle in host code; the device address
// has to be asked for, once per device, with that device current.
struct NoAllocDevice { float *scratch; int sm_count; bool ready; };
static NoAllocDevice noalloc_dev[64];

static int noalloc_setup(int dev) {
    NoAllocDevice &d = noalloc_dev[dev];
    if (d.ready) return 0;
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, noalloc_partials);
    if (e != cudaSuccess || !p) { cudaGetLastError(); set_error("channel_sums_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e)); return 2; }
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || sms <= 0) { cudaGetLastError(); set_error("channel_sums_noalloc: device attribute query: %s", cudaGetErrorString(e)); return 2; }
    d.scratch = (float *)p; d.sm_count = sms; d.ready = true;
    return 0;
}

}  // namespace thc

extern "C" int thvm_cuda_channel_sums_noalloc(const float *x, float *out, uint32_t B, uint32_t C, uint32_t HW, void *stream) {
    using namespace thc;
    if (!x || !out || B == 0 || C == 0 || HW == 0) { set_error("channel_sums_noalloc: null pointer or empty shape"); return 3; }
    if (C > NOALLOC_MAX_PARTIALS) {
        set_error("channel_sums_noalloc: %u channels exceed the built-in scratch of %u partial sums", C, NOALLOC_MAX_PARTIALS);
        return 1;
    }
    const unsigned long long n_red = (unsigned long long)B * HW, numel = n_red * C;
    if (n_red > 0xFFFFFFFFull || numel > (1ull << 40)) { set_error("channel_sums_noalloc: %llu elements per channel is out of range", n_red); return 1; }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); set_error("channel_sums_noalloc: no current CUDA device"); return 2; }
    if (int rc = noalloc_setup(dev)) return rc;
    const NoAllocDevice &nd = noalloc_dev[dev];

    // [B, C, HW] with dims 0 and 2 reduced; the leaf is laid out exactly like the iteration space
    FDesc D;
    memset(&D, 0, sizeof D);
    D.rank = 3; D.dims[0] = B; D.dims[1] = C; D.dims[2] = HW;
    D.is_red[0] = 1; D.is_red[2] = 1;
    D.n_k = 1; D.kd[0] = 1; D.n_r = 2; D.rd[0] = 0; D.rd[1] = 2;
    D.numel = numel; D.n_out = C; D.n_red = n_red; D.rtype = THC_SUM;
    D.fstride[2] = 1; D.fstride[1] = HW; D.fstride[0] = (unsigned long long)C * HW;
    const bool vec = HW % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    D.vec = vec ? 4u : 1u;
    D.prog.n_leaves = 1; D.prog.n_ops = 0; D.chain = 6;
    FLeaf &L = D.leaf[0];
    L.ptr = x; L.off = 0; L.mode = 1; L.vec = vec ? 1u : 0u;
    L.stride[0] = (int)((unsigned long long)C * HW > 0x7FFFFFFFull ? 0 : C * HW); L.stride[1] = (int)HW; L.stride[2] = 1;
    // split every channel across enough CTAs to fill the GPU, within the scratch size
    const unsigned long long items = n_red / D.vec;
    unsigned long long split = ((unsigned long long)4 * nd.sm_count + C - 1) / C;
    if (split > items / 1024) split = items / 1024;
    if (split > NOALLOC_MAX_PARTIALS / C) split = NOALLOC_MAX_PARTIALS / C;
    if (split < 1) split = 1;
    D.split = (unsigned)split;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned long long groups = (unsigned long long)C * D.split;
    const unsigned cap = (unsigned)nd.sm_count * 8u;
    const unsigned grid = (unsigned)(groups < cap ? groups : cap);
    // Every (channel, split) slot of the scratch is written before the second pass
    // reads it, so nothing has to be cleared between calls.
    float *dst = D.split > 1 ? nd.scratch : out;
    if (D.vec == 4) k_red_inner<StaticEval<6>, 256, 4><<<grid, 256, 0, s>>>(D, dst);
    else            k_red_inner<StaticEval<6>, 256, 1><<<grid, 256, 0, s>>>(D, dst);
    if (D.split > 1) k_red_final<<<(C + 255) / 256, 256, 0, s>>>(nd.scratch, out, C, D.split, THC_SUM);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("channel_sums_noalloc: launch failed: %s", cudaGetErrorString(e)); return 2; }
    g.launches += D.split > 1 ? 2 : 1;
    return 0;
}
