// layout.cu — bandwidth kernels for the layout-changing copies every convolutional training step is full of:
//   * padding materialised as ADD(pad(x), z): out[.., y, x] = in[.., y - pt, x - pl] + z inside the mask, 0 + z outside
//     (src/tensor/view/pad.c:2-16 turns PAD into a mask and a negative offset; the staged convolutions realise it
//     before the convolution reads it);
//   * the opposite, a window cut out of every padded plane (SHRINK materialised): the valid part of a gradient;
//   * window layout back to plane layout, out[.., oy, i, ox, j] = in[.., oy, ox, i, j] + z: the copy that follows the
//     max-pool gradient (the pooled dims are split into windows by reshape + permute, src/nn/conv.c:484-513).
// The general elementwise kernel decodes a rank-4..6 coordinate per pair of outputs for these (innermost dims of 66
// or 2 floats); here a padded plane is walked as the flat run it is, four outputs and one division per thread, and a
// pair of 2x2 windows is two 16-byte loads and two 16-byte stores.  `z` is the dispatch's scalar leaf (the ADD is
// kept: -0.0 + 0.0 is +0.0, bit for bit what the CPU computes).
#include "device_common.cuh"
#include "plans.h"
#include "state.h"

namespace thc {

// grid.x = plane, grid.y * 256 threads cover the plane's Hp * Wp / 4 groups of four outputs
__global__ void __launch_bounds__(256) k_pad2d(const float *__restrict__ x, const float *__restrict__ zp, float *__restrict__ y,
                                               unsigned H, unsigned W, unsigned Hp, unsigned Wp, unsigned pt, unsigned pl, unsigned has_z) {
    const unsigned long long plane = blockIdx.x;
    const unsigned quads = Hp * Wp / 4u;
    const float z = has_z ? zp[0] : 0.0f;
    const float *src = x + plane * H * W;
    float4 *dst = reinterpret_cast<float4 *>(y + plane * (unsigned long long)Hp * Wp);
    for (unsigned q = blockIdx.y * 256u + threadIdx.x; q < quads; q += gridDim.y * 256u) {
        const unsigned f = 4u * q;
        unsigned yy = f / Wp, xx = f - yy * Wp;
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const unsigned sy = yy - pt, sx = xx - pl;                  // unsigned: below the mask wraps to a huge value
            const float in = (sy < H && sx < W) ? __ldg(src + sy * W + sx) : 0.0f;
            v[i] = has_z ? __fadd_rn(in, z) : in;
            if (++xx == Wp) { xx = 0; yy++; }
        }
        dst[q] = make_float4(v[0], v[1], v[2], v[3]);
    }
}

// The opposite copy: an H x W window cut out of every plane of pitch Ws (a SHRINK, e.g. the valid part of a padded
// gradient), out[plane, y, x] = in[plane * Ps + (y * Ws + x)] + z with `in` already at the window's first element.
// grid.x = plane, grid.y * 256 threads cover the plane's H * W / 4 groups of four outputs (W is a multiple of 4, so a
// group never leaves its row); the source rows start anywhere, so they are read element by element, 128 bytes per warp.
__global__ void __launch_bounds__(256) k_crop2d(const float *__restrict__ x, const float *__restrict__ zp, float *__restrict__ y,
                                                unsigned H, unsigned W, unsigned Ws, unsigned long long Ps, unsigned has_z) {
    const unsigned long long plane = blockIdx.x;
    const unsigned quads = H * W / 4u;
    const float z = has_z ? zp[0] : 0.0f;
    const float *src = x + plane * Ps;
    float4 *dst = reinterpret_cast<float4 *>(y + plane * (unsigned long long)H * W);
    for (unsigned q = blockIdx.y * 256u + threadIdx.x; q < quads; q += gridDim.y * 256u) {
        const unsigned f = 4u * q, yy = f / W, xx = f - yy * W;
        const float *s = src + (unsigned long long)yy * Ws + xx;
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; i++) { const float in = __ldg(s + i); v[i] = has_z ? __fadd_rn(in, z) : in; }
        dst[q] = make_float4(v[0], v[1], v[2], v[3]);
    }
}

// one thread per pair of neighbouring windows: in [planes, OH, OW, 2, 2] -> out [planes, 2 OH, 2 OW]
__global__ void __launch_bounds__(256) k_window_to_plane(const float *__restrict__ x, const float *__restrict__ zp, float *__restrict__ y,
                                                         unsigned long long rows, unsigned OW, unsigned has_z) {
    const unsigned half = OW / 2u;                                      // pairs of windows per window row
    const float z = has_z ? zp[0] : 0.0f;
    const unsigned long long items = rows * half;                       // rows = planes * OH
    for (unsigned long long it = (unsigned long long)blockIdx.x * 256 + threadIdx.x; it < items; it += (unsigned long long)gridDim.x * 256) {
        const unsigned long long r = it / half;
        const unsigned c = (unsigned)(it - r * half);
        const float4 *in = reinterpret_cast<const float4 *>(x + (r * OW + 2ull * c) * 4ull);
        float4 a = __ldg(in), b = __ldg(in + 1);
        if (has_z) {
            a.x = __fadd_rn(a.x, z); a.y = __fadd_rn(a.y, z); a.z = __fadd_rn(a.z, z); a.w = __fadd_rn(a.w, z);
            b.x = __fadd_rn(b.x, z); b.y = __fadd_rn(b.y, z); b.z = __fadd_rn(b.z, z); b.w = __fadd_rn(b.w, z);
        }
        float *o = y + (2ull * r) * (2ull * OW) + 4ull * c;             // output row 2 r, column 4 c
        *reinterpret_cast<float4 *>(o) = make_float4(a.x, a.y, b.x, b.y);
        *reinterpret_cast<float4 *>(o + 2ull * OW) = make_float4(a.z, a.w, b.z, b.w);
    }
}

// the dispatch is `leaf0` alone, or ADD(leaf0, scalar leaf1) in either operand order
static bool copy_or_add_scalar(const GenDesc &H, int &src, int &sc) {
    if (H.has_reduce || H.post_start || H.out_dtype != THC_F32) return false;
    if (H.n_leaves == 1 && H.n_ops == 0) { src = 0; sc = -1; return H.leaves[0].dtype == THC_F32 && H.leaves[0].tracker < 0; }
    if (H.n_leaves != 2 || H.n_ops != 1 || H.ops[0].uop != THC_ADD) return false;
    if (!((H.ops[0].arg_a == 0 && H.ops[0].arg_b == 1) || (H.ops[0].arg_a == 1 && H.ops[0].arg_b == 0))) return false;
    auto is_scalar = [&](const DLeaf &L) {
        if (L.dtype != THC_F32 || L.tracker >= 0 || L.v.has_mask || L.v.offset < 0) return false;
        for (unsigned d = 0; d < L.v.rank; d++) if (L.v.dims[d] != 1 && L.v.strides[d] != 0) return false;
        return true;
    };
    for (int s = 0; s < 2; s++)
        if (is_scalar(H.leaves[1 - s]) && H.leaves[s].dtype == THC_F32 && H.leaves[s].tracker < 0) { src = s; sc = 1 - s; return true; }
    return false;
}

bool try_pad2d(Plan *p) {
    const GenDesc &H = p->host;
    int src, sc;
    if (!copy_or_add_scalar(H, src, sc)) return false;
    const DLeaf &L = H.leaves[src];
    const int r = (int)H.rank;
    if (r < 2 || (int)L.v.rank != r || !L.v.has_mask || L.v.n_cm) return false;
    for (int d = 0; d < r; d++) if (L.v.dims[d] != H.full_dims[d]) return false;
    const unsigned Hp = H.full_dims[r - 2], Wp = H.full_dims[r - 1];
    const unsigned pt = L.v.mb[r - 2], pl = L.v.mb[r - 1];
    if (L.v.me[r - 2] > Hp || L.v.me[r - 1] > Wp || L.v.me[r - 2] <= pt || L.v.me[r - 1] <= pl) return false;
    const unsigned Hs = L.v.me[r - 2] - pt, Ws = L.v.me[r - 1] - pl;
    if (L.v.strides[r - 1] != 1 || L.v.strides[r - 2] != (int)Ws) return false;
    unsigned long long planes = 1, want = (unsigned long long)Hs * Ws;
    for (int d = r - 3; d >= 0; d--) {
        if (L.v.mb[d] != 0 || L.v.me[d] < H.full_dims[d]) return false;                 // outer dims carry no padding
        if (H.full_dims[d] != 1 && (unsigned long long)L.v.strides[d] != want) return false;
        planes *= H.full_dims[d]; want *= H.full_dims[d];
    }
    if ((long long)L.v.offset != -((long long)pt * Ws + pl)) return false;
    if (((unsigned long long)Hp * Wp) % 4 != 0 || Wp < 4 || planes > 0x7FFFFFFFull || (unsigned long long)Hp * Wp > 0xFFFFFFFFull) return false;
    p->pool_planes = planes; p->pool_h = Hs; p->pool_w = Ws;
    p->pool_off = ((long long)Hp << 32) | Wp;        // padded extents
    p->pool_g_off = ((long long)pt << 32) | pl;      // top / left padding
    p->pool_m_off = src; p->pool_one_off = sc >= 0 ? H.leaves[sc].v.offset : 0;
    p->kind = PLAN_PAD2D;
    return true;
}

bool launch_pad2d(Plan *p, const GenArgs &args) {
    const int src = (int)p->pool_m_off, sc = p->host.n_leaves == 2 ? 1 - src : -1;
    const unsigned Hp = (unsigned)(p->pool_off >> 32), Wp = (unsigned)(p->pool_off & 0xFFFFFFFFll);
    const unsigned pt = (unsigned)(p->pool_g_off >> 32), pl = (unsigned)(p->pool_g_off & 0xFFFFFFFFll);
    const unsigned long long in_n = p->pool_planes * p->pool_h * p->pool_w;
    if (in_n > args.cap[src] || (sc >= 0 && (unsigned long long)p->pool_one_off >= args.cap[sc])) return false;   // the checked generic kernel runs instead
    if (reinterpret_cast<uintptr_t>(args.out) & 15u) return false;
    const float *z = sc >= 0 ? (const float *)args.leaf[sc] + p->pool_one_off : nullptr;
    const unsigned quads = Hp * Wp / 4u;
    unsigned gy = (quads + 255u) / 256u;
    if (gy > 8u) gy = 8u;
    if (g.profile_level >= 2) snprintf(g.last_shape, sizeof g.last_shape, "planes=%llu %ux%u -> %ux%u", p->pool_planes, p->pool_h, p->pool_w, Hp, Wp);
    profile_begin();
    k_pad2d<<<dim3((unsigned)p->pool_planes, gy), 256, 0, g.stream>>>((const float *)args.leaf[src], z, (float *)args.out, p->pool_h, p->pool_w, Hp, Wp, pt, pl, sc >= 0 ? 1u : 0u);
    after_launch("pad_planes");
    return true;
}

bool try_crop2d(Plan *p) {
    const GenDesc &H = p->host;
    int src, sc;
    if (!copy_or_add_scalar(H, src, sc)) return false;
    const DLeaf &L = H.leaves[src];
    const int r = (int)H.rank;
    if (r < 3 || (int)L.v.rank != r || L.v.has_mask || L.v.n_cm || L.v.offset < 0) return false;
    for (int d = 0; d < r; d++) if (L.v.dims[d] != H.full_dims[d]) return false;
    const unsigned Hc = H.full_dims[r - 2], Wc = H.full_dims[r - 1];
    if (L.v.strides[r - 1] != 1 || L.v.strides[r - 2] <= (int)Wc || Wc % 4 != 0 || Hc == 0) return false;     // (pitch == W is a plain copy: other kernels)
    const unsigned Ws = (unsigned)L.v.strides[r - 2];
    // the planes form one run of constant pitch Ps
    int d0 = r - 3;
    while (d0 >= 0 && H.full_dims[d0] == 1) d0--;
    if (d0 < 0) return false;
    const long long Ps = L.v.strides[d0];
    if (Ps < (long long)(Hc - 1) * Ws + Wc) return false;
    unsigned long long planes = 1, want = (unsigned long long)Ps;
    for (int d = r - 3; d >= 0; d--) {
        if (H.full_dims[d] != 1 && (unsigned long long)L.v.strides[d] != want) return false;
        planes *= H.full_dims[d]; want *= H.full_dims[d];
    }
    if (planes > 0x7FFFFFFFull || (unsigned long long)Hc * Wc > 0xFFFFFFFFull) return false;
    p->pool_planes = planes; p->pool_h = Hc; p->pool_w = Wc;
    p->pool_off = L.v.offset;                       // first element of the window in plane 0
    p->pool_g_off = (Ps << 32) | (long long)Ws;     // plane pitch / row pitch (both below 2^31: strides are 32-bit)
    p->pool_m_off = src; p->pool_one_off = sc >= 0 ? H.leaves[sc].v.offset : 0;
    p->kind = PLAN_CROP2D;
    return true;
}

bool launch_crop2d(Plan *p, const GenArgs &args) {
    const int src = (int)p->pool_m_off, sc = p->host.n_leaves == 2 ? 1 - src : -1;
    const unsigned long long Ps = (unsigned long long)(p->pool_g_off >> 32);
    const unsigned Ws = (unsigned)(p->pool_g_off & 0xFFFFFFFFll);
    const unsigned long long last = (unsigned long long)p->pool_off + (p->pool_planes - 1) * Ps + (unsigned long long)(p->pool_h - 1) * Ws + p->pool_w - 1;
    if (last >= args.cap[src] || (sc >= 0 && (unsigned long long)p->pool_one_off >= args.cap[sc])) return false;   // the checked generic kernel runs instead
    if (reinterpret_cast<uintptr_t>(args.out) & 15u) return false;
    const float *z = sc >= 0 ? (const float *)args.leaf[sc] + p->pool_one_off : nullptr;
    const unsigned quads = p->pool_h * p->pool_w / 4u;
    unsigned gy = (quads + 255u) / 256u;
    if (gy > 8u) gy = 8u;
    if (g.profile_level >= 2) snprintf(g.last_shape, sizeof g.last_shape, "planes=%llu %ux%u out of pitch %u", p->pool_planes, p->pool_h, p->pool_w, Ws);
    profile_begin();
    k_crop2d<<<dim3((unsigned)p->pool_planes, gy), 256, 0, g.stream>>>((const float *)args.leaf[src] + p->pool_off, z, (float *)args.out, p->pool_h, p->pool_w, Ws, Ps, sc >= 0 ? 1u : 0u);
    after_launch("crop_planes");
    return true;
}

bool try_window_to_plane(Plan *p) {
    const GenDesc &H = p->host;
    int src, sc;
    if (!copy_or_add_scalar(H, src, sc)) return false;
    const DLeaf &L = H.leaves[src];
    const int r = (int)H.rank;
    if (r < 4 || (int)L.v.rank != r || L.v.has_mask || L.v.n_cm || L.v.offset < 0 || L.v.offset % 4 != 0) return false;
    for (int d = 0; d < r; d++) if (L.v.dims[d] != H.full_dims[d]) return false;
    // iteration dims [.., OH, 2, OW, 2] over a source stored as [.., OH, OW, 2, 2]
    if (H.full_dims[r - 1] != 2 || H.full_dims[r - 3] != 2) return false;
    const unsigned long long OW = H.full_dims[r - 2], OH = H.full_dims[r - 4];
    if (OW < 2 || OW % 2 != 0) return false;
    if (L.v.strides[r - 1] != 1 || L.v.strides[r - 2] != 4 || L.v.strides[r - 3] != 2 || L.v.strides[r - 4] != (long long)(4 * OW)) return false;
    unsigned long long planes = 1, want = 4 * OW * OH;
    for (int d = r - 5; d >= 0; d--) {
        if (H.full_dims[d] != 1 && (unsigned long long)L.v.strides[d] != want) return false;
        planes *= H.full_dims[d]; want *= H.full_dims[d];
    }
    p->pool_planes = planes * OH; p->pool_w = (uint32_t)OW;
    p->pool_off = L.v.offset; p->pool_m_off = src; p->pool_one_off = sc >= 0 ? H.leaves[sc].v.offset : 0;
    p->kind = PLAN_WIN2PLANE;
    return true;
}

bool launch_window_to_plane(Plan *p, const GenArgs &args) {
    const int src = (int)p->pool_m_off, sc = p->host.n_leaves == 2 ? 1 - src : -1;
    const unsigned long long n = p->pool_planes * p->pool_w * 4ull;
    if ((unsigned long long)p->pool_off + n > args.cap[src] || (sc >= 0 && (unsigned long long)p->pool_one_off >= args.cap[sc])) return false;
    const float *x = (const float *)args.leaf[src] + p->pool_off;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(args.out)) & 15u) return false;
    const float *z = sc >= 0 ? (const float *)args.leaf[sc] + p->pool_one_off : nullptr;
    if (g.profile_level >= 2) snprintf(g.last_shape, sizeof g.last_shape, "window rows=%llu OW=%u", p->pool_planes, p->pool_w);
    profile_begin();
    k_window_to_plane<<<grid_for(p->pool_planes * (p->pool_w / 2), 256, 8), 256, 0, g.stream>>>(x, z, (float *)args.out, p->pool_planes, p->pool_w, sc >= 0 ? 1u : 0u);
    after_launch("window_to_plane");
    return true;
}

}  // namespace thc
