// gemm.cu — contraction kernel on the 5th-generation tensor cores (tcgen05,
// accumulators in tensor memory) with a 3xTF32 operand split that keeps f32
// accuracy: x = hi + lo with hi = tf32(x), lo = tf32(x - hi), and
//     a*b ~= a_lo*b_hi + a_hi*b_lo + a_hi*b_hi        (f32 accumulate in TMEM).
//
// It serves every SUM(MUL(a,b)) dispatch whose operands are separable
// (gemm_desc.h): matmul in all four transpose forms, and convolution forward /
// weight gradient / input gradient, which the reference expresses as MUL + SUM
// over expanded pool views (src/ctx/init.c:555-582, src/nn/conv.c:390-478) and
// its CPU backend evaluates one product at a time (src/backend/cpu/dispatch.c:169-218).
//
// Kernels in this translation unit, chosen per plan by the recogniser (gemm_host.inc):
//   k_gemm_ps            (gemm_ps.inc) persistent single-CTA kernel for outputs of at most 128 columns: one CTA per SM
//                        walks 128-row tiles; A tiles, B tiles and tensor-memory stages are three rings; the A operand
//                        goes to tensor memory (hi and lo split in registers), accumulators are double-buffered so
//                        the epilogue of one tile overlaps the next tile's MMAs;
//   k_gemm_pair_ta       (gemm_ta.inc) CTA pair, 256-row tiles, A operand in tensor memory, B by tile loads: wider
//                        outputs (the 4096^3 matrices, 256-channel convolutions);
//   k_gemm_pair_3xtf32   CTA pair, operands gathered with cp.async through separable offsets (implicit im2col for what
//                        the tile-load forms do not cover: 3 input channels, odd pitches, K not a multiple of 4);
//   k_gemm_3xtf32        single CTA, 128x128 tile, same gather, for outputs with fewer than 256 rows;
//   k_skinny_rows / _k   (gemm_skinny.inc) CUDA-core kernels for shapes too thin for a tensor-core tile.
// The two gather kernels below share this structure: sixteen producer warps put 128x32 k-blocks of A and B into
// shared memory in the K-major 128-byte-swizzled layout the MMA reads.  The raw f32 tile is the high part
// as it stands (the tf32 MMA ignores the low 13 mantissa bits); a pass over the tile writes the low parts.
// One elected lane of the MMA warp issues, per k-block, 4 k-steps x 3 products and hands the stage back
// with tcgen05.commit.  After the last k-block the producer warps read the accumulators back with
// tcgen05.ld and store C through its separable offsets.  Stages are guarded by mbarriers; every wait is
// bounded and raises a status bit instead of hanging.
#include <string.h>
#include <vector>
#include "device_common.cuh"
#include "gemm_desc.h"
#include "plans.h"
#include "state.h"

namespace thc {

constexpr int BM = 128, BN = 128, BK = 32;
constexpr int STAGES = 4;                           // raw (= high part) k-blocks resident: A and B tile each
constexpr int LO_STAGES = 2;                        // low-part k-blocks resident
constexpr int TILE_BYTES = 128 * BK * 4;            // one 128 x 32 f32 tile
constexpr int STAGE_BYTES = 2 * TILE_BYTES;         // one k-block of one ring: A tile, B tile
constexpr int LO_BASE = STAGES * STAGE_BYTES;       // the low-part ring follows the raw ring
constexpr int PROD_WARPS = 16;                      // producer warps (multiple of 4: the epilogue splits the columns among them)
constexpr int NPROD = PROD_WARPS * 32;              // producer threads
constexpr int UNITS = 1024 / NPROD;                 // (row, 16-byte chunk) units of a 128 x 32 tile per producer thread
constexpr int GEMM_THREADS = NPROD + 32;            // + 1 MMA warp
constexpr int MMA_WARP = PROD_WARPS;
constexpr int TMEM_COLS = 128;
constexpr int LOOKAHEAD = 2;                        // k-blocks of cp.async in flight ahead of the split pass
constexpr uint32_t WAIT_LIMIT = 1u << 24;
enum : int { ERR_GEMM_TIMEOUT = 8 };

struct GemmShared {                                 // follows the tile area in dynamic shared memory
    long long am[BM], bn[BN], cm[BM], cn[BN];
    unsigned long long full[STAGES], empty[STAGES], accum;
    uint32_t tmem_base;
    int abort_flag;
};
constexpr int TILE_AREA = (STAGES + LO_STAGES) * STAGE_BYTES;
constexpr size_t GEMM_SMEM = (size_t)TILE_AREA + sizeof(GemmShared) + 1024;   // + alignment slack

// ---- PTX wrappers ----
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// bounded wait: false after WAIT_LIMIT polls or when another thread gave up
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ uint32_t to_tf32(float x) { uint32_t u; asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x)); return u; }
// x = hi + lo with hi = x truncated to tf32 (what the MMA sees of the raw f32); lo is
// exact in f32.  (An infinite x gives lo = nan, so inf inputs yield nan outputs.)
__device__ __forceinline__ uint32_t tf32_low(uint32_t xbits) {
    return __float_as_uint(__uint_as_float(xbits) - __uint_as_float(xbits & 0xFFFFE000u));
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// instruction descriptor: D f32, A/B tf32, both K-major, N = 128, M = 128
constexpr uint32_t UMMA_IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

// mixed-radix decode of an index into its A/B and C element offsets
__device__ __forceinline__ void decode_group(const GSub *subs, uint32_t n, uint32_t idx, bool use_b, long long &op, long long &oc) {
    op = 0; oc = 0;
    for (int i = (int)n - 1; i >= 0; i--) {
        const uint32_t sz = subs[i].size, q = idx / sz, c = idx - q * sz;
        op += (long long)c * (use_b ? subs[i].sb : subs[i].sa);
        oc += (long long)c * subs[i].sc;
        idx = q;
    }
}

// ---- producers: cp.async gather into the swizzled tile, then the low-part pass ----
// Thread t of the NPROD producers owns UNITS (row, 16-byte chunk) units of each 128x32
// operand tile: along k when k is the operand's contiguous direction (a warp
// covers 4 rows x 128 bytes), else along the rows (a warp covers 32 rows of one
// chunk, element-wise 4-byte copies that coalesce across lanes).
__device__ __forceinline__ void unit_of(uint32_t kfast, uint32_t t, int i, uint32_t &row, uint32_t &chunk) {
    if (kfast) { row = (t >> 3) + (uint32_t)(NPROD / 8) * (uint32_t)i; chunk = t & 7u; }
    else       { row = t & 127u; chunk = (t >> 7) + (uint32_t)(NPROD / 128) * (uint32_t)i; }
}
__device__ __forceinline__ uint32_t unit_offset(uint32_t row, uint32_t chunk) {
    return (row >> 3) * 1024u + (row & 7u) * 128u + ((chunk ^ (row & 7u)) << 4);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src, uint32_t bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
// what a producer thread needs per operand, fixed for the whole tile: the global row
// pointers, the column (k) offsets and the swizzled tile offsets of its 4 units
struct UnitSet {
    const float *rowptr[UNITS];
    uint32_t kcol[UNITS], soff[UNITS], live;       // live: bit i set when unit i's row is inside the matrix
};
__device__ __forceinline__ void make_units(UnitSet &U, const float *P, long long base, const long long *rowoff,
                                           uint32_t rows_valid, uint32_t kfast, uint32_t t) {
    U.live = 0;
#pragma unroll
    for (int i = 0; i < UNITS; i++) {
        uint32_t row, chunk;
        unit_of(kfast, t, i, row, chunk);
        const bool ok = row < rows_valid;
        U.rowptr[i] = ok ? P + base + rowoff[row] : P;
        U.kcol[i] = 4u * chunk;
        U.soff[i] = unit_offset(row, chunk);
        if (ok) U.live |= 1u << i;
    }
}
// issue the asynchronous copies of one operand k-block into its raw (= high part) tile;
// k past K is zero-filled (source size 0); rows past the matrix edge are skipped.  `klin` != 0:
// the operand's k offset is k * klin (a single reduced dim), else it comes from `ktab`.
__device__ __forceinline__ void issue_tile(const UnitSet &U, const float *P, const int32_t *__restrict__ ktab, long long klin,
                                           uint32_t k0, uint32_t K, uint32_t kvec, uint32_t tile) {
#pragma unroll
    for (int i = 0; i < UNITS; i++) {
        const uint32_t k = k0 + U.kcol[i], dst = tile + U.soff[i];
        const bool row_ok = (U.live >> i) & 1u;
        if (!row_ok) continue;                 // rows past the edge: their products land in accumulator rows / columns nobody stores
        if (kvec) {
            const bool in = row_ok && k < K;
            const long long ko = klin ? (long long)k * klin : (long long)(in ? ktab[k] : 0);
            cp_async16(dst, in ? U.rowptr[i] + ko : P, in ? 16u : 0u);
        } else {
            // four 4-byte copies; the four k offsets come with one 16-byte load (k is a multiple of 4 and the
            // table is padded with zeros to a multiple of 32 entries), nv = how many of them are inside K
            const uint32_t nv = (row_ok && k < K) ? (K - k < 4u ? K - k : 4u) : 0u;
            long long o0, o1, o2, o3;
            if (klin) { o0 = (long long)k * klin; o1 = o0 + klin; o2 = o1 + klin; o3 = o2 + klin; }
            else { const int4 t = *reinterpret_cast<const int4 *>(ktab + k); o0 = t.x; o1 = t.y; o2 = t.z; o3 = t.w; }
            const float *rp = U.rowptr[i];
            cp_async4(dst, nv > 0u ? rp + o0 : P, nv > 0u ? 4u : 0u);
            cp_async4(dst + 4u, nv > 1u ? rp + o1 : P, nv > 1u ? 4u : 0u);
            cp_async4(dst + 8u, nv > 2u ? rp + o2 : P, nv > 2u ? 4u : 0u);
            cp_async4(dst + 12u, nv > 3u ? rp + o3 : P, nv > 3u ? 4u : 0u);
        }
    }
}
// low-part pass over this thread's own units: lo = x - trunc_tf32(x).  The raw f32
// tile doubles as the high part: the tf32 MMA reads only the upper 19 bits.
__device__ __forceinline__ void split_tile(const UnitSet &U, uint32_t raw_tile, uint32_t lo_tile) {
#pragma unroll
    for (int i = 0; i < UNITS; i++) {
        if (!((U.live >> i) & 1u)) continue;
        uint32_t x0, x1, x2, x3;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3) : "r"(raw_tile + U.soff[i]) : "memory");
        st_shared_v4(lo_tile + U.soff[i], tf32_low(x0), tf32_low(x1), tf32_low(x2), tf32_low(x3));
    }
}

__global__ void __launch_bounds__(GEMM_THREADS, 1) k_gemm_3xtf32(const __grid_constant__ GemmDesc G) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *tiles = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    GemmShared &S = *reinterpret_cast<GemmShared *>(tiles + (size_t)TILE_AREA);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // tile order: bands of 8 row-tiles, column-tiles fastest inside a band, so the CTAs
    // that run together share a few A and B panels that stay in L2
    const uint32_t tm = (G.M + BM - 1) / BM, tn = (G.N + BN - 1) / BN;
    const uint32_t BH = 8u;                                          // band height in row tiles
    const uint32_t band = BH * tn, b0 = (blockIdx.x / band) * BH;
    const uint32_t bh = tm - b0 < BH ? tm - b0 : BH, within = blockIdx.x % band;
    const uint32_t m0 = (b0 + within % bh) * BM, n0 = (within / bh) * BN;
    const uint32_t nkb_all = (G.K + BK - 1) / BK;
    const uint32_t kb_lo = blockIdx.z * G.kb_chunk;                       // this CTA's share of the k-blocks (split-K)
    const uint32_t nkb = nkb_all - kb_lo < G.kb_chunk ? nkb_all - kb_lo : G.kb_chunk;
    volatile int *abort_flag = &S.abort_flag;

    // ---- setup: barriers, tensor memory, row / column offsets of this tile ----
    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(smem_u32(&S.full[s]), NPROD); mbar_init(smem_u32(&S.empty[s]), 1); }
        mbar_init(smem_u32(&S.accum), 1);
        S.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&S.tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid < BM) {
        long long oa = 0, oc = 0;
        if (m0 + tid < G.M) decode_group(G.md, G.nm, m0 + tid, false, oa, oc);
        if (G.partial) oc = ((long long)blockIdx.z * G.M + (m0 + tid)) * G.N;      // dense partial tile
        S.am[tid] = oa; S.cm[tid] = oc;
    } else if (tid < BM + BN) {
        const uint32_t j = tid - BM;
        long long ob = 0, oc = 0;
        if (n0 + j < G.N) decode_group(G.nd, G.nn, n0 + j, true, ob, oc);
        if (G.partial) oc = n0 + j;
        S.bn[j] = ob; S.cn[j] = oc;
    }
    float *const Cout = G.partial ? G.partial : G.C;
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = S.tmem_base;
    const uint32_t tiles_s = smem_u32(tiles);
    const uint32_t rows_a = G.M - m0 < (uint32_t)BM ? G.M - m0 : (uint32_t)BM;
    const uint32_t rows_b = G.N - n0 < (uint32_t)BN ? G.N - n0 : (uint32_t)BN;

    if (warp < MMA_WARP) {
        // ================= producers =================
        const uint32_t t = tid;                                          // 0..NPROD-1
        bool ok = true;
        UnitSet UA, UB;
        make_units(UA, G.A, G.a_off, S.am, rows_a, G.a_kfast, t);
        make_units(UB, G.B, G.b_off, S.bn, rows_b, G.b_kfast, t);
        auto issue = [&](uint32_t kb) {                                  // copies for local k-block kb into its stage
            const uint32_t st = tiles_s + (kb % STAGES) * STAGE_BYTES, k0 = (kb_lo + kb) * BK;
            issue_tile(UA, G.A, G.ka, G.a_klin, k0, G.K, G.a_kvec, st);
            issue_tile(UB, G.B, G.kb, G.b_klin, k0, G.K, G.b_kvec, st + TILE_BYTES);
        };
        // prologue: LOOKAHEAD k-blocks in flight (one commit group per k-block, empty groups keep the count uniform)
        for (uint32_t kb = 0; kb < (uint32_t)LOOKAHEAD; kb++) {
            if (kb < nkb) issue(kb);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        for (uint32_t kb = 0; kb < nkb && ok; kb++) {
            // k-block kb has landed (this thread's part).  Its low parts go to lo[kb % 2], which
            // the MMAs of k-block kb - 2 were the last to read.
            asm volatile("cp.async.wait_group %0;" ::"n"(LOOKAHEAD - 1) : "memory");
            if (kb >= (uint32_t)LO_STAGES) {
                const uint32_t prev = kb - LO_STAGES;
                ok = mbar_wait(smem_u32(&S.empty[prev % STAGES]), (prev / STAGES) & 1u, abort_flag);
                if (!ok) break;
            }
            const uint32_t st = tiles_s + (kb % STAGES) * STAGE_BYTES, lo = tiles_s + LO_BASE + (kb % LO_STAGES) * STAGE_BYTES;
            split_tile(UA, st, lo);
            split_tile(UB, st + TILE_BYTES, lo + TILE_BYTES);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");              // generic-proxy writes -> visible to the MMA
            mbar_arrive(smem_u32(&S.full[kb % STAGES]));
            // refill the raw stage whose MMAs (k-block kb - 1) finish next: three k-blocks of copies stay in flight
            const uint32_t nxt = kb + LOOKAHEAD;
            if (nxt < nkb) {
                const uint32_t use = nxt / STAGES;                       // stage (nxt % STAGES) was last read by k-block nxt - STAGES
                if (use >= 1) ok = mbar_wait(smem_u32(&S.empty[nxt % STAGES]), (use - 1) & 1u, abort_flag);
                if (ok) issue(nxt);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        // ================= epilogue =================
        if (ok) ok = mbar_wait(smem_u32(&S.accum), 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);                                 // tcgen05.ld needs the whole warp
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            // warp w may read TMEM lanes 32*(w%4)..+31; the PROD_WARPS/4 warps of a lane quarter share its 128 columns
            constexpr int COLS_PER_WARP = BN / (PROD_WARPS / 4);
            const uint32_t q = warp & 3u, part = warp >> 2;
            const uint32_t row = q * 32u + lane;
            const bool row_ok = row < rows_a;
            const long long crow = S.cm[row];
#pragma unroll
            for (int c = 0; c < COLS_PER_WARP / 32; c++) {
                const uint32_t col0 = part * (uint32_t)COLS_PER_WARP + (uint32_t)c * 32u;
                uint32_t r[32];
                const uint32_t taddr = tmem + ((q * 32u) << 16) + col0;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                             "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                             "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                               "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                               "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                               "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                             : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row_ok) {
                    if (G.c_nvec && col0 + 32u <= rows_b) {
                        float4 *dst = reinterpret_cast<float4 *>(Cout + crow + S.cn[col0]);
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                 __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (col0 + j < rows_b) Cout[crow + S.cn[col0 + j]] = __uint_as_float(r[j]);
                    }
                }
            }
        }
    } else {
        // ================= MMA issuer =================
        if (lane == 0) {
            bool ok = true;
            for (uint32_t kb = 0; kb < nkb && ok; kb++) {
                const uint32_t s = kb % STAGES, use = kb / STAGES;
                ok = mbar_wait(smem_u32(&S.full[s]), use & 1u, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t st = tiles_s + s * STAGE_BYTES, lo = tiles_s + LO_BASE + (kb % LO_STAGES) * STAGE_BYTES;
                const uint64_t a_hi = umma_desc(st), b_hi = umma_desc(st + TILE_BYTES);
                const uint64_t a_lo = umma_desc(lo), b_lo = umma_desc(lo + TILE_BYTES);
#pragma unroll
                for (uint32_t ks = 0; ks < (uint32_t)(BK / 8); ks++) {
                    const uint64_t adv = (uint64_t)(ks * 2u);           // 8 tf32 = 32 bytes, in 16-byte units
                    umma_tf32(tmem, a_lo + adv, b_hi + adv, UMMA_IDESC, (kb | ks) ? 1u : 0u);
                    umma_tf32(tmem, a_hi + adv, b_lo + adv, UMMA_IDESC, 1u);
                    umma_tf32(tmem, a_hi + adv, b_hi + adv, UMMA_IDESC, 1u);
                }
                umma_commit(smem_u32(&S.empty[s]));                      // stage free once these MMAs retire
            }
            if (ok) umma_commit(smem_u32(&S.accum));
        }
        __syncwarp();
    }

    // ---- teardown ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && S.abort_flag) atomicOr(G.status, ERR_GEMM_TIMEOUT);
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ CTA-pair kernel (cta_group::2)
// Two CTAs of a cluster compute one 256 x (2 * n_half) tile of C together: CTA r of the pair
// gathers rows [128 r, 128 r + 128) of the A tile and rows [n_half r, n_half r + n_half) of the
// B tile into its own shared memory, and one thread of the pair's first CTA issues
// tcgen05.mma.cta_group::2, which reads both CTAs' tiles and accumulates 128 rows x (2 n_half)
// columns into each CTA's tensor memory.  Per flop this halves what every SM pulls from L2 and
// what the MMAs read from shared memory, the two limits of the single-CTA kernel at large sizes.
// Barriers: the "stage full" barriers live in the first CTA and collect one arrival per producer
// warp of both CTAs (remote arrivals through the cluster shared window); "stage empty" and
// "accumulator ready" live in each CTA and are signalled by a commit per CTA.  All waits are
// bounded; both CTAs always reach the closing cluster barrier.
constexpr int TMEM_COLS2 = 256;
struct GemmShared2 {
    long long am[BM], bn[128], cm[BM], cn[256];
    unsigned long long full[STAGES], empty[STAGES], accum;
    uint32_t tmem_base;
    int abort_flag;
};
constexpr size_t GEMM2_SMEM = (size_t)TILE_AREA + sizeof(GemmShared2) + 1024;

__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((it & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void umma2_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma2_commit(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1) k_gemm_pair_3xtf32(const __grid_constant__ GemmDesc G) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *tiles = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    GemmShared2 &S = *reinterpret_cast<GemmShared2 *>(tiles + (size_t)TILE_AREA);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank();                                  // 0 = the CTA that issues the MMAs
    const uint32_t n_half = G.n_half, n_tile = 2u * n_half;
    const uint32_t pm = (G.M + 255u) / 256u;
    const uint32_t pair = blockIdx.x >> 1;
    const uint32_t m0 = (pair % pm) * 256u + rank * 128u;                  // first A / C row of this CTA
    const uint32_t n0 = (pair / pm) * n_tile;                              // first C column of the pair
    const uint32_t nb0 = n0 + rank * n_half;                               // first B row this CTA loads
    const uint32_t nkb_all = (G.K + BK - 1) / BK;
    const uint32_t kb_lo = blockIdx.z * G.kb_chunk;
    const uint32_t nkb = nkb_all - kb_lo < G.kb_chunk ? nkb_all - kb_lo : G.kb_chunk;
    volatile int *abort_flag = &S.abort_flag;

    // ---- setup ----
    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(smem_u32(&S.full[s]), 2 * PROD_WARPS); mbar_init(smem_u32(&S.empty[s]), 1); }
        mbar_init(smem_u32(&S.accum), 1);
        S.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&S.tmem_base)), "r"(TMEM_COLS2) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    if (tid < 128) {
        long long oa = 0, oc = 0;
        if (m0 + tid < G.M) decode_group(G.md, G.nm, m0 + tid, false, oa, oc);
        if (G.partial) oc = ((long long)blockIdx.z * G.M + (m0 + tid)) * G.N;
        S.am[tid] = oa; S.cm[tid] = oc;
    } else if (tid < 256) {
        const uint32_t j = tid - 128;
        long long ob = 0, oc = 0;
        if (j < n_half && nb0 + j < G.N) decode_group(G.nd, G.nn, nb0 + j, true, ob, oc);
        S.bn[j] = ob;
    } else if (tid < 512) {
        const uint32_t j = tid - 256;
        long long ob = 0, oc = 0;
        if (j < n_tile && n0 + j < G.N) decode_group(G.nd, G.nn, n0 + j, true, ob, oc);
        if (G.partial) oc = n0 + j;
        S.cn[j] = oc;
    }
    float *const Cout = G.partial ? G.partial : G.C;
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();                                                    // both CTAs' barriers and tables are ready
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = S.tmem_base;
    const uint32_t tiles_s = smem_u32(tiles);
    const uint32_t rows_a = m0 >= G.M ? 0u : (G.M - m0 < 128u ? G.M - m0 : 128u);
    const uint32_t rows_b = nb0 >= G.N ? 0u : (G.N - nb0 < n_half ? G.N - nb0 : n_half);
    const uint32_t cols_c = n0 >= G.N ? 0u : (G.N - n0 < n_tile ? G.N - n0 : n_tile);

    if (warp < MMA_WARP) {
        // ================= producers (both CTAs) =================
        const uint32_t t = tid;
        bool ok = true;
        UnitSet UA, UB;
        make_units(UA, G.A, G.a_off, S.am, rows_a, G.a_kfast, t);
        make_units(UB, G.B, G.b_off, S.bn, rows_b, G.b_kfast, t);
        auto issue = [&](uint32_t kb) {
            const uint32_t st = tiles_s + (kb % STAGES) * STAGE_BYTES, k0 = (kb_lo + kb) * BK;
            issue_tile(UA, G.A, G.ka, G.a_klin, k0, G.K, G.a_kvec, st);
            issue_tile(UB, G.B, G.kb, G.b_klin, k0, G.K, G.b_kvec, st + TILE_BYTES);
        };
        for (uint32_t kb = 0; kb < (uint32_t)LOOKAHEAD; kb++) {
            if (kb < nkb) issue(kb);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        for (uint32_t kb = 0; kb < nkb && ok; kb++) {
            asm volatile("cp.async.wait_group %0;" ::"n"(LOOKAHEAD - 1) : "memory");
            if (kb >= (uint32_t)LO_STAGES) {
                const uint32_t prev = kb - LO_STAGES;
                ok = mbar_wait(smem_u32(&S.empty[prev % STAGES]), (prev / STAGES) & 1u, abort_flag);
                if (!ok) break;
            }
            const uint32_t st = tiles_s + (kb % STAGES) * STAGE_BYTES, lo = tiles_s + LO_BASE + (kb % LO_STAGES) * STAGE_BYTES;
            split_tile(UA, st, lo);
            split_tile(UB, st + TILE_BYTES, lo + TILE_BYTES);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&S.full[kb % STAGES]), 0));   // one arrival per warp, on the first CTA's barrier
            const uint32_t nxt = kb + LOOKAHEAD;
            if (nxt < nkb) {
                const uint32_t use = nxt / STAGES;
                if (use >= 1) ok = mbar_wait(smem_u32(&S.empty[nxt % STAGES]), (use - 1) & 1u, abort_flag);
                if (ok) issue(nxt);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        // ================= epilogue: this CTA's 128 rows x cols_c columns =================
        if (ok) ok = mbar_wait(smem_u32(&S.accum), 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            constexpr int COLS_PER_WARP = 256 / (PROD_WARPS / 4);
            const uint32_t q = warp & 3u, part = warp >> 2;
            const uint32_t row = q * 32u + lane;
            const bool row_ok = row < rows_a;
            const long long crow = S.cm[row];
#pragma unroll
            for (int c = 0; c < COLS_PER_WARP / 32; c++) {
                const uint32_t col0 = part * (uint32_t)COLS_PER_WARP + (uint32_t)c * 32u;
                if (col0 >= cols_c) continue;                              // warp-uniform
                uint32_t r[32];
                const uint32_t taddr = tmem + ((q * 32u) << 16) + col0;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                             "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                             "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                               "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                               "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                               "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                             : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row_ok) {
                    if (G.c_nvec && col0 + 32u <= cols_c) {
                        float4 *dst = reinterpret_cast<float4 *>(Cout + crow + S.cn[col0]);
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                 __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (col0 + j < cols_c) Cout[crow + S.cn[col0 + j]] = __uint_as_float(r[j]);
                    }
                }
            }
        }
    } else if (rank == 0) {
        // ================= MMA issuer: one lane of the first CTA, for the pair =================
        if (lane == 0) {
            // D f32, A/B tf32, both K-major, M = 256 over the pair, N = n_tile
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((n_tile >> 3) << 17) | ((256u >> 4) << 24);
            bool ok = true;
            for (uint32_t kb = 0; kb < nkb && ok; kb++) {
                const uint32_t s = kb % STAGES, use = kb / STAGES;
                ok = mbar_wait_cluster(smem_u32(&S.full[s]), use & 1u, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t st = tiles_s + s * STAGE_BYTES, lo = tiles_s + LO_BASE + (kb % LO_STAGES) * STAGE_BYTES;
                const uint64_t a_hi = umma_desc(st), b_hi = umma_desc(st + TILE_BYTES);
                const uint64_t a_lo = umma_desc(lo), b_lo = umma_desc(lo + TILE_BYTES);
#pragma unroll
                for (uint32_t ks = 0; ks < (uint32_t)(BK / 8); ks++) {
                    const uint64_t adv = (uint64_t)(ks * 2u);
                    umma2_tf32(tmem, a_lo + adv, b_hi + adv, idesc, (kb | ks) ? 1u : 0u);
                    umma2_tf32(tmem, a_hi + adv, b_lo + adv, idesc, 1u);
                    umma2_tf32(tmem, a_hi + adv, b_hi + adv, idesc, 1u);
                }
                umma2_commit(map_to_cta(smem_u32(&S.empty[s]), 0));       // the stage is free in both CTAs once these MMAs retire
                umma2_commit(map_to_cta(smem_u32(&S.empty[s]), 1));
            }
            if (ok) {
                umma2_commit(map_to_cta(smem_u32(&S.accum), 0));
                umma2_commit(map_to_cta(smem_u32(&S.accum), 1));
            }
        }
        __syncwarp();
    }

    // ---- teardown: nobody leaves while the other CTA may still signal it or read its tiles ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();
    if (tid == 0 && S.abort_flag) atomicOr(G.status, ERR_GEMM_TIMEOUT);
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS2) : "memory");
    }
}

}  // namespace thc

#include "gemm_skinny.inc"
#include "gemm_tma.inc"
#include "gemm_ta.inc"
#include "gemm_ps.inc"
#include "gemm_host.inc"
