// gemm_desc.h — a SUM(MUL(a, b)) dispatch recognised as a contraction
//     C[m, n] = sum_k A[m, k] * B[k, n]
// where m, n and k are mixed-radix indices over groups of iteration dims:
// k = the reduced dims, m = kept dims that only leaf A walks, n = kept dims that
// only leaf B walks.  Every operand address is separable,
//     addr_A(m, k) = a_off + am(m) + ak(k),   addr_B(k, n) = b_off + bn(n) + bk(k),
//     addr_C(m, n) = cm(m) + cn(n),
// which covers plain and transposed matmul, convolution forward (implicit
// im2col: m = (b, oh, ow), k = (ci, kh, kw)), weight gradient and input
// gradient as the reference's scheduler emits them (MUL + SUM over expanded
// and pooled views).
#pragma once
#include <stdint.h>

namespace thc {

constexpr int GS = 4;   // max sub-dims per index group

struct GSub {
    uint32_t  size;
    long long sa, sb, sc;   // element stride of this sub-dim in A, B and C (0 where unused)
};

struct GemmDesc {
    uint32_t M, N, K;
    uint32_t nm, nn, nk;
    GSub md[GS], nd[GS], kd[GS];       // outermost first
    long long a_off, b_off;
    const int32_t *ka, *kb;            // per-k element offsets (device tables, K rounded up to 32 entries)
    uint32_t a_kfast, a_kvec;          // A tile: threads run along k (else along m); 16-byte loads along k legal
    uint32_t b_kfast, b_kvec;
    long long a_klin, b_klin;          // non-zero: the operand's k offset is k * klin (one reduced dim, no table lookup)
    uint32_t c_nvec;                   // C: n is contiguous and 16-byte aligned per row
    uint32_t kb_chunk;                 // k-blocks (of 32) per split; gridDim.z splits share one output tile
    uint32_t n_half;                   // CTA-pair kernel: B rows (output columns) each CTA of a pair loads: 128, 64 or 32
    float *partial;                    // split-K: dense [split][M][N] partial sums (library scratch), else null
    const float *A, *B;                // filled per launch
    float *C;
    int *status;
};

}  // namespace thc
