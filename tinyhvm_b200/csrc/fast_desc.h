// fast_desc.h — parameters of the specialised (f32, single-view) kernel
// families.  A dispatch qualifies after its iteration space has been collapsed:
// size-1 dims dropped and neighbouring dims merged whenever every leaf walks
// them as one dense run, which turns e.g. [B,C,H,W] with a [1,C,1,1] leaf into
// [B, C, H*W] and a fully contiguous chain into a single flat dim.
#pragma once
#include <stdint.h>

namespace thc {

constexpr int FR = 6;    // max collapsed rank
constexpr int FL = 8;    // max leaves
constexpr int FO = 24;   // max ops

struct FLeaf {
    const float *ptr;            // filled per launch
    long long    off;            // element offset (may be negative: PAD)
    int          stride[FR];     // elements per step of each collapsed dim
    unsigned     mlo[FR], mhi[FR];   // valid coordinate range [mlo, mhi) where masked
    unsigned     masked;         // bit d set: dim d carries a partial mask
    unsigned     vec;            // 1: 16-byte loads along the innermost dim are legal
    unsigned     mode;           // 0: strided (general), 1: flat (off + row-major position), 2: one element
};

struct FProg {
    unsigned      n_leaves, n_ops;
    unsigned char uop[FO], a[FO], b[FO], aux[FO];
};

struct FDesc {
    unsigned rank;
    unsigned dims[FR];
    unsigned char is_red[FR];
    unsigned n_k, kd[FR];        // kept collapsed dims, outermost first
    unsigned n_r, rd[FR];        // reduced collapsed dims, outermost first
    unsigned long long numel, n_out, n_red;
    unsigned rtype;              // 0, THC_SUM, THC_RMAX
    unsigned vec;                // elements per thread along the innermost dim (1 or 4)
    unsigned split;              // CTAs sharing one output (two-pass reduce), >= 1
    unsigned chain;              // index into the static chain registry, or 0 = interpreted
    unsigned long long fstride[FR];  // row-major strides of the collapsed dims (flat position of a coordinate)
    unsigned long long omul[FR], smul[FR];   // row kernels: contribution of an outer coordinate to the output index / to the partial-sum slot
    unsigned row_split;              // row kernels: partial sums per output (product of the reduced outer dims), >= 1
    FLeaf    leaf[FL];
    FProg    prog;
};

}  // namespace thc
