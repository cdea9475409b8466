// device_common.cuh — arithmetic shared by every kernel of the backend:
// dtype conversion on load/store and the scalar UOp semantics.
//
// The semantics follow the reference's CPU backend so results can be compared
// value for value:
//   * ALU ops:            src/backend/cpu/dispatch.c:5-21
//   * dtype load/store:   src/tinyhvm.h:488-526
//   * f32 <-> f16 bits:   src/tinyhvm.h:433-486 (round-half-up on the 13 dropped
//                         mantissa bits, NOT IEEE round-to-nearest-even, hence
//                         the hand-written conversion instead of __float2half)
// Multiplies and adds use the non-contracting intrinsics so a fused chain
// MUL,ADD never becomes an FMA (the CPU backend evaluates op by op).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/thvm_cuda.h"

namespace thc {

// ---- f16 bit conversions -------------------------------------------------
__host__ __device__ __forceinline__ uint16_t f32_to_f16_bits(float f) {
#ifdef __CUDA_ARCH__
    uint32_t x = __float_as_uint(f);
#else
    uint32_t x; memcpy(&x, &f, 4);
#endif
    const uint32_t sgn = (x >> 16) & 0x8000u;
    const int32_t  e   = (int32_t)((x >> 23) & 0xFFu) - 112;   // rebias 127 -> 15
    uint32_t m = x & 0x7FFFFFu;
    if (e >= 31)                                   // overflow, inf, nan: any mantissa bit sets the quiet bit,
        return (uint16_t)(sgn | 0x7C00u | (m ? 0x0200u : 0u));   // also for finite overflow, as the reference does
    if (e <= 0) {                                  // subnormal half or zero
        if (e < -10) return (uint16_t)sgn;
        m = (m | 0x800000u) >> (1 - e);
        if (m & 0x1000u) m += 0x2000u;
        return (uint16_t)(sgn | (m >> 13));
    }
    int32_t ee = e;
    if (m & 0x1000u) {
        m += 0x2000u;
        if (m & 0x800000u) { m = 0; ee += 1; if (ee >= 31) return (uint16_t)(sgn | 0x7C00u); }
    }
    return (uint16_t)(sgn | ((uint32_t)ee << 10) | (m >> 13));
}

__host__ __device__ __forceinline__ float f16_bits_to_f32(uint16_t h) {
    const uint32_t sgn = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = ((uint32_t)h >> 10) & 0x1Fu;
    uint32_t m = (uint32_t)h & 0x3FFu;
    uint32_t bits;
    if (e == 0x1Fu)      bits = sgn | 0x7F800000u | (m << 13);
    else if (e != 0)     bits = sgn | ((e + 112u) << 23) | (m << 13);
    else if (m == 0)     bits = sgn;
    else {                                          // normalise a subnormal half
        e = 1;
        while (!(m & 0x400u)) { m <<= 1; e -= 1; }
        bits = sgn | ((e + 112u) << 23) | ((m & 0x3FFu) << 13);
    }
#ifdef __CUDA_ARCH__
    return __uint_as_float(bits);
#else
    float out; memcpy(&out, &bits, 4); return out;
#endif
}

// ---- C casts as x86-64 performs them (cvttss2si) ---------------------------
// (i32)f: out-of-range and NaN give INT_MIN.  (u32)f goes through a 64-bit
// signed conversion and keeps the low word, so small negatives wrap.
__host__ __device__ __forceinline__ int32_t cast_i32(float v) {
    if (!(v > -2147483904.0f && v < 2147483648.0f)) return (int32_t)0x80000000u;
    return (int32_t)v;
}
__host__ __device__ __forceinline__ uint32_t cast_u32(float v) {
    if (!(v > -9223373136366403584.0f && v < 9223372036854775808.0f)) return 0u;
    return (uint32_t)(uint64_t)(long long)v;
}

__host__ __device__ __forceinline__ uint32_t dtype_bytes(uint32_t dt) { return dt == THC_F16 ? 2u : 4u; }

__device__ __forceinline__ float load_as_f32(const void *base, uint32_t dt, uint64_t i) {
    switch (dt) {
        case THC_F32: return ((const float *)base)[i];
        case THC_F16: return f16_bits_to_f32(((const uint16_t *)base)[i]);
        case THC_I32: return (float)((const int32_t *)base)[i];
        case THC_U32: return (float)((const uint32_t *)base)[i];
        default:      return 0.0f;
    }
}
__device__ __forceinline__ void store_from_f32(void *base, uint32_t dt, uint64_t i, float v) {
    switch (dt) {
        case THC_F32: ((float *)base)[i] = v; break;
        case THC_F16: ((uint16_t *)base)[i] = f32_to_f16_bits(v); break;
        case THC_I32: ((int32_t *)base)[i] = cast_i32(v); break;
        case THC_U32: ((uint32_t *)base)[i] = cast_u32(v); break;
        default: break;
    }
}
// value -> stored dtype -> value, i.e. what a store followed by a load yields
__host__ __device__ __forceinline__ float roundtrip(float v, uint32_t dt) {
    switch (dt) {
        case THC_F16: return f16_bits_to_f32(f32_to_f16_bits(v));
        case THC_I32: return (float)cast_i32(v);
        case THC_U32: return (float)cast_u32(v);
        default:      return v;
    }
}

// A stored element as raw bits (what memory holds after a store) and back.
// u32/i32 -> f32 is not injective above 2^24, so an accumulator that lives in
// a non-f32 output buffer has to be carried in this form.
__host__ __device__ __forceinline__ uint32_t encode_bits(float v, uint32_t dt) {
    switch (dt) {
        case THC_F16: return f32_to_f16_bits(v);
        case THC_I32: return (uint32_t)cast_i32(v);
        case THC_U32: return cast_u32(v);
        default: {
#ifdef __CUDA_ARCH__
            return __float_as_uint(v);
#else
            uint32_t b; memcpy(&b, &v, 4); return b;
#endif
        }
    }
}
__host__ __device__ __forceinline__ float decode_bits(uint32_t b, uint32_t dt) {
    switch (dt) {
        case THC_F16: return f16_bits_to_f32((uint16_t)b);
        case THC_I32: return (float)(int32_t)b;
        case THC_U32: return (float)b;
        default: {
#ifdef __CUDA_ARCH__
            return __uint_as_float(b);
#else
            float f; memcpy(&f, &b, 4); return f;
#endif
        }
    }
}
__device__ __forceinline__ void store_bits(void *base, uint32_t dt, uint64_t i, uint32_t b) {
    if (dt == THC_F16) ((uint16_t *)base)[i] = (uint16_t)b;
    else ((uint32_t *)base)[i] = b;
}

// ---- scalar UOp ------------------------------------------------------------
__device__ __forceinline__ float alu(uint32_t uop, uint32_t aux, float a, float b) {
    switch (uop) {
        case THC_ADD:  return __fadd_rn(a, b);
        case THC_MUL:  return __fmul_rn(a, b);
        case THC_SUB:  return __fsub_rn(a, b);
        case THC_DIV:  return b != 0.0f ? __fdiv_rn(a, b) : 0.0f;
        case THC_MAX:  return a > b ? a : b;
        case THC_CMP:  return a > b ? 1.0f : 0.0f;
        case THC_NEG:  return -a;
        case THC_RELU: return a > 0.0f ? a : 0.0f;
        case THC_EXP:  return expf(a);
        case THC_LOG:  return logf(a);
        case THC_SQRT: return __fsqrt_rn(a);
        case THC_CAST: return roundtrip(a, aux);
        default:       return a;
    }
}

// reduce combine, written exactly as the accumulate step of the CPU backend
// (src/backend/cpu/dispatch.c:209-216): acc = v > acc ? v : acc for RMAX.
__device__ __forceinline__ float red_combine(uint32_t rtype, float acc, float v) {
    return rtype == THC_RMAX ? (v > acc ? v : acc) : __fadd_rn(acc, v);
}
__device__ __forceinline__ float red_init(uint32_t rtype) { return rtype == THC_RMAX ? -1e30f : 0.0f; }

// error bits a kernel can raise into the device status word
enum : int { ERR_LOAD_OOB = 1, ERR_STORE_OOB = 2, ERR_BAD_PROGRAM = 4 };

}  // namespace thc
