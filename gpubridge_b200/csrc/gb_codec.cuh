// Device-side codec of the compressed bridge leg: bf16 and block-scaled fp8-e4m3.
//
// Bit-compatible with the PyTorch oracle in gpubridge_b200/compression.py: values are
// prepared (plus residual, saturated to the finite float32 range, |v| < 2^-100 flushed),
// quantised with round-to-nearest-even and saturation, and the residual is what the code
// leaves out.  fp8 uses the hardware conversion cvt.rn.satfinite.e4m3x2.f32; every float
// operation that must not be contracted into an FMA is written with an explicit intrinsic.
//   format REF : 256 values per block, scale 2^k (smallest with amax/2^k <= 448, k <= 119)
//   format B200: 128 values per block, scale amax/448 (fp32), values multiplied by 448/amax
#pragma once
#include <cuda_fp8.h>
#include "gb_common.cuh"

#define GB_TINY 7.888609052210118e-31f      /* 2^-100 */
#define GB_FLT_MAX 3.4028234663852886e+38f

enum GbCodec { GB_RAW = 0, GB_C_BF16 = 1, GB_C_FP8_REF = 2, GB_C_FP8_B200 = 3 };

template <int CODEC> struct GbBlock { static const int size = 256; };
template <> struct GbBlock<GB_C_FP8_B200> { static const int size = 128; };

// x (+ residual) as float32, saturated and flushed; `finite` says whether it may be encoded.
__device__ __forceinline__ float gb_prepare(float x, bool x_finite, float residual, bool& finite) {
    float v = x;
    if (x_finite) v = fminf(fmaxf(v, -GB_FLT_MAX), GB_FLT_MAX);
    v = __fadd_rn(v, residual);
    if (x_finite) v = fminf(fmaxf(v, -GB_FLT_MAX), GB_FLT_MAX);
    finite = x_finite && !(v != v);
    if (finite && fabsf(v) < GB_TINY) v = 0.0f;
    return v;
}

__device__ __forceinline__ unsigned gb_bf16_bits(float v) {
    unsigned bits = __float_as_uint(v);
    unsigned r = ((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16) & 0xFFFFu;
    return (v != v) ? 0x7FC0u : r;
}
// bf16-mode code: a finite value that would round to +-inf keeps the largest finite bfloat16.
__device__ __forceinline__ unsigned gb_bf16_code(float v, bool finite) {
    unsigned c = gb_bf16_bits(v);
    if (finite && (c & 0x7FFFu) == 0x7F80u) c -= 1u;
    return c;
}
__device__ __forceinline__ float gb_from_bf16_bits(unsigned c) { return __uint_as_float(c << 16); }

__device__ __forceinline__ float gb_e4m3_decode(unsigned code) {
    if ((code & 0x7Fu) == 0x7Fu) return __uint_as_float(0x7FC00000u);
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)code, __NV_E4M3);
    return __half2float(__half(h));
}
__device__ __forceinline__ unsigned gb_e4m3_encode(float q) {
    if (q == 0.0f) return 0u;                       // either zero encodes as +0
    return (unsigned)__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3);
}

// Two codes at once (the hardware converts e4m3 in pairs): the low byte of `pair` first.
__device__ __forceinline__ float2 gb_e4m3_decode2(unsigned pair) {
    __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(pair & 0xFFFFu), __NV_E4M3);
    float2 f = __half22float2(__half2(h));
    if ((pair & 0x7Fu) == 0x7Fu) f.x = __uint_as_float(0x7FC00000u);
    if ((pair & 0x7F00u) == 0x7F00u) f.y = __uint_as_float(0x7FC00000u);
    return f;
}
// Two values to two codes (low byte = a); a zero of either sign encodes as +0.
__device__ __forceinline__ unsigned gb_e4m3_encode2(float a, float b) {
    a = a == 0.0f ? 0.0f : a;
    b = b == 0.0f ? 0.0f : b;
    return (unsigned)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
}

// Scale of one block from its largest magnitude: (stored scale, multiplier).
template <int CODEC>
__device__ __forceinline__ void gb_block_scale(float amax, float& scale, float& mult) {
    if (CODEC == GB_C_FP8_REF) {
        int k = 0;
        if (amax != 0.0f) {
            unsigned bits = __float_as_uint(amax);
            k = (int)((bits >> 23) & 0xFFu) - 135 + (((bits & 0x7FFFFFu) > 0x600000u) ? 1 : 0);
            if (k > 119) k = 119;
        }
        scale = __uint_as_float((unsigned)(k + 127) << 23);
        mult = __uint_as_float((unsigned)(127 - k) << 23);
    } else {
        if (amax == 0.0f) { scale = 1.0f; mult = 1.0f; }
        else { scale = __fdiv_rn(amax, 448.0f); mult = __fdiv_rn(448.0f, amax); }
    }
}

__device__ __forceinline__ float gb_warp_max(float v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float gb_flush(float v) { return fabsf(v) < GB_TINY ? 0.0f : v; }
