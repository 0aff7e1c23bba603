// Stand-alone codec kernels: quantise a tensor into the bridge payload layout and
// dequantise-accumulate the members' payloads.  They replace the reference's four Triton
// kernels (src/gpubridge/_compression_kernels.py:116-176) and produce the same bits as the
// PyTorch oracle.  Payload: fp8 = fp32 scales, then one code byte per value, padded to 4
// bytes with zeros; bf16 = one 16-bit code per value, padded to 4 bytes.
//
// quantise (fp8): one warp per block of 256 (128) values, each lane 8 (4) consecutive values
// loaded as 16-byte vectors; the block maximum is a warp shuffle reduction; codes leave as
// 4-byte words.  Memory traffic per value: read x (+ read/write the fp32 residual), write
// one byte - the kernel is bound by HBM bandwidth.
#include "gb_codec.cuh"

namespace {

template <typename T> __device__ __forceinline__ float to_float(T v, bool& finite);
template <> __device__ __forceinline__ float to_float<float>(float v, bool& f) {
    f = isfinite(v); return v;
}
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v, bool& f) {
    float x = __bfloat162float(v); f = isfinite(x); return x;
}
template <> __device__ __forceinline__ float to_float<__half>(__half v, bool& f) {
    float x = __half2float(v); f = isfinite(x); return x;
}
template <> __device__ __forceinline__ float to_float<double>(double v, bool& f) {
    f = isfinite(v);
    if (!f) return (float)v;
    double c = fmin(fmax(v, -(double)GB_FLT_MAX), (double)GB_FLT_MAX);
    return __double2float_rn(c);
}

template <typename T> __device__ __forceinline__ void from_float(T* p, float v);
template <> __device__ __forceinline__ void from_float<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void from_float<__nv_bfloat16>(__nv_bfloat16* p, float v) {
    *reinterpret_cast<unsigned short*>(p) = (unsigned short)gb_bf16_bits(v);
}
template <> __device__ __forceinline__ void from_float<__half>(__half* p, float v) {
    *p = __float2half_rn(v);
}
template <> __device__ __forceinline__ void from_float<double>(double* p, float v) { *p = (double)v; }

// Load EPL consecutive values starting at x[i0]; values at or past n read as 0 (finite).
template <typename T, int EPL>
__device__ __forceinline__ void load_run(const T* x, size_t i0, size_t n, float (&v)[EPL],
                                         bool (&fin)[EPL]) {
    const bool whole = i0 + EPL <= n;
    const bool aligned = ((uintptr_t)(x + i0) & 15u) == 0;
    if (whole && aligned && sizeof(T) * EPL >= 16) {
        constexpr int VEC = 16 / sizeof(T);
        #pragma unroll
        for (int g = 0; g < EPL / VEC; ++g) {
            union { uint4 u; T e[VEC]; } w;
            w.u = __ldg(reinterpret_cast<const uint4*>(x + i0) + g);
            #pragma unroll
            for (int j = 0; j < VEC; ++j) v[g * VEC + j] = to_float<T>(w.e[j], fin[g * VEC + j]);
        }
    } else {
        #pragma unroll
        for (int j = 0; j < EPL; ++j) {
            if (i0 + j < n) v[j] = to_float<T>(x[i0 + j], fin[j]);
            else { v[j] = 0.0f; fin[j] = true; }
        }
    }
}

template <typename T, int CODEC>
__global__ void __launch_bounds__(256)
quantize_fp8_kernel(const T* __restrict__ x, float* __restrict__ residual,
                    unsigned char* __restrict__ payload, size_t n) {
    constexpr int BS = GbBlock<CODEC>::size;
    constexpr int EPL = BS / 32;
    const size_t nb = (n + BS - 1) / BS;
    const size_t n4 = (n + 3) & ~(size_t)3;
    float* scales = reinterpret_cast<float*>(payload);
    unsigned char* codes = payload + 4 * nb;
    const int lane = threadIdx.x & 31;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t blk = warp; blk < nb; blk += nwarps) {
        const size_t i0 = blk * BS + (size_t)lane * EPL;
        float v[EPL]; bool fin[EPL];
        load_run<T, EPL>(x, i0, n, v, fin);
        // residual: 16-byte vectors for whole, aligned runs (always the case away from the tail)
        float r[EPL];
        const bool rvec = residual != nullptr && i0 + EPL <= n &&
                          ((uintptr_t)(residual + i0) & 15u) == 0;
        if (rvec) {
            #pragma unroll
            for (int g = 0; g < EPL / 4; ++g) {
                float4 q = *(reinterpret_cast<const float4*>(residual + i0) + g);
                r[4 * g] = q.x; r[4 * g + 1] = q.y; r[4 * g + 2] = q.z; r[4 * g + 3] = q.w;
            }
        } else {
            #pragma unroll
            for (int j = 0; j < EPL; ++j)
                r[j] = (residual != nullptr && i0 + j < n) ? residual[i0 + j] : 0.0f;
        }
        float amax = 0.0f;
        #pragma unroll
        for (int j = 0; j < EPL; ++j) {
            bool f;
            v[j] = gb_prepare(v[j], fin[j], r[j], f);
            fin[j] = f;
            if (f) amax = fmaxf(amax, fabsf(v[j]));
        }
        amax = gb_warp_max(amax);
        float scale, mult;
        gb_block_scale<CODEC>(amax, scale, mult);
        if (lane == 0) scales[blk] = scale;
        unsigned words[EPL / 4];
        #pragma unroll
        for (int w = 0; w < EPL / 4; ++w) words[w] = 0u;
        #pragma unroll
        for (int j = 0; j < EPL; j += 2) {                  // the hardware converts in pairs
            unsigned pair = gb_e4m3_encode2(__fmul_rn(v[j], mult), __fmul_rn(v[j + 1], mult));
            if (!fin[j]) pair = (pair & 0xFF00u) | 0x7Fu;
            if (!fin[j + 1]) pair = (pair & 0x00FFu) | 0x7F00u;
            if (i0 + j >= n) pair &= 0xFF00u;
            if (i0 + j + 1 >= n) pair &= 0x00FFu;
            const float2 sent = gb_e4m3_decode2(pair);
            if (i0 + j < n) r[j] = fin[j] ? __fsub_rn(v[j], __fmul_rn(sent.x, scale)) : 0.0f;
            if (i0 + j + 1 < n) r[j + 1] = fin[j + 1] ? __fsub_rn(v[j + 1], __fmul_rn(sent.y, scale)) : 0.0f;
            words[j / 4] |= pair << (8 * (j & 3));
        }
        if (rvec) {
            #pragma unroll
            for (int g = 0; g < EPL / 4; ++g)
                *(reinterpret_cast<float4*>(residual + i0) + g) =
                    make_float4(r[4 * g], r[4 * g + 1], r[4 * g + 2], r[4 * g + 3]);
        } else if (residual != nullptr) {
            #pragma unroll
            for (int j = 0; j < EPL; ++j)
                if (i0 + j < n) residual[i0 + j] = r[j];
        }
        #pragma unroll
        for (int w = 0; w < EPL / 4; ++w)
            if (i0 + 4 * w < n4) *reinterpret_cast<unsigned*>(codes + i0 + 4 * w) = words[w];
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
quantize_bf16_kernel(const T* __restrict__ x, float* __restrict__ residual,
                     unsigned char* __restrict__ payload, size_t n) {
    // two values (one 4-byte word of codes) per thread per step
    const size_t npairs = (n + 1) / 2;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nth = (size_t)gridDim.x * blockDim.x;
    for (size_t p = tid; p < npairs; p += nth) {
        unsigned word = 0u;
        #pragma unroll
        for (int j = 0; j < 2; ++j) {
            const size_t i = 2 * p + j;
            if (i >= n) continue;
            bool xf, f;
            float xv = to_float<T>(x[i], xf);
            float r = residual != nullptr ? residual[i] : 0.0f;
            float v = gb_prepare(xv, xf, r, f);
            unsigned code = gb_bf16_code(v, f);
            if (residual != nullptr)
                residual[i] = f ? __fsub_rn(v, gb_from_bf16_bits(code)) : 0.0f;
            word |= code << (16 * j);
        }
        *reinterpret_cast<unsigned*>(payload + 4 * p) = word;
    }
}

// Sixteen results as vector stores (whole, aligned runs) or one by one (the tail).
template <typename T>
__device__ __forceinline__ void store_run16(T* out, size_t i0, size_t n, const float (&acc)[16]) {
    const bool whole = i0 + 16 <= n;
    if (whole && ((uintptr_t)(out + i0) & 15u) == 0 && sizeof(T) <= 4) {
        if (sizeof(T) == 4) {
            #pragma unroll
            for (int g = 0; g < 4; ++g)
                *(reinterpret_cast<float4*>(out + i0) + g) =
                    make_float4(acc[4 * g], acc[4 * g + 1], acc[4 * g + 2], acc[4 * g + 3]);
        } else {
            union { uint4 u[2]; T e[16]; } w;
            #pragma unroll
            for (int j = 0; j < 16; ++j) from_float<T>(&w.e[j], acc[j]);
            *(reinterpret_cast<uint4*>(out + i0)) = w.u[0];
            *(reinterpret_cast<uint4*>(out + i0) + 1) = w.u[1];
        }
        return;
    }
    #pragma unroll
    for (int j = 0; j < 16; ++j)
        if (i0 + j < n) from_float<T>(out + i0 + j, acc[j]);
}

// Sixteen consecutive values per thread and step: a block's scale is read once per member,
// codes arrive as four 4-byte words (rows are only 4-byte aligned) that are all in flight at
// once, pairs of codes are decoded by one hardware conversion, and results leave as 16-byte
// vectors.  Members are added one after the other, each sum flushed, as the oracle does.
template <typename T, int CODEC>
__global__ void __launch_bounds__(256)
dequantize_kernel(const unsigned char* __restrict__ payloads, size_t row_bytes, int members,
                  T* __restrict__ out, size_t n) {
    constexpr int BS = GbBlock<CODEC>::size;
    const size_t nb = (n + BS - 1) / BS;
    const size_t n4 = (n + 3) & ~(size_t)3;                  // code bytes present in a row (padded)
    const size_t ngroups = (n + 15) / 16;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nth = (size_t)gridDim.x * blockDim.x;
    for (size_t g = tid; g < ngroups; g += nth) {
        const size_t i0 = 16 * g;
        float acc[16];
        #pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
        for (int m = 0; m < members; ++m) {
            const unsigned char* row = payloads + (size_t)m * row_bytes;
            if (CODEC == GB_C_BF16) {
                // 16-bit codes: eight 4-byte words; the row holds (n + 1) / 2 of them
                const size_t words = (n + 1) / 2;
                unsigned w[8];
                #pragma unroll
                for (int q = 0; q < 8; ++q)
                    w[q] = (i0 / 2 + q < words) ? __ldg(reinterpret_cast<const unsigned*>(row) + i0 / 2 + q) : 0u;
                #pragma unroll
                for (int q = 0; q < 8; ++q) {
                    acc[2 * q] = gb_flush(__fadd_rn(acc[2 * q], gb_from_bf16_bits(w[q] & 0xFFFFu)));
                    acc[2 * q + 1] = gb_flush(__fadd_rn(acc[2 * q + 1], gb_from_bf16_bits(w[q] >> 16)));
                }
            } else {
                const float scale = __ldg(reinterpret_cast<const float*>(row) + i0 / BS);
                const unsigned* codes = reinterpret_cast<const unsigned*>(row + 4 * nb + i0);
                unsigned w[4];
                #pragma unroll
                for (int q = 0; q < 4; ++q) w[q] = (i0 + 4 * q < n4) ? __ldg(codes + q) : 0u;
                #pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 lo = gb_e4m3_decode2(w[q] & 0xFFFFu), hi = gb_e4m3_decode2(w[q] >> 16);
                    acc[4 * q] = gb_flush(__fadd_rn(acc[4 * q], __fmul_rn(lo.x, scale)));
                    acc[4 * q + 1] = gb_flush(__fadd_rn(acc[4 * q + 1], __fmul_rn(lo.y, scale)));
                    acc[4 * q + 2] = gb_flush(__fadd_rn(acc[4 * q + 2], __fmul_rn(hi.x, scale)));
                    acc[4 * q + 3] = gb_flush(__fadd_rn(acc[4 * q + 3], __fmul_rn(hi.y, scale)));
                }
            }
        }
        store_run16<T>(out, i0, n, acc);
    }
}

inline int grid_for(size_t work_items, int per_block) {
    size_t blocks = (work_items + per_block - 1) / per_block;
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 8) blocks = 148 * 8;
    return (int)blocks;
}

template <typename T>
cudaError_t quantize_t(int mode, int fmt, const void* x, float* residual, unsigned char* payload,
                       size_t n, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    const T* xp = static_cast<const T*>(x);
    if (mode == 0) {
        quantize_bf16_kernel<T><<<grid_for((n + 1) / 2, 256 * 4), 256, 0, stream>>>(
            xp, residual, payload, n);
    } else if (fmt == 0) {
        quantize_fp8_kernel<T, GB_C_FP8_REF><<<grid_for((n + 255) / 256, 8), 256, 0, stream>>>(
            xp, residual, payload, n);
    } else {
        quantize_fp8_kernel<T, GB_C_FP8_B200><<<grid_for((n + 127) / 128, 8), 256, 0, stream>>>(
            xp, residual, payload, n);
    }
    return cudaGetLastError();
}

template <typename T>
cudaError_t dequantize_t(int mode, int fmt, const unsigned char* payloads, size_t row_bytes,
                         int members, void* out, size_t n, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    T* op = static_cast<T*>(out);
    const int grid = grid_for((n + 15) / 16, 256);
    if (mode == 0)
        dequantize_kernel<T, GB_C_BF16><<<grid, 256, 0, stream>>>(payloads, row_bytes, members, op, n);
    else if (fmt == 0)
        dequantize_kernel<T, GB_C_FP8_REF><<<grid, 256, 0, stream>>>(payloads, row_bytes, members, op, n);
    else
        dequantize_kernel<T, GB_C_FP8_B200><<<grid, 256, 0, stream>>>(payloads, row_bytes, members, op, n);
    return cudaGetLastError();
}

}  // namespace

// mode: 0 bf16, 1 fp8.  fmt: 0 ref (256 / power of two), 1 b200 (128 / amax over 448).
// dtype: GbDtype of x / out (float32, bfloat16, float16, float64).  Returns a cudaError_t.
extern "C" int gb_codec_quantize(int mode, int fmt, int dtype, const void* x, float* residual,
                                 unsigned char* payload, size_t n, cudaStream_t stream) {
    switch (dtype) {
        case GB_F32: return quantize_t<float>(mode, fmt, x, residual, payload, n, stream);
        case GB_BF16: return quantize_t<__nv_bfloat16>(mode, fmt, x, residual, payload, n, stream);
        case GB_F16: return quantize_t<__half>(mode, fmt, x, residual, payload, n, stream);
        case GB_F64: return quantize_t<double>(mode, fmt, x, residual, payload, n, stream);
    }
    return cudaErrorInvalidValue;
}

extern "C" int gb_codec_dequantize(int mode, int fmt, int dtype, const unsigned char* payloads,
                                   size_t row_bytes, int members, void* out, size_t n,
                                   cudaStream_t stream) {
    switch (dtype) {
        case GB_F32: return dequantize_t<float>(mode, fmt, payloads, row_bytes, members, out, n, stream);
        case GB_BF16: return dequantize_t<__nv_bfloat16>(mode, fmt, payloads, row_bytes, members, out, n, stream);
        case GB_F16: return dequantize_t<__half>(mode, fmt, payloads, row_bytes, members, out, n, stream);
        case GB_F64: return dequantize_t<double>(mode, fmt, payloads, row_bytes, members, out, n, stream);
    }
    return cudaErrorInvalidValue;
}
