// Fused LayerNorm, forward and backward, for the transformer benchmarks.
//
// A launch list of one training step of the GPT-2 benchmark (one B200, eager) put 18 % of the
// kernel time into LayerNorm: the stock backward spends 75 us per layer on the gamma / beta
// reduction alone.  Here one warp owns a row: the row stays in registers, the row statistics
// are warp shuffles (no block barrier), the output is written once in the dtype the consumer
// wants (bf16 under autocast, so the cast kernel that would follow disappears), and the
// backward produces dx and per-warp partial sums of dgamma / dbeta in the same pass; a second
// small kernel adds the partials in a fixed order (deterministic, no atomics).
//
// Shapes: x [rows, d] row-major, d a multiple of 128 up to 2048 (EPL = d / 32 values per lane).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace {

constexpr int WARPS = 4;

template <typename T> struct Io;
template <> struct Io<float> {
    static __device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
    static __device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Io<__nv_bfloat16> {
    static __device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
        const uint2 q = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
        const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    static __device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
        uint2 q;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
        h[0] = __floats2bfloat162_rn(v[0], v[1]);
        h[1] = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(p) = q;
    }
};

__device__ __forceinline__ float warp_sum(float v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Lane l of a warp holds columns (k * 32 + l) * 4 .. + 3 for k = 0 .. EPL / 4 - 1.
template <int EPL, typename TX, typename TY>
__global__ void __launch_bounds__(WARPS * 32)
ln_fwd_kernel(const TX* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
              TY* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, long rows,
              float eps) {
    constexpr int V = EPL / 4;
    constexpr int D = EPL * 32;
    const int lane = threadIdx.x & 31;
    const long warp = (long)blockIdx.x * WARPS + (threadIdx.x >> 5);
    const long nwarps = (long)gridDim.x * WARPS;
    float gw[V][4], gb[V][4];
    #pragma unroll
    for (int k = 0; k < V; ++k) {
        Io<float>::load4(w + (k * 32 + lane) * 4, gw[k]);
        Io<float>::load4(b + (k * 32 + lane) * 4, gb[k]);
    }
    for (long row = warp; row < rows; row += nwarps) {
        float v[V][4];
        float sum = 0.0f;
        #pragma unroll
        for (int k = 0; k < V; ++k) {
            Io<TX>::load4(x + row * D + (k * 32 + lane) * 4, v[k]);
            sum += (v[k][0] + v[k][1]) + (v[k][2] + v[k][3]);
        }
        const float mu = warp_sum(sum) * (1.0f / D);
        float sq = 0.0f;
        #pragma unroll
        for (int k = 0; k < V; ++k) {
            #pragma unroll
            for (int j = 0; j < 4; ++j) { const float c = v[k][j] - mu; sq += c * c; }
        }
        const float rs = rsqrtf(warp_sum(sq) * (1.0f / D) + eps);
        #pragma unroll
        for (int k = 0; k < V; ++k) {
            float o[4];
            #pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = (v[k][j] - mu) * rs * gw[k][j] + gb[k][j];
            Io<TY>::store4(y + row * D + (k * 32 + lane) * 4, o);
        }
        if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
    }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)), g = dy * w;  dgamma = sum dy * xhat,
// dbeta = sum dy.  Every warp leaves its partial dgamma / dbeta in part[warp][2][D].
template <int EPL, typename TX, typename TDY>
__global__ void __launch_bounds__(WARPS * 32)
ln_bwd_kernel(const TDY* __restrict__ dy, const TX* __restrict__ x, const float* __restrict__ w,
              const float* __restrict__ mean, const float* __restrict__ rstd, TX* __restrict__ dx,
              float* __restrict__ part, long rows) {
    constexpr int V = EPL / 4;
    constexpr int D = EPL * 32;
    const int lane = threadIdx.x & 31;
    const long warp = (long)blockIdx.x * WARPS + (threadIdx.x >> 5);
    const long nwarps = (long)gridDim.x * WARPS;
    float gw[V][4], dw[V][4], db[V][4];
    #pragma unroll
    for (int k = 0; k < V; ++k) {
        Io<float>::load4(w + (k * 32 + lane) * 4, gw[k]);
        #pragma unroll
        for (int j = 0; j < 4; ++j) { dw[k][j] = 0.0f; db[k][j] = 0.0f; }
    }
    for (long row = warp; row < rows; row += nwarps) {
        const float mu = mean[row], rs = rstd[row];
        float xh[V][4], g[V][4];
        float s1 = 0.0f, s2 = 0.0f;
        #pragma unroll
        for (int k = 0; k < V; ++k) {
            float xv[4], dv[4];
            Io<TX>::load4(x + row * D + (k * 32 + lane) * 4, xv);
            Io<TDY>::load4(dy + row * D + (k * 32 + lane) * 4, dv);
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                xh[k][j] = (xv[j] - mu) * rs;
                g[k][j] = dv[j] * gw[k][j];
                s1 += g[k][j];
                s2 += g[k][j] * xh[k][j];
                dw[k][j] += dv[j] * xh[k][j];
                db[k][j] += dv[j];
            }
        }
        const float m1 = warp_sum(s1) * (1.0f / D), m2 = warp_sum(s2) * (1.0f / D);
        #pragma unroll
        for (int k = 0; k < V; ++k) {
            float o[4];
            #pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = rs * (g[k][j] - m1 - xh[k][j] * m2);
            Io<TX>::store4(dx + row * D + (k * 32 + lane) * 4, o);
        }
    }
    float* mine = part + warp * 2 * D;
    #pragma unroll
    for (int k = 0; k < V; ++k) {
        Io<float>::store4(mine + (k * 32 + lane) * 4, dw[k]);
        Io<float>::store4(mine + D + (k * 32 + lane) * 4, db[k]);
    }
}

// out[c] = sum over parts of part[p][c], parts added in index order; c < 2 * D.
__global__ void ln_reduce_kernel(const float* __restrict__ part, float* __restrict__ dgamma,
                                 float* __restrict__ dbeta, long parts, int d) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= 2 * d) return;
    float acc = 0.0f;
    for (long p = 0; p < parts; ++p) acc += part[p * 2 * d + c];
    if (c < d) dgamma[c] = acc; else dbeta[c - d] = acc;
}

int grid_for(long rows) {
    const long want = (rows + WARPS - 1) / WARPS;
    const long cap = 148 * 4;
    return (int)(want < cap ? want : cap);
}

template <int EPL>
cudaError_t fwd(int xdt, int ydt, const void* x, const float* w, const float* b, void* y,
                float* mean, float* rstd, long rows, float eps, cudaStream_t s) {
    const int grid = grid_for(rows);
    if (xdt == 0 && ydt == 0)
        ln_fwd_kernel<EPL, float, float><<<grid, WARPS * 32, 0, s>>>(
            (const float*)x, w, b, (float*)y, mean, rstd, rows, eps);
    else if (xdt == 0 && ydt == 1)
        ln_fwd_kernel<EPL, float, __nv_bfloat16><<<grid, WARPS * 32, 0, s>>>(
            (const float*)x, w, b, (__nv_bfloat16*)y, mean, rstd, rows, eps);
    else if (xdt == 1 && ydt == 1)
        ln_fwd_kernel<EPL, __nv_bfloat16, __nv_bfloat16><<<grid, WARPS * 32, 0, s>>>(
            (const __nv_bfloat16*)x, w, b, (__nv_bfloat16*)y, mean, rstd, rows, eps);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

template <int EPL>
cudaError_t bwd(int xdt, int dydt, const void* dy, const void* x, const float* w, const float* mean,
                const float* rstd, void* dx, float* part, float* dgamma, float* dbeta, long rows,
                cudaStream_t s) {
    const int grid = grid_for(rows);
    if (xdt == 0 && dydt == 0)
        ln_bwd_kernel<EPL, float, float><<<grid, WARPS * 32, 0, s>>>(
            (const float*)dy, (const float*)x, w, mean, rstd, (float*)dx, part, rows);
    else if (xdt == 0 && dydt == 1)
        ln_bwd_kernel<EPL, float, __nv_bfloat16><<<grid, WARPS * 32, 0, s>>>(
            (const __nv_bfloat16*)dy, (const float*)x, w, mean, rstd, (float*)dx, part, rows);
    else if (xdt == 1 && dydt == 1)
        ln_bwd_kernel<EPL, __nv_bfloat16, __nv_bfloat16><<<grid, WARPS * 32, 0, s>>>(
            (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, w, mean, rstd, (__nv_bfloat16*)dx,
            part, rows);
    else return cudaErrorInvalidValue;
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    const int d = EPL * 32;
    ln_reduce_kernel<<<(2 * d + 255) / 256, 256, 0, s>>>(part, dgamma, dbeta, (long)grid * WARPS, d);
    return cudaGetLastError();
}

}  // namespace

// dtype codes: 0 float32, 1 bfloat16.  d must be 128 * k, k = 1 .. 16 (checked).  All pointers
// 16-byte aligned.  Returns a cudaError_t.
extern "C" int gb_layernorm_fwd(int x_dtype, int y_dtype, const void* x, const float* weight,
                                const float* bias, void* y, float* mean, float* rstd, long rows,
                                int d, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    switch (d) {
#define GB_LN_CASE(K) case 128 * K: return (int)fwd<4 * K>(x_dtype, y_dtype, x, weight, bias, y, mean, rstd, rows, eps, stream);
        GB_LN_CASE(1) GB_LN_CASE(2) GB_LN_CASE(3) GB_LN_CASE(4) GB_LN_CASE(5) GB_LN_CASE(6)
        GB_LN_CASE(7) GB_LN_CASE(8) GB_LN_CASE(10) GB_LN_CASE(12) GB_LN_CASE(16)
#undef GB_LN_CASE
    }
    return (int)cudaErrorInvalidValue;
}

// The number of float values `part` must hold: parts * 2 * d with parts = warps of the launch.
extern "C" long gb_layernorm_scratch(long rows, int d) {
    return (long)grid_for(rows) * WARPS * 2 * d;
}

extern "C" int gb_layernorm_bwd(int x_dtype, int dy_dtype, const void* dy, const void* x,
                                const float* weight, const float* mean, const float* rstd, void* dx,
                                float* part, float* dgamma, float* dbeta, long rows, int d,
                                cudaStream_t stream) {
    if (rows <= 0) return 0;
    switch (d) {
#define GB_LN_CASE(K) case 128 * K: return (int)bwd<4 * K>(x_dtype, dy_dtype, dy, x, weight, mean, rstd, dx, part, dgamma, dbeta, rows, stream);
        GB_LN_CASE(1) GB_LN_CASE(2) GB_LN_CASE(3) GB_LN_CASE(4) GB_LN_CASE(5) GB_LN_CASE(6)
        GB_LN_CASE(7) GB_LN_CASE(8) GB_LN_CASE(10) GB_LN_CASE(12) GB_LN_CASE(16)
#undef GB_LN_CASE
    }
    return (int)cudaErrorInvalidValue;
}
