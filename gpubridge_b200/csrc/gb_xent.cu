// Fused softmax cross-entropy over the vocabulary, forward and backward in one kernel.
//
// The benchmark models end in a [tokens x vocab] logit matrix (8192 x 50257 for GPT-2 small,
// 0.8 GB in bf16).  The stock path upcasts it to fp32, runs log_softmax, nll_loss and their
// backward kernels and casts the gradient back: about ten passes over 0.8-1.6 GB.  Here one
// block owns a row: a first sweep computes the running maximum and the sum of exponentials
// (online softmax), a second sweep - served from L2, a row is about 100 KB - overwrites the
// logits in place with d(mean loss)/d(logits) in the logits' dtype.  The rows may be padded
// (leading dimension ld >= vocab, so the head GEMM runs on aligned shapes); padding columns
// get a zero gradient.  The mean of the row losses is reduced in a fixed order by the last
// block to finish, so the result does not depend on scheduling.
//
// Scratch: row_loss[rows] floats and one arrival counter (which the kernel leaves at zero).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <math_constants.h>

namespace {

constexpr int THREADS = 512;

template <typename T> struct Pack;
template <> struct Pack<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
        #pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = raw;
    }
};
template <> struct Pack<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        float4 raw = *reinterpret_cast<const float4*>(p);
        v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
    const float mx = fmaxf(m, m2);
    if (mx == -CUDART_INF_F) { m = mx; s = 0.0f; return; }
    s = s * __expf(m - mx) + s2 * __expf(m2 - mx);
    m = mx;
}

// Block-wide (max, sum-of-exponentials) of per-thread partials; every thread gets the result.
__device__ __forceinline__ void block_softmax_stats(float& m, float& s) {
    __shared__ float sm[THREADS / 32], ss[THREADS / 32];
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float m2 = __shfl_xor_sync(0xffffffffu, m, o);
        float s2 = __shfl_xor_sync(0xffffffffu, s, o);
        online_merge(m, s, m2, s2);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                       // the arrays may still be read from the last row
    if (lane == 0) { sm[warp] = m; ss[warp] = s; }
    __syncthreads();
    m = sm[0]; s = ss[0];
    #pragma unroll
    for (int w = 1; w < THREADS / 32; ++w) online_merge(m, s, sm[w], ss[w]);
}

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// 2^x by the special-function unit (about 2 ulp; results below 2^-126 flush to zero, which
// is below what a sum of exponentials can resolve anyway).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Statistics are kept in the base-2 domain: t = logit * log2(e), m = running max of t,
// s = sum of 2^(t - m).  One vector at a time: the vector's maximum decides whether the
// running sum is rescaled (rare after the first few vectors), then each element costs one
// fused multiply-add, one ex2 and one add.  Columns at or beyond `limit` do not count.
template <int N>
__device__ __forceinline__ void stats_vector(const float (&e)[N], size_t col0, size_t limit,
                                             bool checked, float& m, float& s) {
    float t[N];
    float vm = -CUDART_INF_F;
    #pragma unroll
    for (int j = 0; j < N; ++j) {
        t[j] = e[j] * LOG2E;
        if (checked && col0 + j >= limit) t[j] = -CUDART_INF_F;
        vm = fmaxf(vm, t[j]);
    }
    if (vm > m) { s *= fast_exp2(m - vm); m = vm; }       // m = -inf: s is 0 and 2^(-inf) is 0
    if (m == -CUDART_INF_F) return;
    #pragma unroll
    for (int j = 0; j < N; ++j) s += fast_exp2(t[j] - m);
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
xent_kernel(T* __restrict__ logits, const long long* __restrict__ targets, size_t rows,
            size_t vocab, size_t ld, float grad_scale, float* __restrict__ row_loss,
            unsigned int* __restrict__ counter, float* __restrict__ loss_out) {
    constexpr int N = Pack<T>::N;
    const size_t nvec = ld / N;                       // ld is a multiple of N
    const size_t nfull = vocab / N;                   // vectors that lie wholly inside the vocabulary
    for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
        T* x = logits + row * ld;
        const long long target = targets[row];
        float m = -CUDART_INF_F, s = 0.0f;
        size_t v = threadIdx.x;
        for (; v + THREADS < nfull; v += 2 * THREADS) {       // two vectors in flight per thread
            float e0[N], e1[N];
            Pack<T>::load(x + v * N, e0);
            Pack<T>::load(x + (v + THREADS) * N, e1);
            stats_vector<N>(e0, 0, 0, false, m, s);
            stats_vector<N>(e1, 0, 0, false, m, s);
        }
        for (; v < nvec; v += THREADS) {
            float e[N];
            Pack<T>::load(x + v * N, e);
            stats_vector<N>(e, v * N, vocab, v >= nfull, m, s);
        }
        m *= LN2;                                     // natural units from here on
        block_softmax_stats(m, s);
        const bool counted = target >= 0 && (size_t)target < vocab;   // ignore_index style
        if (threadIdx.x == 0) {
            float picked = counted ? (float)x[target] : 0.0f;
            row_loss[row] = counted ? (__logf(s) + m - picked) : 0.0f;
        }
        __syncthreads();                              // x[target] is read before it is rewritten
        const float coef = counted ? grad_scale / s : 0.0f;
        const float m2 = m * LOG2E;
        const size_t tvec = counted ? (size_t)target / N : (size_t)-1;
        const int tlane = counted ? (int)((size_t)target % N) : 0;
        for (v = threadIdx.x; v < nvec; v += THREADS) {
            float e[N];
            Pack<T>::load(x + v * N, e);
            const bool tail = v >= nfull;
            #pragma unroll
            for (int j = 0; j < N; ++j) {
                float g = fast_exp2(fmaf(e[j], LOG2E, -m2)) * coef;
                if (tail && v * N + j >= vocab) g = 0.0f;
                e[j] = g;
            }
            if (v == tvec) {
                #pragma unroll
                for (int j = 0; j < N; ++j) if (j == tlane) e[j] -= grad_scale;
            }
            Pack<T>::store(x + v * N, e);
        }
    }
    // the last block to finish adds the row losses in a fixed order
    __shared__ unsigned int s_last;
    __shared__ float s_part[THREADS / 32];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(counter, 1u) + 1u == gridDim.x);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float acc = 0.0f;
    for (size_t r = threadIdx.x; r < rows; r += THREADS)
        acc += *reinterpret_cast<volatile float*>(row_loss + r);
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int w = 0; w < THREADS / 32; ++w) total += s_part[w];
        *loss_out = total * grad_scale;               // grad_scale = 1 / rows: the mean
        *counter = 0u;
    }
}

template <typename T>
cudaError_t launch(void* logits, const long long* targets, size_t rows, size_t vocab, size_t ld,
                   float* row_loss, unsigned int* counter, float* loss_out, cudaStream_t stream) {
    size_t grid = rows < 148 * 4 ? rows : 148 * 4;
    xent_kernel<T><<<(int)grid, THREADS, 0, stream>>>(static_cast<T*>(logits), targets, rows, vocab,
                                                      ld, 1.0f / (float)rows, row_loss, counter,
                                                      loss_out);
    return cudaGetLastError();
}

}  // namespace

// dtype: 0 float32, 1 bfloat16.  logits: [rows, ld] row-major, 16-byte aligned, ld a multiple
// of 8 (bf16) or 4 (fp32); overwritten with the gradient of the mean loss.  targets: int64.
// row_loss: rows floats of scratch; counter: one zeroed unsigned int of scratch.
extern "C" int gb_xent_fwd_bwd(void* logits, int dtype, const long long* targets, size_t rows,
                               size_t vocab, size_t ld, float* row_loss, unsigned int* counter,
                               float* loss_out, cudaStream_t stream) {
    if (rows == 0 || vocab == 0 || vocab > ld) return (int)cudaErrorInvalidValue;
    if (dtype == 1) {
        if (ld % 8) return (int)cudaErrorInvalidValue;
        return (int)launch<__nv_bfloat16>(logits, targets, rows, vocab, ld, row_loss, counter,
                                          loss_out, stream);
    }
    if (dtype == 0) {
        if (ld % 4) return (int)cudaErrorInvalidValue;
        return (int)launch<float>(logits, targets, rows, vocab, ld, row_loss, counter, loss_out, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// ---- entry point that allocates nothing -------------------------------------------------------
// See gb_xent_noalloc.h.  The scratch that gb_xent_fwd_bwd takes from its caller lives here in a
// file-scope device array instead, so the call needs no allocation of any kind.
#include <mutex>
#include "gb_xent_noalloc.h"

namespace {

// Layout of the array: GB_XENT_NOALLOC_MAX_ROWS row losses (float), then the arrival counter.
constexpr size_t NOALLOC_COUNTER_AT = sizeof(float) * GB_XENT_NOALLOC_MAX_ROWS;
constexpr size_t NOALLOC_BYTES = NOALLOC_COUNTER_AT + 256;

// One copy per GPU that loads the library, held until the process exits.  In host code this
// name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char gb_xent_noalloc_scratch[NOALLOC_BYTES];

constexpr int MAX_DEVICES = 64;
std::mutex g_noalloc_mutex;
unsigned char* g_noalloc_ptr[MAX_DEVICES] = {};

// The device address of the array on the current device, looked up once per device.
cudaError_t noalloc_scratch(unsigned char** out) {
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return err;
    if (device < 0 || device >= MAX_DEVICES) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> guard(g_noalloc_mutex);
    if (g_noalloc_ptr[device] == nullptr) {
        void* ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, gb_xent_noalloc_scratch);
        if (err != cudaSuccess) return err;
        g_noalloc_ptr[device] = static_cast<unsigned char*>(ptr);
    }
    *out = g_noalloc_ptr[device];
    return cudaSuccess;
}

}  // namespace

extern "C" int gb_xent_fwd_bwd_noalloc(void* logits, int dtype, const long long* targets,
                                       size_t rows, size_t vocab, size_t ld, float* loss_out,
                                       cudaStream_t stream) {
    if (rows > GB_XENT_NOALLOC_MAX_ROWS) return GB_XENT_NOALLOC_TOO_MANY_ROWS;
    unsigned char* scratch = nullptr;
    cudaError_t err = noalloc_scratch(&scratch);
    if (err != cudaSuccess) return (int)err;
    float* row_loss = reinterpret_cast<float*>(scratch);
    unsigned int* counter = reinterpret_cast<unsigned int*>(scratch + NOALLOC_COUNTER_AT);
    // The arrival counter must start at zero; an earlier call that was cut short may have left
    // it otherwise.  A memset on the stream allocates nothing.
    err = cudaMemsetAsync(counter, 0, sizeof(unsigned int), stream);
    if (err != cudaSuccess) return (int)err;
    return gb_xent_fwd_bwd(logits, dtype, targets, rows, vocab, ld, row_loss, counter, loss_out,
                           stream);
}

extern "C" const char* gb_xent_noalloc_error(int code) {
    if (code == GB_XENT_NOALLOC_TOO_MANY_ROWS)
        return "gb_xent_fwd_bwd_noalloc: more rows than GB_XENT_NOALLOC_MAX_ROWS (65536); "
               "split the batch or use gb_xent_fwd_bwd with scratch of your own";
    return cudaGetErrorString((cudaError_t)code);
}
