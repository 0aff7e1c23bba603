// Fused AdamW over flat buffers: one launch updates every parameter of the model.
//
// The data-parallel trainer keeps all parameters in one flat float32 buffer and all
// gradients in another (gpubridge_b200/parallel/trainer.py), so the optimizer is a single
// bandwidth-bound pass: read p, g, m, v; write p, m, v; clear g for the next backward.  The
// step count lives in device memory and is advanced by the kernel itself (by the last block to have read it, after a
// grid-wide arrival count), so the launch has no host-side state and can be replayed from a
// CUDA graph.  Arithmetic follows torch.optim.AdamW (decoupled weight decay, bias
// correction, eps added after the square root).
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

struct AdamState {
    unsigned int arrived;     // blocks that have read the step of this launch
    unsigned int pad;
    float step;               // completed steps
    float pad2;
};

__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
             float* __restrict__ v, size_t n, AdamState* state, float lr, float beta1,
             float beta2, float eps, float weight_decay, float grad_scale, int zero_grad,
             int advance) {
    __shared__ float s_step;
    if (threadIdx.x == 0) {
        s_step = *reinterpret_cast<volatile float*>(&state->step) + 1.0f;
        __threadfence();
        // the last block to have read the old value publishes the new one
        if (atomicAdd(&state->arrived, 1u) + 1u == gridDim.x) {
            state->arrived = 0u;
            if (advance) *reinterpret_cast<volatile float*>(&state->step) = s_step;
        }
    }
    __syncthreads();
    const float step = s_step;
    const float bc1 = 1.0f - powf(beta1, step);
    const float bc2 = 1.0f - powf(beta2, step);
    const float step_size = lr / bc1;
    const float sqrt_bc2 = sqrtf(bc2);
    const float decay = 1.0f - lr * weight_decay;
    const size_t nvec = n >> 2;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nth = (size_t)gridDim.x * blockDim.x;
    float4* p4 = reinterpret_cast<float4*>(p);
    float4* g4 = reinterpret_cast<float4*>(g);
    float4* m4 = reinterpret_cast<float4*>(m);
    float4* v4 = reinterpret_cast<float4*>(v);
    for (size_t i = tid; i < nvec; i += nth) {
        float4 pp = p4[i], gg = g4[i], mm = m4[i], vv = v4[i];
        float* pe = &pp.x; float* ge = &gg.x; float* me = &mm.x; float* ve = &vv.x;
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float grad = ge[j] * grad_scale;
            float w = pe[j] * decay;
            me[j] = beta1 * me[j] + (1.0f - beta1) * grad;
            ve[j] = beta2 * ve[j] + (1.0f - beta2) * grad * grad;
            const float denom = sqrtf(ve[j]) / sqrt_bc2 + eps;
            pe[j] = w - step_size * (me[j] / denom);
        }
        p4[i] = pp; m4[i] = mm; v4[i] = vv;
        if (zero_grad) g4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (size_t i = (nvec << 2) + tid; i < n; i += nth) {
        const float grad = g[i] * grad_scale;
        float w = p[i] * decay;
        m[i] = beta1 * m[i] + (1.0f - beta1) * grad;
        v[i] = beta2 * v[i] + (1.0f - beta2) * grad * grad;
        const float denom = sqrtf(v[i]) / sqrt_bc2 + eps;
        p[i] = w - step_size * (m[i] / denom);
        if (zero_grad) g[i] = 0.f;
    }
}

}  // namespace

// All pointers are 16-byte aligned device memory; `state` is 16 zeroed bytes that persist
// across steps.  `advance` = 0 updates a part of the buffers as a part of the step in progress
// (the step count is read but left as it is); the launch for the last part passes 1.  The parts
// of one step run one after another (one stream, or events between them).  `max_blocks` > 0
// caps the grid.  Returns a cudaError_t.
extern "C" int gb_adamw_span(float* p, float* g, float* m, float* v, size_t n, void* state,
                             float lr, float beta1, float beta2, float eps, float weight_decay,
                             float grad_scale, int zero_grad, int advance, int max_blocks,
                             cudaStream_t stream) {
    if (n == 0 && !advance) return 0;
    size_t blocks = (n / 4 + 256 * 4 - 1) / (256 * 4);
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 8) blocks = 148 * 8;
    // a part that runs beside other kernels can be told to leave them the SMs
    if (max_blocks > 0 && blocks > (size_t)max_blocks) blocks = (size_t)max_blocks;
    adamw_kernel<<<(int)blocks, 256, 0, stream>>>(p, g, m, v, n, static_cast<AdamState*>(state),
                                                  lr, beta1, beta2, eps, weight_decay, grad_scale,
                                                  zero_grad, advance);
    return (int)cudaGetLastError();
}

extern "C" int gb_adamw_step(float* p, float* g, float* m, float* v, size_t n, void* state,
                             float lr, float beta1, float beta2, float eps, float weight_decay,
                             float grad_scale, int zero_grad, cudaStream_t stream) {
    if (n == 0) return 0;
    return gb_adamw_span(p, g, m, v, n, state, lr, beta1, beta2, eps, weight_decay, grad_scale,
                         zero_grad, 1, 0, stream);
}
