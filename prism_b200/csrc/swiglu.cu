// SwiGLU gate: out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(z) = z * sigmoid(z),
// gate columns first and up columns second (andre-fu/prism engine/executor.py:125-127;
// fused buffer engine/weight_pool.py:194-197).  float32 arithmetic, one rounding at the store.
#include "common.cuh"
#include "vec.cuh"

namespace prism {

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I, i = idx % I;
        const float g = to_float(gu[t * 2 * I + i]);
        const float u = to_float(gu[t * 2 * I + I + i]);
        out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
    }
}

// I % 8 == 0: a thread takes 8 neighbouring columns of one row (16-byte accesses for bf16).
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int I) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= I) return;
    float g[8], u[8];
    load8(gu + (size_t)t * 2 * I + c, g);
    load8(gu + (size_t)t * 2 * I + I + c, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = g[k] / (1.f + expf(-g[k])) * u[k];
    store8(out + (size_t)t * I + c, g);
}

}  // namespace prism

PRISM_EXPORT int prism_swiglu(const void* gu, void* out, int dtype, int T, int I, cudaStream_t stream) {
    const size_t total = (size_t)T * I;
    if (total == 0) return 0;
    if (I % 8 == 0 && T <= 65535) {
        dim3 grid((I / 8 + 255) / 256, T);
        if (dtype == PRISM_DTYPE_BF16)
            prism::swiglu_vec_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I);
        else
            prism::swiglu_vec_kernel<float><<<grid, 256, 0, stream>>>((const float*)gu, (float*)out, I);
        return (int)cudaPeekAtLastError();
    }
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (dtype == PRISM_DTYPE_BF16)
        prism::swiglu_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, total);
    else
        prism::swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, I, total);
    return (int)cudaPeekAtLastError();
}
