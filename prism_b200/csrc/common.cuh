// Shared device helpers for the prism_b200 kernels (sm_100a).
//
// Conventions used by every kernel in this directory:
//  * activations are float or __nv_bfloat16 (template parameter T); all
//    arithmetic is float, with one rounding where a tensor is stored;
//  * one-dimensional parameters (norm weights, biases) and the embedding
//    table keep the dtype they have in the model file; a kernel receives
//    them as `const void*` plus a flag (`PARAM_F32` / `PARAM_BF16`);
//  * a kernel that meets an index it must not follow (token id outside the
//    vocabulary, page id outside the pool) records a code in the device
//    error word and skips the access instead of faulting;
//  * launchers are `extern "C"`, take raw device pointers and a stream, and
//    return the cudaError_t of the launch as an int.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define PRISM_DTYPE_F32 0
#define PRISM_DTYPE_BF16 1

// error codes written to the device error word (first one wins)
#define PRISM_ERR_TOKEN_RANGE 1
#define PRISM_ERR_PAGE_RANGE 2
#define PRISM_ERR_POSITION_RANGE 3
#define PRISM_ERR_WAIT_TIMEOUT 4

#define PRISM_EXPORT extern "C" __attribute__((visibility("default")))

namespace prism {

// Programmatic dependent launch.  A kernel launched with the attribute below may
// start while the kernel before it in the stream is still running; it must call
// pdl_wait() before it reads or writes anything that kernel (or an earlier one)
// touches - the call returns once all of the earlier grid's memory operations
// are done and visible.  pdl_trigger() tells the runtime that the next kernel
// may be launched as soon as every CTA of this one has started.  Both are
// no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// What the kernel before this one wrote must be read through pdl_fresh(pointer), taken after pdl_wait(),
// never straight through a `const T* __restrict__` parameter: the compiler treats loads through such a
// parameter as invariant for the whole kernel and may hoist them above the wait (the "memory" clobber
// does not hold them back).  That happened: decode attention read the previous step's q from a CUDA
// graph's static buffer.  The empty volatile asm makes the pointer a value produced after the wait.
template <typename T> __device__ __forceinline__ T* pdl_fresh(T* p) {
    asm volatile("" : "+l"(p)::"memory");
    return p;
}
#ifndef PRISM_PDL_TRIGGER_SMALL
#define PRISM_PDL_TRIGGER_SMALL 1
#endif
#ifndef PRISM_PDL_TRIGGER_GEMM
#define PRISM_PDL_TRIGGER_GEMM 1
#endif
__device__ __forceinline__ void pdl_trigger() {
#if PRISM_PDL_TRIGGER_SMALL
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}
__device__ __forceinline__ void pdl_trigger_gemm() {
#if PRISM_PDL_TRIGGER_GEMM
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}

// 1: kernels of this library are launched with programmatic stream serialization
// (the default); 0: plain launches.  Set through prism_set_pdl().
inline int& pdl_enabled() {
    static int on = 1;
    return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ void report_error(int* err, int code) {
    if (err != nullptr) atomicCAS(err, 0, code);
}

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

// element i of a parameter vector stored as float or bf16
__device__ __forceinline__ float load_param(const void* p, int is_bf16, size_t i) {
    return is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i])
                   : reinterpret_cast<const float*>(p)[i];
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` is 33 floats of shared memory.  The order of additions depends
// only on the block size, never on the data or the grid.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

}  // namespace prism
