// Residual add fused with RMSNorm.
//
//   residual[r, :] += sum_s delta[s, r, :]          (float32, in place)
//   out[i, :] = residual[r, :] * rsqrt(mean(residual[r, :]^2) + eps) * w
//
// which is andre-fu/prism's `residual + F.linear(...)` followed by
// `fused_rms_norm` (engine/executor.py:122-124; formula
// engine/fused_kernels.py:41-49), with the sum and the norm in float32 and a
// single rounding at the store of `out`.  `rows` (optional) lists the rows to
// process, so that the final norm touches only the rows whose logits are
// wanted (executor.py:130).  One block per row; the order of additions is
// fixed by the block size, so a row's result does not depend on the batch.
#include "common.cuh"
#include "vec.cuh"

namespace prism {

template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta_in,
                                   int nsplit, size_t split_stride,
                                   const void* __restrict__ weight, int weight_bf16, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows, int H) {
    pdl_trigger();
    pdl_wait();
    const TD* delta = pdl_fresh(delta_in);          // the previous kernel's output
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* res = residual + (size_t)r * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = res[c];
        if (delta != nullptr) {
            for (int s = 0; s < nsplit; ++s)
                v += to_float(delta[(size_t)s * split_stride + (size_t)r * H + c]);
            res[c] = v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)i * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        o[c] = from_float<TO>(res[c] * inv * load_param(weight, weight_bf16, c));
}

// Vector version for H % 8 == 0 and H <= 8 * 1024 * ITERS: a thread keeps its
// 8 * ITERS values in registers between the sum of squares and the store, so
// the row is read once.  One block per row, as above.
template <typename TD, typename TO, int ITERS>
__global__ void __launch_bounds__(1024) add_rmsnorm_vec_kernel(float* __restrict__ residual, const TD* __restrict__ delta_in,
                                       int nsplit, size_t split_stride,
                                       const void* __restrict__ weight, int weight_bf16, float eps,
                                       TO* __restrict__ out, const int* __restrict__ rows, int H) {
    pdl_trigger();
    // the norm's weight is a constant: it is in registers before the kernels before this one have ended
    float w[ITERS][8];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int c = (threadIdx.x + it * blockDim.x) * 8;
        if (c < H) load_param8(weight, weight_bf16, c, w[it]);
    }
    pdl_wait();
    const TD* delta = pdl_fresh(delta_in);          // the previous kernel's output
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* res = residual + (size_t)r * H;
    float v[ITERS][8];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int c = (threadIdx.x + it * blockDim.x) * 8;
        if (c < H) {
            load8(res + c, v[it]);
            if (delta != nullptr) {
                for (int s = 0; s < nsplit; ++s) {
                    float d[8];
                    load8(delta + (size_t)s * split_stride + (size_t)r * H + c, d);
#pragma unroll
                    for (int k = 0; k < 8; ++k) v[it][k] += d[k];
                }
                store8(res + c, v[it]);
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) ss += v[it][k] * v[it][k];
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)i * H;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int c = (threadIdx.x + it * blockDim.x) * 8;
        if (c < H) {
#pragma unroll
            for (int k = 0; k < 8; ++k) w[it][k] *= v[it][k] * inv;
            store8(o + c, w[it]);
        }
    }
}

}  // namespace prism

// delta_dtype / out_dtype: PRISM_DTYPE_*.  delta may be null (plain norm).
PRISM_EXPORT int prism_add_rmsnorm(float* residual, const void* delta, int delta_dtype, int nsplit,
                                   long long split_stride, const void* weight, int weight_dtype,
                                   float eps, void* out, int out_dtype, const int* rows, int nrows,
                                   int H, cudaStream_t stream) {
    if (nrows <= 0) return 0;
    const int wb = weight_dtype == PRISM_DTYPE_BF16;
    const int chunks = H / 8;
    const bool vec = (H % 8 == 0) && chunks <= 2048;
    const int iters = chunks > 1024 ? 2 : 1;
    const int threads = vec ? ((chunks + iters - 1) / iters + 31) / 32 * 32
                            : (H >= 2048 ? 256 : (H >= 512 ? 128 : 64));
    cudaError_t rc = cudaSuccess;
#define ARGS residual, (const TD*)delta, nsplit, (size_t)split_stride, weight, wb, eps, (TO*)out, rows, H
#define LAUNCH(TDx, TOx)                                                                          \
    do {                                                                                          \
        using TD = TDx; using TO = TOx;                                                           \
        if (vec && iters == 1) rc = prism::launch_kernel(prism::add_rmsnorm_vec_kernel<TD, TO, 1>, dim3(nrows), dim3(threads), 0, stream, ARGS); \
        else if (vec) rc = prism::launch_kernel(prism::add_rmsnorm_vec_kernel<TD, TO, 2>, dim3(nrows), dim3(threads), 0, stream, ARGS);          \
        else rc = prism::launch_kernel(prism::add_rmsnorm_kernel<TD, TO>, dim3(nrows), dim3(threads), 0, stream, ARGS);              \
    } while (0)
    if (delta_dtype == PRISM_DTYPE_BF16) {
        if (out_dtype == PRISM_DTYPE_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
        else LAUNCH(__nv_bfloat16, float);
    } else {
        if (out_dtype == PRISM_DTYPE_BF16) LAUNCH(float, __nv_bfloat16);
        else LAUNCH(float, float);
    }
#undef LAUNCH
#undef ARGS
    return (int)rc;
}
