// Token embedding: out[t, :] = table[ids[t], :] as float32 (the residual
// stream is float32 in both precisions).  No scaling of the embeddings
// (andre-fu/prism engine/executor.py:74-75).
#include "common.cuh"
#include "vec.cuh"

namespace prism {

template <typename W>
__global__ void embed_kernel(const int* __restrict__ ids, const W* __restrict__ table,
                             float* __restrict__ out, int H, int V, int* err) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = pdl_fresh(ids)[t];            // in pipelined decoding the ids are the sampler's output
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) report_error(err, PRISM_ERR_TOKEN_RANGE);
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const W* row = table + (size_t)id * H;
    if (H % 8 == 0) {
        for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
            float v[8];
            load8(row + i, v);
            store8(o + i, v);
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]);
}

}  // namespace prism

PRISM_EXPORT int prism_embed(const int* ids, const void* table, int table_dtype, float* out,
                             int T, int H, int V, int* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    if (table_dtype == PRISM_DTYPE_BF16)
        return (int)prism::launch_kernel(prism::embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, ids,
                                         (const __nv_bfloat16*)table, out, H, V, err);
    return (int)prism::launch_kernel(prism::embed_kernel<float>, dim3(T), dim3(threads), 0, stream, ids,
                                     (const float*)table, out, H, V, err);
}
