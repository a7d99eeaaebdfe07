// Paged causal grouped-query attention, shape-generic version: any head size
// up to 256, any page size, any number of heads and groups, float32 or bf16
// storage, optional sliding window.  It is the attention of the float32 path
// and the fallback of the bf16 path for shapes the tensor-core kernels refuse.
//
// For query token t of request seg at absolute position p, head h:
//     s_j = (q . k_j) * scale          for keys  max(0, p - window + 1) <= j <= p
//     o   = softmax(s) @ v             q-head h reads kv-head h / (nh / nkv)
// i.e. flash_attn_with_kvcache(causal=True) over the request's pages
// (andre-fu/prism engine/executor.py:119-120), with scores, running max and
// sum and the output accumulation in float32.  Keys are visited in blocks of
// 32 starting at the window's first key, so the order of additions for a
// position depends only on that position, not on how the request was cut
// into steps or on what else is in the batch.
//
// One warp per (token, head): each lane scores one key of the block, the
// block's probabilities are exchanged by shuffles, and each lane accumulates
// the output dims lane, lane+32, ...
#include "common.cuh"

namespace prism {

template <typename T> struct VecLoad;
template <> struct VecLoad<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ float dot(const float* __restrict__ a, const float* __restrict__ q) {
        const float4 v = *reinterpret_cast<const float4*>(a);
        return v.x * q[0] + v.y * q[1] + v.z * q[2] + v.w * q[3];
    }
};
template <> struct VecLoad<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ float dot(const __nv_bfloat16* __restrict__ a, const float* __restrict__ q) {
        const uint4 raw = *reinterpret_cast<const uint4*>(a);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            s += f.x * q[2 * i] + f.y * q[2 * i + 1];
        }
        return s;
    }
};

constexpr int ATTN_GENERIC_MAXD = 8;   // output dims per lane: head_dim <= 256

template <typename T>
__global__ void attn_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out,
                                    int out_stride, const T* __restrict__ kc,
                                    const T* __restrict__ vc, const int* __restrict__ block_table,
                                    int bt_width, const int* __restrict__ positions,
                                    const int* __restrict__ tok_seg, int Ttot, int nh, int nkv,
                                    int hd, int page_size, int num_pages, int window, float scale,
                                    int* err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (w >= (long long)Ttot * nh) return;
    const int t = (int)(w / nh), h = (int)(w % nh);
    const int kvh = h / (nh / nkv);
    const int pos = positions[t];
    const int* bt = block_table + (size_t)tok_seg[t] * bt_width;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    float* qs = smem + warp * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = to_float(q[(size_t)t * q_stride + h * hd + d]);
    __syncwarp();

    float acc[ATTN_GENERIC_MAXD];
#pragma unroll
    for (int i = 0; i < ATTN_GENERIC_MAXD; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const bool vec_ok = (hd % VecLoad<T>::N) == 0;

    for (int kb = lo; kb <= pos; kb += 32) {
        const int j = kb + lane;
        bool valid = j <= pos;
        int rowidx = -1;
        if (valid) {
            const int page = bt[j / page_size];
            if (page < 0 || page >= num_pages) {
                report_error(err, PRISM_ERR_PAGE_RANGE);
                valid = false;
            } else {
                rowidx = page * page_size + j % page_size;
            }
        }
        float s = -INFINITY;
        if (valid) {
            const T* kr = kc + ((size_t)rowidx * nkv + kvh) * hd;
            float dot = 0.f;
            if (vec_ok) {
                for (int d = 0; d < hd; d += VecLoad<T>::N) dot += VecLoad<T>::dot(kr + d, qs + d);
            } else {
                for (int d = 0; d < hd; ++d) dot += qs[d] * to_float(kr[d]);
            }
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;            // only after a page error
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < ATTN_GENERIC_MAXD; ++i) acc[i] *= corr;
        const int cnt = min(32, pos - kb + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int rj = __shfl_sync(0xffffffffu, rowidx, jj);
            if (rj < 0) continue;
            const T* vr = vc + ((size_t)rj * nkv + kvh) * hd;
#pragma unroll
            for (int i = 0; i < ATTN_GENERIC_MAXD; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] += pj * to_float(vr[d]);
            }
        }
        m = m_new;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < ATTN_GENERIC_MAXD; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) out[(size_t)t * out_stride + h * hd + d] = from_float<T>(acc[i] * inv);
    }
}

}  // namespace prism

// window <= 0: all keys.  Returns cudaErrorInvalidValue for head_dim > 256.
PRISM_EXPORT int prism_attention_generic(const void* q, int q_stride, void* out, int out_stride,
                                         const void* kc, const void* vc, int dtype,
                                         const int* block_table, int bt_width,
                                         const int* positions, const int* tok_seg, int T, int nh,
                                         int nkv, int hd, int page_size, int num_pages, int window,
                                         float scale, int* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd > 32 * prism::ATTN_GENERIC_MAXD || nkv <= 0 || nh % nkv != 0) return (int)cudaErrorInvalidValue;
    const int warps = 4;
    const long long total = (long long)T * nh;
    const int blocks = (int)((total + warps - 1) / warps);
    const size_t smem = (size_t)warps * hd * sizeof(float);
    if (dtype == PRISM_DTYPE_BF16)
        prism::attn_generic_kernel<__nv_bfloat16><<<blocks, warps * 32, smem, stream>>>(
            (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride,
            (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, block_table, bt_width, positions,
            tok_seg, T, nh, nkv, hd, page_size, num_pages, window, scale, err);
    else
        prism::attn_generic_kernel<float><<<blocks, warps * 32, smem, stream>>>(
            (const float*)q, q_stride, (float*)out, out_stride, (const float*)kc, (const float*)vc,
            block_table, bt_width, positions, tok_seg, T, nh, nkv, hd, page_size, num_pages,
            window, scale, err);
    return (int)cudaPeekAtLastError();
}
