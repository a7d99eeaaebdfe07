// Rotary position encoding of q and k fused with the store of k and v into
// the paged cache.
//
// Rotation (andre-fu/prism engine/executor.py:18-21,48-57,117-118): pairs
// (j, j + rd/2) of the first `rd` dims of a head,
//     x1' = x1*cos(a) - x2*sin(a),  x2' = x2*cos(a) + x1*sin(a),
//     a = position * inv_freq[j]
// with the angle, cos and sin in float32 (no rounded table).  q is rotated in
// place; k is rotated and written, with v unrotated, to slot `position` of
// the request's pages: page = block_table[seg, position / P], offset
// position % P (the append that flash_attn_with_kvcache does at
// executor.py:119-120).  Cache layout: [page, P, nkv, hd].
#include "common.cuh"
#include "vec.cuh"

namespace prism {

template <typename T>
__global__ void rope_kv_kernel(T* __restrict__ q, T* __restrict__ k, const T* __restrict__ v,
                               int row_stride, const int* __restrict__ positions,
                               const int* __restrict__ tok_seg, const float* __restrict__ inv_freq,
                               int rd, T* __restrict__ kc, T* __restrict__ vc,
                               const int* __restrict__ block_table, int bt_width, int page_size,
                               int num_pages, int nh, int nkv, int hd, int max_pos, int* err) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0) report_error(err, PRISM_ERR_POSITION_RANGE);
        return;
    }
    T* qrow = q + (size_t)t * row_stride;
    T* krow = k + (size_t)t * row_stride;
    const T* vrow = v + (size_t)t * row_stride;

    size_t slot = 0;
    bool store = kc != nullptr;
    if (store) {
        const int page = block_table[(size_t)tok_seg[t] * bt_width + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) report_error(err, PRISM_ERR_PAGE_RANGE);
            store = false;
        } else {
            slot = ((size_t)page * page_size + (pos % page_size)) * (size_t)nkv * hd;
        }
    }
    const int half = rd / 2;
    const int pairs_per_head = hd - half;   // `half` rotated pairs + (hd - rd) pass-through dims
    // q heads: rotate in place
    for (int i = threadIdx.x; i < nh * half; i += blockDim.x) {
        const int h = i / half, j = i % half;
        float s, c;
        sincosf((float)pos * inv_freq[j], &s, &c);
        T* p = qrow + h * hd;
        const float x1 = to_float(p[j]), x2 = to_float(p[j + half]);
        p[j] = from_float<T>(x1 * c - x2 * s);
        p[j + half] = from_float<T>(x2 * c + x1 * s);
    }
    // k heads: rotate, keep in place (a layer that shares another layer's
    // cache still sees its own rotated k in the activation buffer) and store
    for (int i = threadIdx.x; i < nkv * pairs_per_head; i += blockDim.x) {
        const int h = i / pairs_per_head, j = i % pairs_per_head;
        T* p = krow + h * hd;
        if (j < half) {
            float s, c;
            sincosf((float)pos * inv_freq[j], &s, &c);
            const float x1 = to_float(p[j]), x2 = to_float(p[j + half]);
            const T y1 = from_float<T>(x1 * c - x2 * s), y2 = from_float<T>(x2 * c + x1 * s);
            p[j] = y1;
            p[j + half] = y2;
            if (store) {
                kc[slot + h * hd + j] = y1;
                kc[slot + h * hd + j + half] = y2;
            }
        } else if (store) {
            const int d = j + half;          // dims rd .. hd-1 are not rotated
            kc[slot + h * hd + d] = p[d];
        }
    }
    if (store)
        for (int i = threadIdx.x; i < nkv * hd; i += blockDim.x) vc[slot + i] = vrow[i];
}

// cos/sin of every (token, pair) of a step, computed once and shared by all
// layers and heads: table[t, j] = (cos, sin)(position[t] * inv_freq[j]), float32.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  int half, int T, float2* __restrict__ table) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * half) return;
    float s, c;
    sincosf((float)positions[i / half] * inv_freq[i % half], &s, &c);
    table[i] = make_float2(c, s);
}

// Vector version: head_dim % 8 == 0 and rotary_dim % 16 == 0; cos/sin come from
// the table.  A thread rotates 8 neighbouring pairs (two 16-byte accesses for
// bf16), or copies 8 unrotated dims.
template <typename T>
__global__ void rope_kv_vec_kernel(T* __restrict__ q, T* __restrict__ k, const T* __restrict__ v_in,
                                   int row_stride, const int* __restrict__ positions,
                                   const int* __restrict__ tok_seg, const float2* __restrict__ table_in,
                                   int rd, T* __restrict__ kc, T* __restrict__ vc,
                                   const int* __restrict__ block_table, int bt_width, int page_size,
                                   int num_pages, int nh, int nkv, int hd, int max_pos, int* err) {
    pdl_trigger();
    // The step's own inputs (positions, segments, block table) were complete before its first kernel
    // started: the chain position -> page -> slot is followed while the kernels before this one still run.
    const int t = blockIdx.x;
    const int pos = positions[t];
    const bool pos_ok = pos >= 0 && pos < max_pos;
    size_t slot = 0;
    bool store = kc != nullptr, page_ok = true;
    if (store && pos_ok) {
        const int page = block_table[(size_t)tok_seg[t] * bt_width + pos / page_size];
        page_ok = page >= 0 && page < num_pages;
        if (page_ok) slot = ((size_t)page * page_size + (pos % page_size)) * (size_t)nkv * hd;
        else store = false;
    }
    pdl_wait();
    if (!pos_ok || !page_ok) {
        if (threadIdx.x == 0) report_error(err, pos_ok ? PRISM_ERR_PAGE_RANGE : PRISM_ERR_POSITION_RANGE);
        if (!pos_ok) return;
    }
    const T* v = pdl_fresh(v_in);                      // outputs of the kernels before this one
    const float2* table = pdl_fresh(table_in);
    const int half = rd / 2;
    const int rot_chunks = half / 8;                   // chunks of 8 rotated pairs per head
    const int pass_chunks = (hd - rd) / 8;             // chunks of 8 unrotated dims per head
    const int per_k = rot_chunks + pass_chunks;
    const int n_q = nh * rot_chunks, n_k = nkv * per_k, n_v = nkv * (hd / 8);
    const float2* tab = table + (size_t)t * half;
    // gridDim.y CTAs share a token's items (few tokens: more CTAs, shorter latency chain)
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n_q + n_k + n_v; i += blockDim.x * gridDim.y) {
        if (i < n_q + n_k) {
            const bool is_q = i < n_q;
            const int ii = is_q ? i : i - n_q;
            const int per = is_q ? rot_chunks : per_k;
            const int h = ii / per, c = ii % per;
            T* p = (is_q ? q : k) + (size_t)t * row_stride + h * hd;
            if (c < rot_chunks) {
                const int j = c * 8;
                float x1[8], x2[8], y1[8], y2[8];
                load8(p + j, x1);
                load8(p + j + half, x2);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float2 cs = tab[j + e];
                    y1[e] = x1[e] * cs.x - x2[e] * cs.y;
                    y2[e] = x2[e] * cs.x + x1[e] * cs.y;
                }
                store8(p + j, y1);
                store8(p + j + half, y2);
                if (!is_q && store) {
                    store8(kc + slot + h * hd + j, y1);
                    store8(kc + slot + h * hd + j + half, y2);
                }
            } else if (store) {                          // only k has these items
                const int d = rd + (c - rot_chunks) * 8;
                float x[8];
                load8(p + d, x);
                store8(kc + slot + h * hd + d, x);
            }
        } else if (store) {
            const int d = (i - n_q - n_k) * 8;
            float x[8];
            load8(v + (size_t)t * row_stride + d, x);
            store8(vc + slot + d, x);
        }
    }
}

// The same rotation and store, reading q/k/v as a stack of float32 partial sums
// [ks, T, D] of the qkv projection (D = (nh + 2 nkv) * hd; a K-split product leaves
// them so) plus an optional bias, and writing the rotated q to its own buffer.
// Sum, bias and rotation in float32, one rounding at each store.
template <typename T>
__global__ void rope_kv_partial_kernel(const float* __restrict__ parts_in, int ks, size_t part_stride, int D,
                                       const void* __restrict__ bias, int bias_bf16, T* __restrict__ q_out,
                                       int q_out_stride, const int* __restrict__ positions,
                                       const int* __restrict__ tok_seg, const float2* __restrict__ table_in, int rd,
                                       T* __restrict__ kc, T* __restrict__ vc, const int* __restrict__ block_table,
                                       int bt_width, int page_size, int num_pages, int nh, int nkv, int hd,
                                       int max_pos, int* err) {
    pdl_trigger();
    // The step's own inputs (positions, segments, block table) were complete before its first kernel
    // started: the chain position -> page -> slot is followed, and the bias brought into L2, while the
    // kernels before this one still run.
    const int t = blockIdx.x;
    const int pos = positions[t];
    const bool pos_ok = pos >= 0 && pos < max_pos;
    size_t slot = 0;
    bool store = kc != nullptr, page_ok = true;
    if (store && pos_ok) {
        const int page = block_table[(size_t)tok_seg[t] * bt_width + pos / page_size];
        page_ok = page >= 0 && page < num_pages;
        if (page_ok) slot = ((size_t)page * page_size + (pos % page_size)) * (size_t)nkv * hd;
        else store = false;
    }
    if (bias != nullptr && blockIdx.x == 0) {
        const size_t bias_bytes = (size_t)D * (bias_bf16 ? 2 : 4);
        for (size_t b = ((size_t)blockIdx.y * blockDim.x + threadIdx.x) * 128; b < bias_bytes;
             b += (size_t)blockDim.x * gridDim.y * 128)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(bias) + b));
    }
    pdl_wait();
    if (!pos_ok || !page_ok) {
        if (threadIdx.x == 0) report_error(err, pos_ok ? PRISM_ERR_PAGE_RANGE : PRISM_ERR_POSITION_RANGE);
        if (!pos_ok) return;
    }
    const float* parts = pdl_fresh(parts_in);          // outputs of the kernels before this one
    const float2* table = pdl_fresh(table_in);
    auto load_sum8 = [&](int col, float (&v)[8]) {
        if (bias != nullptr) load_param8(bias, bias_bf16, col, v);
        else
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = 0.f;
        // four splits' loads in flight together; the additions stay in the order s = 0, 1, ...
        for (int s0 = 0; s0 < ks; s0 += 4) {
            float p[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (s0 + u < ks) load8(parts + (size_t)(s0 + u) * part_stride + (size_t)t * D + col, p[u]);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (s0 + u < ks)
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] += p[u][e];
        }
    };
    const int half = rd / 2;
    const int rot_chunks = half / 8, pass_chunks = (hd - rd) / 8, per = rot_chunks + pass_chunks;
    const int n_q = nh * per, n_k = nkv * per, n_v = nkv * (hd / 8);
    const float2* tab = table + (size_t)t * half;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n_q + n_k + n_v; i += blockDim.x * gridDim.y) {
        if (i < n_q + n_k) {
            const bool is_q = i < n_q;
            if (!is_q && !store) continue;
            const int ii = is_q ? i : i - n_q;
            const int h = ii / per, c = ii % per;
            const int col0 = (is_q ? 0 : nh * hd) + h * hd;
            T* dst = is_q ? q_out + (size_t)t * q_out_stride + h * hd : kc + slot + h * hd;
            if (c < rot_chunks) {
                const int j = c * 8;
                float x1[8], x2[8], y1[8], y2[8];
                load_sum8(col0 + j, x1);
                load_sum8(col0 + j + half, x2);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float2 cs = tab[j + e];
                    y1[e] = x1[e] * cs.x - x2[e] * cs.y;
                    y2[e] = x2[e] * cs.x + x1[e] * cs.y;
                }
                store8(dst + j, y1);
                store8(dst + j + half, y2);
            } else {
                const int d = rd + (c - rot_chunks) * 8;
                float x[8];
                load_sum8(col0 + d, x);
                store8(dst + d, x);
            }
        } else if (store) {
            const int d = (i - n_q - n_k) * 8;
            float x[8];
            load_sum8((nh + nkv) * hd + d, x);
            store8(vc + slot + d, x);
        }
    }
}

}  // namespace prism

// inv_freq may be null with rotary_dim 0: no rotation, only the cache store.
// kc/vc may be null: only the rotation.
PRISM_EXPORT int prism_rope_table(const int* positions, const float* inv_freq, int half, int T,
                                  float* table, cudaStream_t stream) {
    if (T <= 0 || half <= 0) return 0;
    const int n = T * half;
    return (int)prism::launch_kernel(prism::rope_table_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, positions,
                                     inv_freq, half, T, (float2*)table);
}

// q/k/v as float32 partial sums [ks, T, (nh + 2 nkv) * hd] (+ bias): rotate, write q to q_out [T, nh * hd]
// (row stride q_out_stride) and k, v to the cache.  Needs the table, head_dim % 8 == 0, rotary_dim % 16 == 0.
PRISM_EXPORT int prism_rope_kv_write_partial(const float* parts, int ks, const void* bias, int bias_dtype, void* q_out,
                                             int q_out_stride, int dtype, const int* positions, const int* tok_seg,
                                             const float* table, int rotary_dim, void* kc, void* vc,
                                             const int* block_table, int bt_width, int page_size, int num_pages,
                                             int T, int nh, int nkv, int hd, int max_pos, int* err,
                                             cudaStream_t stream) {
    if (T <= 0) return 0;
    if (table == nullptr || hd % 8 || rotary_dim % 16 || rotary_dim > hd || q_out_stride % 8 || ks < 1)
        return (int)cudaErrorInvalidValue;
    const int D = (nh + 2 * nkv) * hd;
    const int items = (nh + nkv) * ((hd - rotary_dim / 2) / 8) + nkv * (hd / 8);
    // a few tokens: several CTAs of 32-64 threads per token, about 64 CTAs in all, instead of one of 256
    int cta_per_tok = 1;
    while (cta_per_tok < 8 && T * cta_per_tok < 64 && items / (cta_per_tok * 2) >= 32) cta_per_tok *= 2;
    const int per_cta = (items + cta_per_tok - 1) / cta_per_tok;
    const int threads = per_cta >= 256 ? 256 : (per_cta + 31) / 32 * 32;
    const dim3 grid(T, cta_per_tok);
    const int bb = bias_dtype == PRISM_DTYPE_BF16;
    if (dtype == PRISM_DTYPE_BF16)
        return (int)prism::launch_kernel(prism::rope_kv_partial_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream,
                                         parts, ks, (size_t)T * D, D, bias, bb, (__nv_bfloat16*)q_out, q_out_stride,
                                         positions, tok_seg, (const float2*)table, rotary_dim, (__nv_bfloat16*)kc,
                                         (__nv_bfloat16*)vc, block_table, bt_width, page_size, num_pages, nh, nkv, hd,
                                         max_pos, err);
    return (int)prism::launch_kernel(prism::rope_kv_partial_kernel<float>, grid, dim3(threads), 0, stream, parts, ks,
                                     (size_t)T * D, D, bias, bb, (float*)q_out, q_out_stride, positions, tok_seg,
                                     (const float2*)table, rotary_dim, (float*)kc, (float*)vc, block_table, bt_width,
                                     page_size, num_pages, nh, nkv, hd, max_pos, err);
}

// `table` (optional): float2 [T, rotary_dim / 2] from prism_rope_table; with it, and with
// head_dim % 8 == 0 and rotary_dim % 16 == 0, the vector kernel runs.
PRISM_EXPORT int prism_rope_kv_write(void* q, void* k, const void* v, int dtype, int row_stride,
                                     const int* positions, const int* tok_seg,
                                     const float* inv_freq, const float* table, int rotary_dim, void* kc, void* vc,
                                     const int* block_table, int bt_width, int page_size,
                                     int num_pages, int T, int nh, int nkv, int hd, int max_pos,
                                     int* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1)) return (int)cudaErrorInvalidValue;
    if (table != nullptr && hd % 8 == 0 && rotary_dim % 16 == 0 && row_stride % 8 == 0) {
        const int items = (nh + nkv) * (hd / 2 / 8) + nkv * (hd / 8) + nkv * ((hd - rotary_dim) / 8);
        // up to 128 tokens: four CTAs of 64-128 threads per token instead of one of 256
        const int parts = (T <= 128 && items >= 256) ? 4 : 1;
        const int per_cta = (items + parts - 1) / parts;
        const int vthreads = per_cta >= 256 ? 256 : (per_cta + 31) / 32 * 32;
        if (dtype == PRISM_DTYPE_BF16)
            return (int)prism::launch_kernel(prism::rope_kv_vec_kernel<__nv_bfloat16>, dim3(T, parts), dim3(vthreads), 0, stream,
                (__nv_bfloat16*)q, (__nv_bfloat16*)k, (const __nv_bfloat16*)v, row_stride, positions,
                tok_seg, (const float2*)table, rotary_dim, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc,
                block_table, bt_width, page_size, num_pages, nh, nkv, hd, max_pos, err);
        return (int)prism::launch_kernel(prism::rope_kv_vec_kernel<float>, dim3(T, parts), dim3(vthreads), 0, stream,
                (float*)q, (float*)k, (const float*)v, row_stride, positions, tok_seg,
                (const float2*)table, rotary_dim, (float*)kc, (float*)vc, block_table, bt_width,
                page_size, num_pages, nh, nkv, hd, max_pos, err);
    }
    const int threads = 128;
    if (dtype == PRISM_DTYPE_BF16)
        prism::rope_kv_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(
            (__nv_bfloat16*)q, (__nv_bfloat16*)k, (const __nv_bfloat16*)v, row_stride, positions,
            tok_seg, inv_freq, rotary_dim, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, block_table,
            bt_width, page_size, num_pages, nh, nkv, hd, max_pos, err);
    else
        prism::rope_kv_kernel<float><<<T, threads, 0, stream>>>(
            (float*)q, (float*)k, (const float*)v, row_stride, positions, tok_seg, inv_freq,
            rotary_dim, (float*)kc, (float*)vc, block_table, bt_width, page_size, num_pages, nh,
            nkv, hd, max_pos, err);
    return (int)cudaPeekAtLastError();
}
