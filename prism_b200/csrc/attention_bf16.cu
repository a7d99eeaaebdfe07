// extern "C" launchers of the bf16 tensor-core attention kernels (attention_bf16.cuh).
#include "attention_bf16.cuh"

// 1 if the tensor-core kernels take this shape (else the generic kernel must be used): head sizes in steps
// of 16 up to 128 (the output row of a head stays in registers), up to 16 query heads per kv head (the rows of
// one 16-row MMA tile in the decode kernel)
PRISM_EXPORT int prism_attention_bf16_supported(int hd, int nh, int nkv) {
    return hd >= 16 && hd <= 128 && hd % 16 == 0 && nkv > 0 && nh % nkv == 0 && nh / nkv <= 16;
}

// one instantiation per head size
#define PRISM_BY_HEAD_SIZE(hd, CALL)                   \
    switch (hd) {                                      \
        case 16: return CALL(16);                      \
        case 32: return CALL(32);                      \
        case 48: return CALL(48);                      \
        case 64: return CALL(64);                      \
        case 80: return CALL(80);                      \
        case 96: return CALL(96);                      \
        case 112: return CALL(112);                    \
        case 128: return CALL(128);                    \
    }                                                  \
    return (int)cudaErrorInvalidValue

// Decode: T tokens, one per request.  part_o: float [T, nh, nsplit, hd]; part_ml: float [T, nh, nsplit, 2].
// With nsplit > 1 a second kernel merges the splits' partial results.
// items (optional, device, 16-byte aligned): n_items work items {token, split | used << 16, position, segment} and
// starts [T] (token t's items are the `used` ones from `first` on, starts[t] = first | used << 16; at most 65,535
// items): every token's keys are then shared among the
// CTAs the host chose for it (ops.decode_work_items); nsplit is the most items of a token, part_o is
// float [n_items, nh, hd] and part_ml float [n_items, nh, 2], positions and tok_seg are not read.
PRISM_EXPORT int prism_attention_decode_bf16(const void* q, int q_stride, void* out, int out_stride,
                                             const void* kc, const void* vc, const int* block_table,
                                             int bt_width, const int* positions, const int* tok_seg,
                                             int T, int nh, int nkv, int hd, int page_size, int num_pages,
                                             int window, float scale, float* part_o, float* part_ml,
                                             int nsplit, const int* items, const int* starts, int n_items,
                                             int* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!prism_attention_bf16_supported(hd, nh, nkv) || nsplit < 1 || nkv > 65535 || T > 65535 ||
        (items != nullptr && (starts == nullptr || n_items < 1 || n_items > 65535 || ((uintptr_t)items & 15))))
        return (int)cudaErrorInvalidValue;
#define ARGS (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)kc, \
             (const __nv_bfloat16*)vc, block_table, bt_width, positions, tok_seg, T, nh, nkv, page_size, num_pages, \
             window, scale, part_o, part_ml, nsplit, err, stream, nullptr, items, starts, n_items
#define CALL(HD) prism::launch_decode<HD>(ARGS)
    PRISM_BY_HEAD_SIZE(hd, CALL);
#undef CALL
#undef ARGS
}

// Decode with the back half of the qkv projection inside: instead of q and a cache that already holds the tokens'
// own keys and values, the kernel gets the projection's float32 partial sums parts [ks, T, D] (D = (nh + 2 nkv) * hd,
// q | k | v), the bias [D] (float or bf16, or null) and the step's rotary table [T, hd / 2] of (cos, sin) pairs; it
// adds, biases and rotates (all of hd) itself and stores each token's key and value at its position.
PRISM_EXPORT int prism_attention_decode_qkv_bf16(const float* parts, int ks, const void* bias, int bias_dtype,
                                                 const void* table, int max_pos, void* out, int out_stride, void* kc,
                                                 void* vc, const int* block_table, int bt_width, const int* positions,
                                                 const int* tok_seg, int T, int nh, int nkv, int hd, int page_size,
                                                 int num_pages, int window, float scale, float* part_o, float* part_ml,
                                                 int nsplit, const int* items, const int* starts, int n_items,
                                                 int* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!prism_attention_bf16_supported(hd, nh, nkv) || nsplit < 1 || nkv > 65535 || T > 65535 || ks < 1 ||
        (items != nullptr && (starts == nullptr || n_items < 1 || n_items > 65535 || ((uintptr_t)items & 15))) ||
        parts == nullptr || table == nullptr || ((uintptr_t)parts & 15) || ((uintptr_t)table & 15) ||
        ((uintptr_t)bias & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15) ||
        (bias_dtype != PRISM_DTYPE_F32 && bias_dtype != PRISM_DTYPE_BF16))
        return (int)cudaErrorInvalidValue;
    prism::DecodeQKV f;
    f.D = (nh + 2 * nkv) * hd;
    f.parts = parts;
    f.part_stride = (size_t)T * f.D;
    f.ks = ks;
    f.bias = bias;
    f.bias_bf16 = bias_dtype == PRISM_DTYPE_BF16;
    f.table = (const float2*)table;
    f.kc = (__nv_bfloat16*)kc;
    f.vc = (__nv_bfloat16*)vc;
    f.max_pos = max_pos;
#define ARGS (const __nv_bfloat16*)nullptr, 0, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)kc, \
             (const __nv_bfloat16*)vc, block_table, bt_width, positions, tok_seg, T, nh, nkv, page_size, num_pages, \
             window, scale, part_o, part_ml, nsplit, err, stream, &f, items, starts, n_items
#define CALL(HD) prism::launch_decode<HD>(ARGS)
    PRISM_BY_HEAD_SIZE(hd, CALL);
#undef CALL
#undef ARGS
}

// Prefill / mixed: S segments; segment s has tokens seg_start[s] .. seg_start[s+1]-1 at positions cached_len[s] + i.
PRISM_EXPORT int prism_attention_prefill_bf16(const void* q, int q_stride, void* out, int out_stride,
                                              const void* kc, const void* vc, const int* block_table,
                                              int bt_width, const int* seg_start, const int* cached_len,
                                              int S, int max_q_len, int nh, int nkv, int hd, int page_size,
                                              int num_pages, int window, float scale, int* err,
                                              cudaStream_t stream) {
    if (S <= 0 || max_q_len <= 0) return 0;
    if (!prism_attention_bf16_supported(hd, nh, nkv) || S > 65535 || nh > 65535) return (int)cudaErrorInvalidValue;
#define ARGS (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)kc, \
             (const __nv_bfloat16*)vc, block_table, bt_width, seg_start, cached_len, S, max_q_len, nh, nkv, page_size, \
             num_pages, window, scale, err, stream
#define CALL(HD) prism::launch_prefill<HD>(ARGS)
    PRISM_BY_HEAD_SIZE(hd, CALL);
#undef CALL
#undef ARGS
}

// Merge of split partial results (the decode kernel's, or the tcgen05 prefill kernel's with nsplit > 1):
// part_o float [T, nh, nsplit, hd] unnormalised outputs, part_ml float [T, nh, nsplit, 2] (reference exponent in
// log2 units, sum); out bf16 [T, nh * hd] with row stride out_stride.
PRISM_EXPORT int prism_attention_merge_bf16(const float* part_o, const float* part_ml, int nsplit, void* out,
                                            int out_stride, int T, int nh, int hd, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (nsplit < 1 || hd < 16 || hd > 128 || hd % 16) return (int)cudaErrorInvalidValue;
    // one thread per output element: the block is the head size rounded up to whole warps
#define CALL(HD) (int)prism::launch_kernel(prism::attn_merge_kernel<HD>, dim3(T * nh), dim3((HD + 31) / 32 * 32), 0, stream, \
                                           part_o, part_ml, nsplit, (__nv_bfloat16*)out, out_stride, nh,              \
                                           (const int*)nullptr)
    PRISM_BY_HEAD_SIZE(hd, CALL);
#undef CALL
}
