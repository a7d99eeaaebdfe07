// Decode attention without any allocation: the split-KV partial results live
// in a file-scope device array instead of caller-provided buffers.  See
// prism_noalloc.h for who needs this and for the rules; no counterpart of it
// exists in andre-fu/prism.
#include <stdio.h>

#include "attention_bf16.cuh"
#include "prism_noalloc.h"

namespace {

constexpr size_t SCRATCH_FLOATS = PRISM_NOALLOC_SCRATCH_BYTES / sizeof(float);

// The scratch itself.  In host code this name is only a handle for the
// runtime: the address a kernel can use comes from cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_scratch[SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES] = {};      // per device, filled at that device's first call
char g_last_error[256] = "";

int refuse(int code, const char* fmt, long long a = 0, long long b = 0) {
    snprintf(g_last_error, sizeof(g_last_error), fmt, a, b);
    return code;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) const char* prism_noalloc_last_error(void) {
    return g_last_error;
}

extern "C" __attribute__((visibility("default")))
int prism_attention_decode_bf16_noalloc(const void* q, int q_stride, void* out, int out_stride,
                                        const void* k_cache, const void* v_cache,
                                        const int* block_table, int bt_width, const int* positions,
                                        const int* tok_seg, int T, int nh, int nkv, int hd,
                                        int page_size, int num_pages, int window, float scale,
                                        int nsplit, int* err, cudaStream_t stream) {
    g_last_error[0] = 0;
    if (T <= 0) return 0;
    if (!((hd == 64 || hd == 128) && nkv > 0 && nh % nkv == 0 && nh / nkv <= 16) || nsplit < 1 ||
        nkv > 65535 || T > 65535)
        return refuse((int)cudaErrorInvalidValue, "sizes not supported: head_dim must be 64 or 128, at most 16 "
                      "query heads per kv head, nsplit >= 1 (got head_dim %lld, nsplit %lld)", hd, nsplit);
    const size_t need = (size_t)T * nh * nsplit * (hd + 2);
    if (need > SCRATCH_FLOATS)
        return refuse((int)cudaErrorInvalidValue, "this call needs %lld floats of scratch (T*nh*nsplit*(hd+2)); "
                      "the built-in array holds %lld", (long long)need, (long long)SCRATCH_FLOATS);

    // set-up, once per device, with that device current
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return refuse((int)e, "cudaGetDevice failed (%lld)", (long long)e);
    if (dev < 0 || dev >= MAX_DEVICES) return refuse((int)cudaErrorInvalidDevice, "device index %lld out of range", dev);
    if (g_scratch_addr[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr)
            return refuse((int)(e != cudaSuccess ? e : cudaErrorUnknown), "cudaGetSymbolAddress failed (%lld)", (long long)e);
        g_scratch_addr[dev] = p;
    }
    float* part_o = g_scratch_addr[dev];
    float* part_ml = part_o + (size_t)T * nh * nsplit * hd;

#define ARGS (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_cache, \
             (const __nv_bfloat16*)v_cache, block_table, bt_width, positions, tok_seg, T, nh, nkv, page_size, \
             num_pages, window, scale, part_o, part_ml, nsplit, err, stream
    return hd == 64 ? prism::launch_decode<64>(ARGS) : prism::launch_decode<128>(ARGS);
#undef ARGS
}
