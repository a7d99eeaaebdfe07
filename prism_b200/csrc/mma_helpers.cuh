// Warp-level tensor-core and async-copy helpers shared by the bf16 attention
// kernels: m16n8k16 bf16 MMA with float32 accumulation, ldmatrix fragment
// loads, 16-byte cp.async, and a loader that gathers a tile of cache rows
// through a request's block table into padded shared memory.
#pragma once

#include "common.cuh"

namespace prism {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;      // src-size 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem)));
}

// d += a (16x16, row) * b (16x8, col), bf16 in, float32 accumulate
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Rows of a shared-memory tile are padded by 8 bf16 (16 bytes): with a row of
// HD bf16 (HD a multiple of 16) eight consecutive rows then start in eight
// different 16-byte bank groups, which is what ldmatrix needs.
template <int HD> struct TileRow { static constexpr int STRIDE = HD + 8; };

// Gather ROWS cache rows (keys first_key .. first_key + ROWS - 1 of one kv
// head) of both K and V into ks/vs[ROWS][HD + 8].  A row's offset in the cache
// is the same for K and V and is computed once.  Keys outside [lo, hi] are
// zero-filled.  A page id outside the pool is reported and the row
// zero-filled.  page_shift = log2(page_size) when that is a power of two, else -1.
// THREADS threads (a CTA or one warp) load together; tid is the caller's index among them.  Any head size
// that is a multiple of 8: the (row, 16-byte chunk) pairs are dealt out to the threads in turn.
template <int HD, int ROWS, int THREADS>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* ks, __nv_bfloat16* vs,
                                             const __nv_bfloat16* __restrict__ kcache,
                                             const __nv_bfloat16* __restrict__ vcache,
                                             const int* __restrict__ bt, int first_key, int lo, int hi,
                                             int page_size, int page_shift, int num_pages, int nkv, int kvh,
                                             int* err, int tid) {
    constexpr int CHUNKS = HD / 8;                 // 16-byte chunks per row
    constexpr int ITEMS = ROWS * CHUNKS;           // (row, chunk) pairs, dealt out to the threads in turn
    const size_t row_elems = (size_t)nkv * HD;
    const size_t head_off = (size_t)kvh * HD;
    // Fast path: a tile that lies in one page and wholly inside [lo, hi]: one table lookup, then
    // rows at a constant stride.
    if (page_shift >= 0 && (first_key >> page_shift) == ((first_key + ROWS - 1) >> page_shift) && first_key >= lo &&
        first_key + ROWS - 1 <= hi) {
        const int page = bt[first_key >> page_shift];
        if (page >= 0 && page < num_pages) {
            const size_t base = ((size_t)page * page_size + (first_key & (page_size - 1))) * row_elems + head_off;
#pragma unroll
            for (int i = tid; i < ITEMS; i += THREADS) {
                const int r = i / CHUNKS, c = i % CHUNKS;
                cp_async16(ks + r * TileRow<HD>::STRIDE + c * 8, kcache + base + (size_t)r * row_elems + c * 8, true);
                cp_async16(vs + r * TileRow<HD>::STRIDE + c * 8, vcache + base + (size_t)r * row_elems + c * 8, true);
            }
            return;
        }
    }
#pragma unroll
    for (int i = tid; i < ITEMS; i += THREADS) {
        const int r = i / CHUNKS, c = i % CHUNKS;
        const int key = first_key + r;
        bool valid = key >= lo && key <= hi;
        size_t off = 0;
        if (valid) {
            int page, in_page;
            if (page_shift >= 0) {
                page = bt[key >> page_shift];
                in_page = key & (page_size - 1);
            } else {
                page = bt[key / page_size];
                in_page = key % page_size;
            }
            if (page < 0 || page >= num_pages) {
                report_error(err, PRISM_ERR_PAGE_RANGE);
                valid = false;
            } else {
                off = ((size_t)page * page_size + in_page) * row_elems + head_off + c * 8;
            }
        }
        cp_async16(ks + r * TileRow<HD>::STRIDE + c * 8, kcache + off, valid);
        cp_async16(vs + r * TileRow<HD>::STRIDE + c * 8, vcache + off, valid);
    }
}

}  // namespace prism
