// bf16 paged causal grouped-query attention on tensor cores, two kernels:
//
//  * decode: one new token per request.  A CTA takes one (token, kv head,
//    split of the keys); the nh/nkv query heads of that kv head form the rows
//    of one 16-row MMA tile, so a K/V tile is read once for all of them.  Four
//    warps each take 16 of a tile's 64 keys; partial (max, sum, output) of the
//    warps are merged in shared memory, those of the splits by a second small
//    kernel.
//  * prefill / portions: a CTA takes 64 query rows of one head of one
//    segment; keys come from the request's pages (earlier portions and this
//    one), causal with the portion's offset: the row at position p sees keys
//    <= p (and > p - window).
//
// Both compute what flash_attn_with_kvcache(causal=True) computes in
// andre-fu/prism (engine/executor.py:119-120,151-153): scale hd^-1/2, scores,
// running max and sum and output accumulation in float32, probabilities
// rounded to bf16 for the PV product.  K/V tiles of 64 keys are gathered
// through the block table with 16-byte cp.async (any page size) into padded
// shared memory, 3 stages deep (decode) or double-buffered (prefill).
#pragma once

#include "mma_helpers.cuh"

namespace prism {

constexpr int ATT_TILE = 64;       // keys per tile
constexpr int ATT_THREADS = 128;   // 4 warps
#ifndef PRISM_DEC_STAGES
#define PRISM_DEC_STAGES 3
#endif
constexpr int DEC_STAGES = PRISM_DEC_STAGES;
constexpr int DEC_MIN_TILES = 3;   // tiles a split keeps at least: shorter CTAs cost more in fixed latencies than they share
constexpr int PRE_STAGES = 2;
constexpr int PRE_ROWS = 64;       // query rows per CTA

__device__ __forceinline__ float exp2_guard(float x, float m) {   // exp2(x - m), 0 when x is -inf
    return x == -INFINITY ? 0.f : exp2f(x - m);
}
// exp2(x - m) for finite m: the hardware approximation (2 ulp), which gives 0 for x = -inf by itself
__device__ __forceinline__ float exp2_fast(float x, float m) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x - m));
    return y;
}

// ---------------------------------------------------------------------------
// decode
// ---------------------------------------------------------------------------
// FUSED: the kernel takes over the back half of the qkv projection.  The projection of a few tokens
// leaves float32 partial sums [ks, T, D] (D = (nh + 2 nkv) * HD, q | k | v); every CTA adds up, biases
// and rotates the query rows of its kv head itself, and the CTA whose keys end at the token's own
// position does the same for that token's key and value, stores them in the cache and puts them into
// its tile in shared memory.  One kernel and one grid boundary fewer in the decode step; nothing of
// the cache depends on the kernels before this one any more, so all tiles are requested ahead of the wait.
struct DecodeQKV {
    const float* parts;        // [ks, T, D] partial sums of the qkv projection
    size_t part_stride;        // T * D
    int ks, D;
    const void* bias;          // [D] or null
    int bias_bf16;
    const float2* table;       // [T, HD / 2] (cos, sin) of the step's positions
    __nv_bfloat16* kc;         // the cache planes, writable
    __nv_bfloat16* vc;
    int max_pos;
};

// 4 consecutive sums: bias + partial sums in the order s = 0, 1, ... (as rope_kv_partial_kernel adds them)
__device__ __forceinline__ void qkv_sum4(const DecodeQKV& f, const float* parts, int t, size_t col, float (&v)[4]) {
    if (f.bias != nullptr) {
        if (f.bias_bf16) {
            const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(f.bias) + col);
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
            v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
        } else {
            const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(f.bias) + col);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        }
    } else {
        v[0] = v[1] = v[2] = v[3] = 0.f;
    }
    const float* p0 = parts + (size_t)t * f.D + col;
    for (int s0 = 0; s0 < f.ks; s0 += 4) {
        float4 p[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (s0 + u < f.ks) p[u] = *reinterpret_cast<const float4*>(p0 + (size_t)(s0 + u) * f.part_stride);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (s0 + u < f.ks) { v[0] += p[u].x; v[1] += p[u].y; v[2] += p[u].z; v[3] += p[u].w; }
    }
}
// rotate the pairs (x1[e], x2[e]) by the angles tab[e] and round: 4 + 4 bf16
__device__ __forceinline__ void rotate4(const float (&x1)[4], const float (&x2)[4], const float2* tab, uint2& lo, uint2& hi) {
    const float4 t01 = reinterpret_cast<const float4*>(tab)[0], t23 = reinterpret_cast<const float4*>(tab)[1];
    const float c[4] = {t01.x, t01.z, t23.x, t23.z}, sn[4] = {t01.y, t01.w, t23.y, t23.w};
    float y1[4], y2[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        y1[e] = x1[e] * c[e] - x2[e] * sn[e];
        y2[e] = x2[e] * c[e] + x1[e] * sn[e];
    }
    lo = make_uint2(pack_bf16(y1[0], y1[1]), pack_bf16(y1[2], y1[3]));
    hi = make_uint2(pack_bf16(y2[0], y2[1]), pack_bf16(y2[2], y2[3]));
}

// Work items.  With `items` the grid is flat: CTA (x = kv head, y = item) takes items[y] = {token, split | used << 16,
// position, segment} - the host has shared every request's keys among `used` CTAs according to its own length
// (ops.decode_work_items), so that a long context among short ones gets many CTAs and a short one a single CTA,
// and no CTA of the step runs much longer than the others.  Items of one token are consecutive (the host may
// put the tokens in any order, e.g. the longest CTAs first); item y leaves its partial result in slot y, and a
// token with a single item writes its output itself.  token < 0: a place of the grid that this step does not use;
// the host puts those last, and with the item as the grid's slow dimension they are launched after all others.
// The items are part of the step's descriptor (complete before the step's first kernel); position and segment
// travel with them so that the CTA's first load is all it needs to find its keys.
template <int HD, bool FUSED = false>
__global__ void __launch_bounds__(ATT_THREADS)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                   const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                   const int* __restrict__ block_table, int bt_width,
                   const int* __restrict__ positions, const int* __restrict__ tok_seg, int nh,
                   int nkv, int page_size, int page_shift, int num_pages, int window, float scale_log2,
                   float* __restrict__ part_o, float* __restrict__ part_ml, int nsplit,
                   __nv_bfloat16* __restrict__ out, int out_stride, int* err, const DecodeQKV fq,
                   const int4* __restrict__ items) {
    __shared__ __align__(16) __nv_bfloat16 s_own_kv[FUSED ? 2 * HD : 8];     // FUSED: this step's own key and value
    constexpr int STRIDE = TileRow<HD>::STRIDE;
    constexpr int SUB_ELEMS = 16 * STRIDE;                           // one warp's 16 keys of a tile
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [16][STRIDE]
    __nv_bfloat16* KV = Qs + 16 * STRIDE;                            // [warp][stage][K|V][16][STRIDE]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = nh / nkv;
    int kvh, split, t, pos, seg, used = 0;
    if (items != nullptr) {
        const int4 it = items[blockIdx.y];
        if (it.x < 0) return;
        kvh = blockIdx.x, t = it.x, split = it.y & 0xffff, used = it.y >> 16, pos = it.z, seg = it.w;
    } else {
        split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
        pos = positions[t], seg = tok_seg[t];
    }
    const int* bt = block_table + (size_t)seg * bt_width;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int hi = pos;
    const int first_tile = lo / ATT_TILE, ntiles = hi / ATT_TILE - first_tile + 1;
    // without items nsplit is chosen for the longest context the launch may meet: a shorter one is shared
    // among fewer CTAs, DEC_MIN_TILES tiles each at least, and the rest leave empty partials
    const int per_split = items != nullptr ? (ntiles + used - 1) / used
                                           : max((ntiles + nsplit - 1) / nsplit, nsplit > 1 ? DEC_MIN_TILES : 1);
    const int t0 = first_tile + split * per_split;
    const int t1 = min(t0 + per_split, first_tile + ntiles);
    const bool direct = items != nullptr ? used == 1 : nsplit == 1;      // the only split: no partial and no merge

    // partial results [token][head][split]: without items every token has nsplit slots per head, with items the
    // token whose first item is f has its used * nh slots from slot f * nh on
    const size_t head0 = (size_t)kvh * g;
    const size_t prow = items != nullptr ? (size_t)used : (size_t)nsplit;      // slots between two heads' partials
    const size_t pslot = (items != nullptr ? (size_t)(blockIdx.y - split) * nh : (size_t)t * nh * nsplit) + head0 * prow + split;
    float* po = part_o + pslot * HD;        // + row * prow * HD
    float* pml = part_ml + pslot * 2;       // + row * prow * 2
    if (t0 >= t1) {                       // nothing for this split: an empty partial
        pdl_wait();
        for (int i = tid; i < g * HD; i += ATT_THREADS) po[(size_t)(i / HD) * prow * HD + i % HD] = 0.f;
        for (int r = tid; r < g; r += ATT_THREADS) {
            pml[(size_t)r * prow * 2] = -INFINITY;
            pml[(size_t)r * prow * 2 + 1] = 0.f;
        }
        pdl_trigger_gemm();
        return;
    }

    // Keys and values of earlier steps are in the cache already; only the tile that holds this
    // step's own position (written by the kernel before this one) and q must wait for the kernels
    // before this one.  Everything else is requested at once, while those kernels still run.
    const int own_tile = hi / ATT_TILE;
    bool waited = false;
    auto load_tile = [&](int tile, int stage) {
        if (!FUSED && tile == own_tile && !waited) {
            pdl_wait();
            waited = true;
        }
        // each warp streams the 16 keys of the tile that it will multiply, into stages of its own:
        // the warps of a CTA never wait for one another inside the loop
        __nv_bfloat16* ks = KV + ((size_t)(warp * DEC_STAGES + stage) * 2) * SUB_ELEMS;
        load_kv_tile<HD, 16, 32>(ks, ks + SUB_ELEMS, kc, vc, bt, tile * ATT_TILE + warp * 16, lo, hi, page_size,
                                 page_shift, num_pages, nkv, kvh, err, lane);
    };
#pragma unroll
    for (int s = 0; s < DEC_STAGES - 1; ++s) {
        if (t0 + s < t1) load_tile(t0 + s, s);
        cp_async_commit();
    }
    if (!waited) {
        pdl_wait();
        waited = true;
    }
    // Q rows of this kv head's group (rows >= g are zero), with plain loads: visible after the
    // first barrier of the loop below
    // FUSED: this CTA holds the token's own position as its last key
    const bool owner = FUSED && t0 < t1 && t1 == own_tile + 1;
    if (FUSED) {
        constexpr int HALF = HD / 2;
        const float* parts = pdl_fresh(fq.parts);            // the projection's partial sums and the step's angles:
        const float2* tab = pdl_fresh(fq.table) + (size_t)t * HALF;      // outputs of kernels before this one
        for (int i = tid; i < (16 - g) * (HD / 8); i += ATT_THREADS)
            *reinterpret_cast<uint4*>(Qs + (g + i / (HD / 8)) * STRIDE + (i % (HD / 8)) * 8) = make_uint4(0u, 0u, 0u, 0u);
        for (int i = tid; i < g * (HALF / 4); i += ATT_THREADS) {
            const int r = i / (HALF / 4), j = (i % (HALF / 4)) * 4;
            const size_t col = ((size_t)kvh * g + r) * HD + j;
            float x1[4], x2[4];
            qkv_sum4(fq, parts, t, col, x1);
            qkv_sum4(fq, parts, t, col + HALF, x2);
            uint2 a, b;
            rotate4(x1, x2, tab + j, a, b);
            *reinterpret_cast<uint2*>(Qs + r * STRIDE + j) = a;
            *reinterpret_cast<uint2*>(Qs + r * STRIDE + j + HALF) = b;
        }
        if (owner) {
            // the token's own key (rotated) and value: into the cache for later steps, and into shared
            // memory for this one
            const bool pos_ok = pos >= 0 && pos < fq.max_pos;
            const int page = pos_ok ? bt[page_shift >= 0 ? pos >> page_shift : pos / page_size] : -1;
            const bool store = pos_ok && page >= 0 && page < num_pages;
            if (!store && tid == 0) report_error(err, pos_ok ? PRISM_ERR_PAGE_RANGE : PRISM_ERR_POSITION_RANGE);
            const int in_page = pos_ok ? (page_shift >= 0 ? pos & (page_size - 1) : pos % page_size) : 0;
            const size_t slot = store ? ((size_t)page * page_size + in_page) * (size_t)nkv * HD + (size_t)kvh * HD : 0;
            for (int i = tid; i < HALF / 4 + HD / 4; i += ATT_THREADS) {
                if (i < HALF / 4) {
                    const int j = i * 4;
                    const size_t col = (size_t)nh * HD + (size_t)kvh * HD + j;
                    float x1[4], x2[4];
                    qkv_sum4(fq, parts, t, col, x1);
                    qkv_sum4(fq, parts, t, col + HALF, x2);
                    uint2 a, b;
                    rotate4(x1, x2, tab + j, a, b);
                    *reinterpret_cast<uint2*>(s_own_kv + j) = a;
                    *reinterpret_cast<uint2*>(s_own_kv + j + HALF) = b;
                    if (store) {
                        *reinterpret_cast<uint2*>(fq.kc + slot + j) = a;
                        *reinterpret_cast<uint2*>(fq.kc + slot + j + HALF) = b;
                    }
                } else {
                    const int d = (i - HALF / 4) * 4;
                    const size_t col = (size_t)(nh + nkv) * HD + (size_t)kvh * HD + d;
                    float x[4];
                    qkv_sum4(fq, parts, t, col, x);
                    const uint2 a = make_uint2(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]));
                    *reinterpret_cast<uint2*>(s_own_kv + HD + d) = a;
                    if (store) *reinterpret_cast<uint2*>(fq.vc + slot + d) = a;
                }
            }
        }
    } else {
        const __nv_bfloat16* q_now = pdl_fresh(q);       // q is the previous kernel's output
        for (int i = tid; i < 16 * (HD / 8); i += ATT_THREADS) {
            const int r = i / (HD / 8), c = i % (HD / 8);
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < g) v = *reinterpret_cast<const uint4*>(q_now + (size_t)t * q_stride + ((size_t)kvh * g + r) * HD + c * 8);
            *reinterpret_cast<uint4*>(Qs + r * STRIDE + c * 8) = v;
        }
    }
    __syncthreads();

    uint32_t qf[HD / 16][4];
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int mat = lane >> 3, lr = lane & 7;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(qf[ks], Qs + (lr + (mat & 1) * 8) * STRIDE + ks * 16 + (mat >> 1) * 8);

    for (int tile = t0; tile < t1; ++tile) {
        const int it = tile - t0;
        if (tile + DEC_STAGES - 1 < t1) load_tile(tile + DEC_STAGES - 1, (it + DEC_STAGES - 1) % DEC_STAGES);
        cp_async_commit();
        cp_async_wait<DEC_STAGES - 1>();
        __syncwarp();
        const __nv_bfloat16* Ks = KV + ((size_t)(warp * DEC_STAGES + it % DEC_STAGES) * 2) * SUB_ELEMS;
        const __nv_bfloat16* Vs = Ks + SUB_ELEMS;
        if (FUSED && owner && tile == own_tile && warp == ((pos & (ATT_TILE - 1)) >> 4)) {
            // the row of the token's own position: what the cache gave for it is stale, the computed
            // key and value take its place
            __nv_bfloat16* krow = KV + ((size_t)(warp * DEC_STAGES + it % DEC_STAGES) * 2) * SUB_ELEMS + (pos & 15) * STRIDE;
            for (int c = lane; c < 2 * (HD / 8); c += 32) {
                const int which = c / (HD / 8), cc = c % (HD / 8);
                *reinterpret_cast<uint4*>(krow + which * SUB_ELEMS + cc * 8) =
                    *reinterpret_cast<const uint4*>(s_own_kv + which * HD + cc * 8);
            }
            __syncwarp();
        }
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};     // odd k-steps: two shorter MMA chains
#pragma unroll
        for (int ks = 0; ks + 1 < HD / 16; ks += 2) {
            uint32_t b[4], b2[4];
            ldmatrix_x4(b, Ks + ((mat >> 1) * 8 + lr) * STRIDE + ks * 16 + (mat & 1) * 8);
            ldmatrix_x4(b2, Ks + ((mat >> 1) * 8 + lr) * STRIDE + (ks + 1) * 16 + (mat & 1) * 8);
            mma_bf16_16816(s[0], qf[ks], b[0], b[1]);
            mma_bf16_16816(s[1], qf[ks], b[2], b[3]);
            mma_bf16_16816(s2[0], qf[ks + 1], b2[0], b2[1]);
            mma_bf16_16816(s2[1], qf[ks + 1], b2[2], b2[3]);
        }
        if ((HD / 16) & 1) {                      // an odd number of 16-wide k-steps (head sizes 16, 48, 80, 112): the last one
            constexpr int ks = HD / 16 - 1;
            uint32_t b[4];
            ldmatrix_x4(b, Ks + ((mat >> 1) * 8 + lr) * STRIDE + ks * 16 + (mat & 1) * 8);
            mma_bf16_16816(s[0], qf[ks], b[0], b[1]);
            mma_bf16_16816(s[1], qf[ks], b[2], b[3]);
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] += s2[nt][e];
        // mask (only a tile that crosses lo or hi needs it), scale, online softmax over this warp's
        // 16 keys (rows lane/4 and lane/4 + 8)
        const int key0 = tile * ATT_TILE + warp * 16 + (lane & 3) * 2;
        const bool edge = tile * ATT_TILE < lo || tile * ATT_TILE + ATT_TILE - 1 > hi;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + nt * 8 + (e & 1);
                const float v = (!edge || (key >= lo && key <= hi)) ? s[nt][e] * scale_log2 : -INFINITY;
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float corr[2], mu[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            mu[r] = m_new == -INFINITY ? 0.f : m_new;       // finite, so exp2_fast(-inf, mu) = 0
            corr[r] = exp2_fast(m_run[r], mu[r]);
            m_run[r] = m_new;
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p = exp2_fast(s[nt][e], mu[e >> 1]);
                s[nt][e] = p;
                l_run[e >> 1] += p;
            }
        uint32_t pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                          pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
        // the running maxima seldom move after the first tiles: rescale the output only when one did
        if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
            for (int j = 0; j < HD / 8; ++j) {
                o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1];
            }
        }
#pragma unroll
        for (int j = 0; j < HD / 16; ++j) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, Vs + ((mat & 1) * 8 + lr) * STRIDE + j * 16 + (mat >> 1) * 8);
            mma_bf16_16816(o[2 * j], pa, b[0], b[1]);
            mma_bf16_16816(o[2 * j + 1], pa, b[2], b[3]);
        }
        __syncwarp();       // the stage is free for this warp's next load
    }
    cp_async_wait<0>();
    pdl_trigger_gemm();     // the keys are read: the next kernel may start its prologue
    __syncthreads();        // every warp is out of its loop: the stage buffers become merge scratch

    // merge the four warps' partials through shared memory
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    float* red_o = reinterpret_cast<float*>(KV);                 // [4][16][HD]
    float* red_m = red_o + 4 * 16 * HD;                          // [4][16]
    float* red_l = red_m + 4 * 16;                               // [4][16]
    const int r0 = lane >> 2;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
        const int d = nt * 8 + (lane & 3) * 2;
        float* w0 = red_o + ((size_t)warp * 16 + r0) * HD + d;
        w0[0] = o[nt][0]; w0[1] = o[nt][1];
        w0[8 * HD] = o[nt][2]; w0[8 * HD + 1] = o[nt][3];
    }
    if ((lane & 3) == 0) {
        red_m[warp * 16 + r0] = m_run[0]; red_m[warp * 16 + r0 + 8] = m_run[1];
        red_l[warp * 16 + r0] = l_run[0]; red_l[warp * 16 + r0 + 8] = l_run[1];
    }
    __syncthreads();
    for (int i = tid; i < g * HD; i += ATT_THREADS) {
        const int r = i / HD, d = i % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, red_m[w * 16 + r]);
        const float Mu = M == -INFINITY ? 0.f : M;
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = exp2_guard(red_m[w * 16 + r], Mu);
            acc += red_o[((size_t)w * 16 + r) * HD + d] * f;
            L += red_l[w * 16 + r] * f;
        }
        if (direct) {
            out[(size_t)t * out_stride + ((size_t)kvh * g + r) * HD + d] = __float2bfloat16_rn(L > 0.f ? acc * (1.f / L) : 0.f);
        } else {
            po[(size_t)r * prow * HD + d] = acc;
            if (d == 0) {
                pml[(size_t)r * prow * 2] = M;
                pml[(size_t)r * prow * 2 + 1] = L;
            }
        }
    }
}

// merge the splits: out[t, h, :] = sum_s o_s * 2^(m_s - M) / sum_s l_s * 2^(m_s - M)
// One CTA per (token, head), one thread per output element.  The kernel is all latency (a few KB per CTA), so
// it makes as few dependent trips to memory as it can: every thread asks for its first MERGE_BATCH partial
// outputs at once, before anything is known about their weights; meanwhile the first warp fetches all
// (max, sum) pairs in one round, reduces them with shuffles and leaves one weight per split in shared memory.
constexpr int MERGE_BATCH = 16;
constexpr int MERGE_MAX_SPLITS = 256;      // weights kept in shared memory; more splits than this take the slow loop

// `starts` (the decode kernel ran on work items): token t has `used` items from item `first` on, starts[t] =
// first | used << 16, and its partials [head][split] lie from slot first * nh on; a token with one item has its
// output already.  Without: [token][head][cap].
template <int HD>
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  int cap, __nv_bfloat16* __restrict__ out, int out_stride, int nh,
                                  const int* __restrict__ starts) {
    __shared__ float s_w[MERGE_MAX_SPLITS];
    __shared__ float s_inv;
    pdl_trigger();
    const int t = blockIdx.x / nh, h = blockIdx.x % nh;
    int nsplit = cap;
    size_t first = (size_t)blockIdx.x * cap;                    // slot of split 0
    if (starts != nullptr) {
        const int s0 = starts[t] & 0xffff;
        nsplit = starts[t] >> 16;
        if (nsplit <= 1) return;
        first = (size_t)s0 * nh + (size_t)h * nsplit;
    }
    pdl_wait();
    const float* po = pdl_fresh(part_o) + first * HD;          // the attention kernel's output
    const float* pml = pdl_fresh(part_ml) + first * 2;
    constexpr size_t ostep = HD, mstep = 2;
    // blockDim.x: HD rounded up to whole warps; a thread beyond HD (head sizes 16, 48, 80, 112) works on element
    // 0 again and stores nothing
    const bool mine = (int)threadIdx.x < HD;
    const int d = mine ? threadIdx.x : 0;
    if (nsplit > MERGE_MAX_SPLITS) {
        float M = -INFINITY;
        for (int s = 0; s < nsplit; ++s) M = fmaxf(M, pml[mstep * s]);
        const float Mu = M == -INFINITY ? 0.f : M;
        float L = 0.f, acc = 0.f;
        for (int s = 0; s < nsplit; ++s) {
            const float f = exp2_guard(pml[mstep * s], Mu);
            L += pml[mstep * s + 1] * f;
            acc += po[ostep * s + d] * f;
        }
        if (mine) out[(size_t)t * out_stride + h * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        return;
    }
    float v[MERGE_BATCH];
#pragma unroll
    for (int i = 0; i < MERGE_BATCH; ++i) v[i] = i < nsplit ? po[ostep * i + d] : 0.f;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float2 mine[MERGE_MAX_SPLITS / 32];
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < MERGE_MAX_SPLITS / 32; ++i) {
            const int s = lane + 32 * i;
            mine[i] = s < nsplit ? *reinterpret_cast<const float2*>(pml + mstep * s) : make_float2(-INFINITY, 0.f);
            M = fmaxf(M, mine[i].x);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        const float Mu = M == -INFINITY ? 0.f : M;
        float L = 0.f;
#pragma unroll
        for (int i = 0; i < MERGE_MAX_SPLITS / 32; ++i) {
            const int s = lane + 32 * i;
            const float f = exp2_guard(mine[i].x, Mu);
            if (s < nsplit) s_w[s] = f;
            L += mine[i].y * f;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
        if (lane == 0) s_inv = L > 0.f ? 1.f / L : 0.f;
    }
    __syncthreads();
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < MERGE_BATCH; ++i)
        if (i < nsplit) acc += v[i] * s_w[i];
    for (int s0 = MERGE_BATCH; s0 < nsplit; s0 += MERGE_BATCH) {
        // splits that saw no key (a launch sized for a longer context) have weight 0: nothing is asked of them
#pragma unroll
        for (int i = 0; i < MERGE_BATCH; ++i)
            v[i] = (s0 + i < nsplit && s_w[s0 + i] != 0.f) ? po[ostep * (s0 + i) + d] : 0.f;
#pragma unroll
        for (int i = 0; i < MERGE_BATCH; ++i)
            if (s0 + i < nsplit) acc += v[i] * s_w[s0 + i];
    }
    if (mine) out[(size_t)t * out_stride + h * HD + d] = __float2bfloat16_rn(acc * s_inv);
}

// ---------------------------------------------------------------------------
// prefill / portions
// ---------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(ATT_THREADS, 3)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                    int out_stride, const __nv_bfloat16* __restrict__ kc,
                    const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_table,
                    int bt_width, const int* __restrict__ seg_start, const int* __restrict__ cached_len,
                    int nh, int nkv, int page_size, int page_shift, int num_pages, int window, float scale_log2,
                    int* err) {
    pdl_trigger();
    pdl_wait();
    constexpr int STRIDE = TileRow<HD>::STRIDE;
    constexpr int TILE_ELEMS = ATT_TILE * STRIDE;
    const int seg = blockIdx.z, h = blockIdx.y;
    const int s0 = seg_start[seg], qlen = seg_start[seg + 1] - s0;
    // later query tiles see more keys: they are started first so that no SM is left with a long tile at the end
    const int q0 = (gridDim.x - 1 - blockIdx.x) * PRE_ROWS;
    if (q0 >= qlen) return;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* KV = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [stage][K|V][64][STRIDE]
    __nv_bfloat16* Qs = KV + 2 * TILE_ELEMS;                         // q passes through stage 1's K buffer on its
                                                                     // way to registers, before that stage is first used

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rows = min(PRE_ROWS, qlen - q0);
    const int tok0 = s0 + q0;
    const int pos0 = cached_len[seg] + q0;
    const int kvh = h / (nh / nkv);
    const int* bt = block_table + (size_t)seg * bt_width;
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int hi = pos0 + rows - 1;
    const int t0 = lo / ATT_TILE, t1 = hi / ATT_TILE + 1;

    for (int i = tid; i < PRE_ROWS * (HD / 8); i += ATT_THREADS) {
        const int r = i / (HD / 8), c = i % (HD / 8);
        const bool valid = r < rows;
        cp_async16(Qs + r * STRIDE + c * 8, q + (size_t)(tok0 + (valid ? r : 0)) * q_stride + (size_t)h * HD + c * 8, valid);
    }
    auto load_tile = [&](int tile, int stage) {
        __nv_bfloat16* ks = KV + (size_t)stage * 2 * TILE_ELEMS;
        load_kv_tile<HD, ATT_TILE, ATT_THREADS>(ks, ks + TILE_ELEMS, kc, vc, bt, tile * ATT_TILE, lo, hi, page_size,
                                                page_shift, num_pages, nkv, kvh, err, threadIdx.x);
    };
    cp_async_commit();
    load_tile(t0, 0);
    cp_async_commit();

    uint32_t qf[HD / 16][4];
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int mat = lane >> 3, lr = lane & 7;
    const int p_row[2] = {pos0 + warp * 16 + (lane >> 2), pos0 + warp * 16 + (lane >> 2) + 8};
    cp_async_wait<1>();            // q has landed (the first tile may still be on its way)
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(qf[ks], Qs + (warp * 16 + lr + (mat & 1) * 8) * STRIDE + ks * 16 + (mat >> 1) * 8);
    __syncthreads();               // stage 1 may now receive the second tile

    for (int tile = t0; tile < t1; ++tile) {
        const int it = tile - t0;
        if (tile + 1 < t1) load_tile(tile + 1, (it + 1) % PRE_STAGES);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const __nv_bfloat16* Ks = KV + (size_t)(it % PRE_STAGES) * 2 * TILE_ELEMS;
        const __nv_bfloat16* Vs = Ks + TILE_ELEMS;
        // a warp whose 16 rows all sit before this tile's first key has nothing to do here
        const bool warp_active = tile * ATT_TILE <= pos0 + warp * 16 + 15;
        if (warp_active) {
            float s[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t b[4];
                    ldmatrix_x4(b, Ks + (np * 16 + (mat >> 1) * 8 + lr) * STRIDE + ks * 16 + (mat & 1) * 8);
                    mma_bf16_16816(s[2 * np], qf[ks], b[0], b[1]);
                    mma_bf16_16816(s[2 * np + 1], qf[ks], b[2], b[3]);
                }
            }
            const int key0 = tile * ATT_TILE + (lane & 3) * 2;
            // only a tile that crosses the diagonal, the window's edge or the first key needs the mask
            const int row_lo = pos0 + warp * 16, row_hi = row_lo + 15;
            const bool edge = tile * ATT_TILE + ATT_TILE - 1 > row_lo || tile * ATT_TILE < lo ||
                              (window > 0 && tile * ATT_TILE <= row_hi - window);
            float mx[2] = {-INFINITY, -INFINITY};
            if (edge) {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + nt * 8 + (e & 1);
                        const int p = p_row[e >> 1];
                        const bool vis = key <= p && key >= lo && (window <= 0 || key > p - window);
                        const float v = vis ? s[nt][e] * scale_log2 : -INFINITY;
                        s[nt][e] = v;
                        mx[e >> 1] = fmaxf(mx[e >> 1], v);
                    }
            } else {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float v = s[nt][e] * scale_log2;
                        s[nt][e] = v;
                        mx[e >> 1] = fmaxf(mx[e >> 1], v);
                    }
            }
            float corr[2], mu[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                mu[r] = m_new == -INFINITY ? 0.f : m_new;       // finite, so exp2_fast(-inf, mu) = 0
                corr[r] = exp2_fast(m_run[r], mu[r]);
                m_run[r] = m_new;
                l_run[r] *= corr[r];
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = exp2_fast(s[nt][e], mu[e >> 1]);
                    s[nt][e] = p;
                    l_run[e >> 1] += p;
                }
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t pa[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                                  pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
                for (int j = 0; j < HD / 16; ++j) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, Vs + (kk * 16 + (mat & 1) * 8 + lr) * STRIDE + j * 16 + (mat >> 1) * 8);
                    mma_bf16_16816(o[2 * j], pa, b[0], b[1]);
                    mma_bf16_16816(o[2 * j + 1], pa, b[2], b[3]);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
    const int r0 = warp * 16 + (lane >> 2);
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
        const int d = nt * 8 + (lane & 3) * 2;
        if (r0 < rows)
            *reinterpret_cast<uint32_t*>(out + (size_t)(tok0 + r0) * out_stride + (size_t)h * HD + d) =
                pack_bf16(o[nt][0] * inv0, o[nt][1] * inv0);
        if (r0 + 8 < rows)
            *reinterpret_cast<uint32_t*>(out + (size_t)(tok0 + r0 + 8) * out_stride + (size_t)h * HD + d) =
                pack_bf16(o[nt][2] * inv1, o[nt][3] * inv1);
    }
}

inline int page_shift_of(int page_size) {
    if (page_size <= 0 || (page_size & (page_size - 1))) return -1;
    int s = 0;
    while ((1 << s) < page_size) ++s;
    return s;
}

template <int HD> constexpr size_t dec_smem() {
    return (size_t)(16 + DEC_STAGES * 2 * ATT_TILE) * TileRow<HD>::STRIDE * sizeof(__nv_bfloat16);
}
template <int HD> constexpr size_t pre_smem() {
    return (size_t)(PRE_STAGES * 2 * ATT_TILE) * TileRow<HD>::STRIDE * sizeof(__nv_bfloat16);
}

template <int HD>
int launch_decode(const __nv_bfloat16* q, int q_stride, __nv_bfloat16* out, int out_stride,
                  const __nv_bfloat16* kc, const __nv_bfloat16* vc, const int* bt, int bt_width,
                  const int* positions, const int* tok_seg, int T, int nh, int nkv, int page_size,
                  int num_pages, int window, float scale, float* part_o, float* part_ml, int nsplit,
                  int* err, cudaStream_t stream, const DecodeQKV* fused = nullptr, const int* items = nullptr,
                  const int* starts = nullptr, int n_items = 0) {
    // with work items: a flat grid of n_items CTAs per kv head; nsplit is then the most items a token has
    static_assert(dec_smem<HD>() >= (size_t)(4 * 16 * HD + 128) * sizeof(float), "merge scratch must fit");
    dim3 grid(items != nullptr ? nkv : nsplit, items != nullptr ? n_items : nkv, items != nullptr ? 1 : T);
    auto kern = fused != nullptr ? attn_decode_kernel<HD, true> : attn_decode_kernel<HD, false>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dec_smem<HD>());
    cudaError_t rc = launch_kernel(kern, grid, dim3(ATT_THREADS), dec_smem<HD>(), stream, q, q_stride, kc, vc, bt, bt_width,
                                   positions, tok_seg, nh, nkv, page_size, page_shift_of(page_size), num_pages, window,
                                   scale * 1.4426950408889634f, part_o, part_ml, nsplit, out, out_stride, err,
                                   fused != nullptr ? *fused : DecodeQKV(), reinterpret_cast<const int4*>(items));
    if (rc != cudaSuccess || nsplit == 1) return (int)rc;
    return (int)launch_kernel(attn_merge_kernel<HD>, dim3(T * nh), dim3((HD + 31) / 32 * 32), 0, stream,
                              (const float*)part_o, (const float*)part_ml, nsplit, out, out_stride, nh,
                              items != nullptr ? starts : (const int*)nullptr);
}

template <int HD>
int launch_prefill(const __nv_bfloat16* q, int q_stride, __nv_bfloat16* out, int out_stride,
                   const __nv_bfloat16* kc, const __nv_bfloat16* vc, const int* bt, int bt_width,
                   const int* seg_start, const int* cached_len, int S, int max_q_len, int nh, int nkv,
                   int page_size, int num_pages, int window, float scale, int* err, cudaStream_t stream) {
    auto kern = attn_prefill_kernel<HD>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pre_smem<HD>());
    dim3 grid((max_q_len + PRE_ROWS - 1) / PRE_ROWS, nh, S);
    kern<<<grid, ATT_THREADS, pre_smem<HD>(), stream>>>(q, q_stride, out, out_stride, kc, vc, bt, bt_width, seg_start,
                                                        cached_len, nh, nkv, page_size, page_shift_of(page_size),
                                                        num_pages, window,
                                                        scale * 1.4426950408889634f, err);
    return (int)cudaPeekAtLastError();
}

}  // namespace prism

