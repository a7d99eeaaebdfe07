// Causal grouped-query attention over the paged cache for portions of prompts, on the
// 5th-generation tensor cores (the F.scaled_dot_product_attention call of andre-fu/prism's
// prefill, engine/executor.py:118-122, here reading keys and values from the pages).
//
// One CTA owns 128 query rows of one head and walks the keys in tiles of 64:
//
//   warp 0     TMA producer: the Q tile once, then K and V tiles (found through the block
//              table) into two-stage rings, 128-byte swizzle
//   warp 1     one thread issues tcgen05.mma:  S = Q K^T  (operands from shared memory, the
//              accumulator in tensor memory, two S buffers) and  O += P V  (P read from tensor
//              memory, V straight from its [key][head dim] rows as an MN-major operand)
//   warps 2-5  softmax: thread r owns query row r = tensor-memory lane r, so the row maximum
//              and sum need no shuffles; it reads its 64 scores with tcgen05.ld, writes the
//              bf16 probabilities over them with tcgen05.st, and rescales its row of O only
//              when the running maximum moved
//
// S of tile j+1 is computed while the softmax of tile j runs; two CTAs share an SM (256 of the
// 512 tensor-memory columns and 97 KB of shared memory each), so one CTA's prologue and
// epilogue hide behind the other's loop.  Softmax, the running maximum and sum, and the
// accumulators are float32; the scores never leave the SM.
//
// Rows of V beyond the last visible key (or before the window) are zeroed in shared memory
// before they are multiplied, so nothing unwritten in a page can reach the result.
// Every mbarrier wait is bounded; on expiry all roles leave through the common exit.
#include <cuda_bf16.h>

#include "tcgen05.cuh"

namespace prism {
namespace tca {

using namespace tc;

constexpr int BQ = 128;              // query rows per CTA (UMMA M)
constexpr int BK = 64;               // keys per tile
constexpr int THREADS = 192;
constexpr int STAGES = 2;
constexpr float RESCALE_STEP = 8.f;  // log2 units

template <int HD> struct ACfg {
    static constexpr int HALVES = HD / 64;                       // 64-column (128-byte) boxes per row
    static constexpr int Q_BYTES = BQ * HD * 2;
    static constexpr int KV_BYTES = BK * HD * 2;                 // one K or V tile
    static constexpr int TMEM_COLS = 256;                        // S0, S1 (64 each), O (HD <= 128)
    static constexpr int O_COL = 2 * BK;
    static constexpr size_t SMEM = (size_t)Q_BYTES + 2 * STAGES * KV_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
};

// MN-major operand with 128-byte swizzle: rows of 128 bytes along K (here: one key's 64 values),
// 8-row groups 1024 bytes apart, the next 64 values of the same keys `lbo` bytes further.
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t saddr, uint32_t lbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// D (+)= A B with A in tensor memory
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two float32 in one 64-bit register and the packed arithmetic of sm_100 on them: one instruction where the
// softmax would otherwise issue two (its warps are short of issue slots, not of arithmetic throughput).
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
    uint64_t v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
    return v;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, int out_stride,
                       const int* __restrict__ block_table, int bt_width, const int* __restrict__ seg_start,
                       const int* __restrict__ cached_len, int nh, int nkv, int page_size, int num_pages, int window,
                       float scale_log2, int* err, int nsplit, float* __restrict__ part_o, float* __restrict__ part_ml) {
    using C = ACfg<HD>;
    pdl_wait();
    // Heads vary fastest, and later query tiles (which see more keys) come first: the longest CTAs of
    // all heads start together and the short ones fill the gaps; the heads of one kv group walk the
    // same keys at the same time, so K and V are read from HBM once.
    // nsplit > 1 (a short portion against a long cache, too few query tiles to fill the GPU): the key
    // tiles of a query tile are shared among nsplit CTAs; each leaves (reference, sum, unnormalised
    // output) per row in part_ml / part_o, laid out as the decode kernel's partials, for the merge kernel.
    const int seg = blockIdx.z, h = blockIdx.x;
    const int s0 = seg_start[seg], qlen = seg_start[seg + 1] - s0;
    const int split = blockIdx.y % nsplit;
    const int q0 = (gridDim.y / nsplit - 1 - blockIdx.y / nsplit) * BQ;
    if (q0 >= qlen) return;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* Qs = tiles;                                   // [half][128 rows][128 B]
    unsigned char* Ks = Qs + C::Q_BYTES;                         // [stage][half][64 keys][128 B]
    unsigned char* Vs = Ks + STAGES * C::KV_BYTES;               // [stage][half][64 keys][128 B]
    uint64_t* bars = reinterpret_cast<uint64_t*>(Vs + STAGES * C::KV_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;      // [2]
    uint64_t* k_empty = bars + 3;     // [2]
    uint64_t* v_full = bars + 5;      // [2]
    uint64_t* v_empty = bars + 7;     // [2]
    uint64_t* s_full = bars + 9;      // [2]
    uint64_t* p_full = bars + 11;     // [2]
    uint64_t* pv_done = bars + 13;    // [2], by tile parity; a phase per P V product: O may be rescaled
    uint64_t* o_done = bars + 15;     // one phase: the last P V product is complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows = min(BQ, qlen - q0);
    const int tok0 = s0 + q0;
    const int pos0 = cached_len[seg] + q0;
    const int kvh = h / (nh / nkv);
    const int* bt = block_table + (size_t)seg * bt_width;
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;     // first key any row sees
    const int hi = pos0 + rows - 1;                                                   // last key any row sees
    int t0 = lo / BK, n = hi / BK + 1 - t0;
    if (nsplit > 1) {
        const int per = (n + nsplit - 1) / nsplit;
        t0 += split * per;
        n = min(per, n - split * per);
        if (n <= 0) {                 // no key tile for this split: an empty partial
            for (int i = threadIdx.x; i < rows * HD; i += THREADS)
                part_o[(((size_t)(tok0 + i / HD) * nh + h) * nsplit + split) * HD + i % HD] = 0.f;
            for (int r = threadIdx.x; r < rows; r += THREADS) {
                float* ml = part_ml + (((size_t)(tok0 + r) * nh + h) * nsplit + split) * 2;
                ml[0] = -INFINITY;
                ml[1] = 0.f;
            }
            return;
        }
    }

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1); mbar_init(&p_full[s], 128);
        }
        mbar_init(&pv_done[0], 1);
        mbar_init(&pv_done[1], 1);
        mbar_init(o_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(C::TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    volatile int* abortp = &abort_flag;
    // Dependents may start from here on, not earlier: this CTA holds its tensor memory now, so a
    // dependent CTA that allocates tensor memory and then waits for this grid cannot starve it.
    pdl_trigger();

    if (warp == 0) {
        // ---- TMA producer ---------------------------------------------------------
        if (lane == 0) {
            mbar_expect_tx(q_full, C::Q_BYTES);
#pragma unroll
            for (int hh = 0; hh < C::HALVES; ++hh) tma_load_2d(Qs + hh * BQ * 128, &map_q, q_full, h * HD + hh * 64, tok0);
            int issued = 0;
            for (int j = 0; j < n; ++j) {
                const int s = j % STAGES;
                const int key0 = (t0 + j) * BK;
                int page = bt[key0 / page_size];
                if (page < 0 || page >= num_pages) {
                    report_error(err, PRISM_ERR_PAGE_RANGE);
                    page = 0;                                    // the result is flagged; read something that exists
                }
                const int row = page * page_size + key0 % page_size;
                if (j >= STAGES && !mbar_wait(&k_empty[s], ((j / STAGES) - 1) & 1, abortp)) break;
                mbar_expect_tx(&k_full[s], C::KV_BYTES);
#pragma unroll
                for (int hh = 0; hh < C::HALVES; ++hh)
                    tma_load_2d(Ks + s * C::KV_BYTES + hh * BK * 128, &map_k, &k_full[s], kvh * HD + hh * 64, row);
                if (j >= STAGES && !mbar_wait(&v_empty[s], ((j / STAGES) - 1) & 1, abortp)) break;
                mbar_expect_tx(&v_full[s], C::KV_BYTES);
#pragma unroll
                for (int hh = 0; hh < C::HALVES; ++hh)
                    tma_load_2d(Vs + s * C::KV_BYTES + hh * BK * 128, &map_v, &v_full[s], kvh * HD + hh * 64, row);
                issued = j + 1;
            }
            if (*abortp) {
                // give the copies already in flight a bounded chance to land before the CTA's memory is reused
                mbar_wait(q_full, 0, abortp);
                for (int j = max(0, issued - STAGES); j < issued; ++j) {
                    mbar_wait(&k_full[j % STAGES], (j / STAGES) & 1, abortp);
                    mbar_wait(&v_full[j % STAGES], (j / STAGES) & 1, abortp);
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue ------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BK >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
            constexpr uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) /* B is MN-major */ |
                                          ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
            const uint32_t q_addr = smem_addr(Qs), k_addr = smem_addr(Ks), v_addr = smem_addr(Vs);
            bool ok = mbar_wait(q_full, 0, abortp);
            for (int j = 0; j <= n && ok; ++j) {
                if (j < n) {
                    const int s = j % STAGES;
                    ok = mbar_wait(&k_full[s], (j / STAGES) & 1, abortp);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < HD / UMMA_K; ++k) {
                        const int hh = k / 4, kk = k % 4;
                        const uint64_t da = umma_desc(q_addr + hh * BQ * 128) + (uint64_t)(kk * 2);
                        const uint64_t db = umma_desc(k_addr + s * C::KV_BYTES + hh * BK * 128) + (uint64_t)(kk * 2);
                        umma_bf16(tmem_base + s * BK, da, db, idesc_s, k > 0 ? 1u : 0u);
                    }
                    umma_commit(&k_empty[s]);
                    umma_commit(&s_full[s]);
                }
                if (j >= 1) {
                    const int jj = j - 1, s = jj % STAGES;
                    ok = mbar_wait(&p_full[s], (jj / STAGES) & 1, abortp) && mbar_wait(&v_full[s], (jj / STAGES) & 1, abortp);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t db = umma_desc_mn(v_addr + s * C::KV_BYTES + k * (UMMA_K * 128), BK * 128);
                        umma_bf16_ts(tmem_base + C::O_COL, tmem_base + s * BK + k * (UMMA_K / 2), db, idesc_pv,
                                     (jj > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&v_empty[s]);
                    umma_commit(&pv_done[jj & 1]);
                    if (jj == n - 1) umma_commit(o_done);
                }
            }
        }
    } else {
        // ---- softmax: warps 2..5, thread = query row = tensor-memory lane ---------------
        const int qd = warp & 3;
        const int r = qd * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(qd * 32) << 16);
        const int pos_r = min(pos0 + r, hi);                       // rows past the end behave like the last one
        const int lo_r = (window > 0 && pos_r - window + 1 > 0) ? pos_r - window + 1 : 0;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n && ok; ++j) {
            const int s = j % STAGES;
            const int key0 = (t0 + j) * BK;
            ok = __all_sync(0xffffffffu, mbar_wait(&s_full[s], (j / STAGES) & 1, abortp));
            if (!ok) break;
            tc_fence_after();
            uint32_t sa[32], sb[32];
            tmem_ld32(lane_base + s * BK, sa);
            tmem_ld32(lane_base + s * BK + 32, sb);
            tmem_wait_ld();
            // some row of the CTA has a masked key in this tile: the causal edge, or the window's start
            const bool edge = key0 + BK - 1 > pos0 || (window > 0 && key0 < hi - window + 1);
            float mx = -INFINITY;
            if (edge) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int ka = key0 + i, kb = key0 + 32 + i;
                    if (ka > pos_r || ka < lo_r) sa[i] = 0xff800000u;          // -inf
                    if (kb > pos_r || kb < lo_r) sb[i] = 0xff800000u;
                }
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = max3(mx, __uint_as_float(sa[i]), __uint_as_float(sb[i]));
            // The exponent's reference m_run follows the row maximum lazily: it moves only when the
            // maximum has grown by more than 2^RESCALE_STEP, so that O seldom has to be rescaled.  Until
            // then the probabilities are at most 2^RESCALE_STEP instead of 1, which float32 sums and bf16
            // operands hold just as well; the final division by the sum (same reference) makes it exact.
            const float m_tile = mx * scale_log2;                      // scale_log2 > 0
            const bool move = m_tile - m_run > RESCALE_STEP;           // also the first visible key (m_run = -inf)
            const float m_new = move ? m_tile : m_run;
            const float mu = m_new == -INFINITY ? 0.f : m_new;
            const float corr = move ? ex2(m_run - mu) : 1.f;           // 0 for a row that saw nothing yet
            uint32_t pr[32];
            const uint64_t scale2 = f2_pack(scale_log2, scale_log2), neg_mu2 = f2_pack(-mu, -mu);
            uint64_t sum_a = f2_pack(0.f, 0.f), sum_b = sum_a;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float p0, p1, p2, p3;
                f2_unpack(f2_fma(f2_pack(__uint_as_float(sa[2 * i]), __uint_as_float(sa[2 * i + 1])), scale2, neg_mu2), p0, p1);
                f2_unpack(f2_fma(f2_pack(__uint_as_float(sb[2 * i]), __uint_as_float(sb[2 * i + 1])), scale2, neg_mu2), p2, p3);
                p0 = ex2(p0), p1 = ex2(p1), p2 = ex2(p2), p3 = ex2(p3);
                sum_a = f2_add(sum_a, f2_pack(p0, p1));
                sum_b = f2_add(sum_b, f2_pack(p2, p3));
                pr[i] = pack2(p0, p1);
                pr[16 + i] = pack2(p2, p3);
            }
            float l0, l1;
            f2_unpack(f2_add(sum_a, sum_b), l0, l1);
            const float lsum = l0 + l1;
            l_run = l_run * corr + lsum;
            m_run = m_new;
            // O holds the sum up to tile j-1 relative to the old maximum: rescale this row when it moved
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
                // the product of tile j-1; its barrier's phase before (tile j-3) is long complete, the
                // one after (tile j+1) cannot begin before this warp has delivered P of tile j
                ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abortp));
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld32(lane_base + C::O_COL + c * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                    tmem_st32(lane_base + C::O_COL + c * 32, o);
                }
            }
            // value rows of keys that no row of the CTA may see are zeroed before P V reads them
            if (key0 + BK - 1 > hi || key0 < lo) {
                ok = __all_sync(0xffffffffu, mbar_wait(&v_full[s], (j / STAGES) & 1, abortp));
                if (!ok) break;
                if (r < BK && (key0 + r > hi || key0 + r < lo)) {
#pragma unroll
                    for (int hh = 0; hh < C::HALVES; ++hh) {
                        uint4* row = reinterpret_cast<uint4*>(Vs + s * C::KV_BYTES + hh * BK * 128 + r * 128);
#pragma unroll
                        for (int c = 0; c < 8; ++c) row[c] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            tmem_st32(lane_base + s * BK, pr);                         // P over the first half of S
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&p_full[s]);
        }
        pdl_trigger_gemm();
        // A barrier of its own, with a single phase.  (A barrier shared with the loop's waits would be
        // asked for a phase by its parity bit alone; the product before the last may still be running here -
        // it was issued after the S that this warp just finished with - and such a wait once passed two
        // phases early, about one step in ten under load.)
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(o_done, 0, abortp));
        if (ok && nsplit > 1) {
            tc_fence_after();
            const size_t slot = ((size_t)(tok0 + r) * nh + h) * nsplit + split;
            float* prow = part_o + slot * HD;
            if (r < rows) {
                part_ml[slot * 2] = m_run;
                part_ml[slot * 2 + 1] = l_run;
            }
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(lane_base + C::O_COL + c * 32, o);
                tmem_wait_ld();
                if (r < rows) {
#pragma unroll
                    for (int v4 = 0; v4 < 8; ++v4)
                        *reinterpret_cast<uint4*>(prow + c * 32 + v4 * 4) =
                            make_uint4(o[v4 * 4], o[v4 * 4 + 1], o[v4 * 4 + 2], o[v4 * 4 + 3]);
                }
            }
        } else if (ok) {
            tc_fence_after();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            __nv_bfloat16* orow = out + (size_t)(tok0 + r) * out_stride + (size_t)h * HD;
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(lane_base + C::O_COL + c * 32, o);
                tmem_wait_ld();
                if (r < rows) {
#pragma unroll
                    for (int v4 = 0; v4 < 4; ++v4) {
                        uint4 w;
                        w.x = pack2(__uint_as_float(o[v4 * 8 + 0]) * inv, __uint_as_float(o[v4 * 8 + 1]) * inv);
                        w.y = pack2(__uint_as_float(o[v4 * 8 + 2]) * inv, __uint_as_float(o[v4 * 8 + 3]) * inv);
                        w.z = pack2(__uint_as_float(o[v4 * 8 + 4]) * inv, __uint_as_float(o[v4 * 8 + 5]) * inv);
                        w.w = pack2(__uint_as_float(o[v4 * 8 + 6]) * inv, __uint_as_float(o[v4 * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + v4 * 8) = w;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag) report_error(err, PRISM_ERR_WAIT_TIMEOUT);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS));
    }
}

template <int HD>
int launch(const void* q, int q_stride, int T, void* out, int out_stride, const void* kc, const void* vc, int cache_pages,
           const int* bt, int bt_width, const int* seg_start, const int* cached_len, int S, int max_q_len, int nh, int nkv,
           int page_size, int num_pages, int window, float scale, int* err, int nsplit, float* part_o, float* part_ml,
           cudaStream_t stream) {
    using C = ACfg<HD>;
    CUtensorMap mq, mk, mv;
    int rc = make_map(&mq, q, T, (long long)nh * HD, q_stride, BQ);
    if (rc) return rc;
    rc = make_map(&mk, kc, (long long)cache_pages * page_size, (long long)nkv * HD, (long long)nkv * HD, BK);
    if (rc) return rc;
    rc = make_map(&mv, vc, (long long)cache_pages * page_size, (long long)nkv * HD, (long long)nkv * HD, BK);
    if (rc) return rc;
    auto kern = attn_prefill_tc_kernel<HD>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
    dim3 grid(nh, (max_q_len + BQ - 1) / BQ * nsplit, S);
    return (int)launch_kernel(kern, grid, dim3(THREADS), C::SMEM, stream, mq, mk, mv, (__nv_bfloat16*)out, out_stride, bt,
                              bt_width, seg_start, cached_len, nh, nkv, page_size, num_pages, window,
                              scale * 1.4426950408889634f, err, nsplit, part_o, part_ml);
}

}  // namespace tca
}  // namespace prism

// 1 if the tcgen05 prefill kernel takes these sizes (else the mma.sync kernel or the generic one is used)
PRISM_EXPORT int prism_attention_prefill_tc_supported(int hd, int nh, int nkv, int page_size) {
    return (hd == 64 || hd == 128) && nkv > 0 && nh % nkv == 0 && page_size > 0 && page_size % prism::tca::BK == 0;
}

// nsplit > 1: the key tiles of every query tile are shared among nsplit CTAs, which leave partial results in
// part_o (float [T, nh, nsplit, hd]) and part_ml (float [T, nh, nsplit, 2]) for prism_attention_merge_bf16; `out`
// is then not written here.
// Prefill / portions: S segments; segment s has tokens seg_start[s] .. seg_start[s+1]-1 of q [T, nh, hd] at positions
// cached_len[s] + i.  kc / vc: bf16 [cache_pages, page_size, nkv, hd]; block-table entries are < num_pages <= cache_pages.
PRISM_EXPORT int prism_attention_prefill_tc(const void* q, int q_stride, int T, void* out, int out_stride, const void* kc,
                                            const void* vc, int cache_pages, const int* block_table, int bt_width,
                                            const int* seg_start, const int* cached_len, int S, int max_q_len, int nh,
                                            int nkv, int hd, int page_size, int num_pages, int window, float scale,
                                            int* err, int nsplit, float* part_o, float* part_ml, cudaStream_t stream) {
    if (S <= 0 || max_q_len <= 0 || T <= 0) return 0;
    if (nsplit < 1 || (nsplit > 1 && (part_o == nullptr || part_ml == nullptr || ((uintptr_t)part_o & 15))))
        return (int)cudaErrorInvalidValue;
    if (!prism_attention_prefill_tc_supported(hd, nh, nkv, page_size) || S > 65535 ||
        (long long)((max_q_len + prism::tca::BQ - 1) / prism::tca::BQ) * nsplit > 65535 || q_stride % 8 ||
        out_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15) ||
        num_pages > cache_pages || scale <= 0.f)
        return (int)cudaErrorInvalidValue;
#define ARGS q, q_stride, T, out, out_stride, kc, vc, cache_pages, block_table, bt_width, seg_start, cached_len, S, \
             max_q_len, nh, nkv, page_size, num_pages, window, scale, err, nsplit, part_o, part_ml, stream
    return hd == 64 ? prism::tca::launch<64>(ARGS) : prism::tca::launch<128>(ARGS);
#undef ARGS
}
