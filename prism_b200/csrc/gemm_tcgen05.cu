// Weight-streaming bf16 matrix product on Blackwell's 5th-generation tensor
// cores:  y[M, N] = x[M, K] @ W[N, K]^T  for a small number of tokens M
// (decode), i.e. the F.linear calls of andre-fu/prism's decode path
// (engine/executor.py:142,155,158,160,162).
//
// The roles are swapped with respect to the usual GEMM: 128 rows of W are the
// M dimension of one tcgen05.mma and the (padded) tokens are its N dimension
// (16..64), so every weight byte crosses the SM once: TMA
// (cp.async.bulk.tensor, 128-byte swizzle) brings 128 x 64 tiles of W and the
// matching 64-wide slice of x into a ring of shared-memory stages, one
// elected thread issues tcgen05.mma (operands straight from shared memory,
// float32 accumulator in tensor memory), tcgen05.commit releases a stage back
// to the TMA producer, and four epilogue warps read the accumulator with
// tcgen05.ld.  Nothing passes through registers on the way in, so the load
// pipeline is as deep as shared memory allows (6 stages of 18 KB, two CTAs
// per SM).
//
//   warp 0: TMA producer      warp 1: TMEM allocation + MMA issue
//   warps 2-5: epilogue (each reads the 32 accumulator lanes it may access)
//
// Epilogues: bf16 or float32 output with optional bias; partial sums of a
// K-split (grid.y) as float32 [split, M, N] for the next kernel to add (the
// fused residual-add + RMSNorm takes such a stack); "paired SwiGLU": two
// weight tiles per stage (gate rows m.., up rows I + m..), two accumulators,
// output silu(gate) * up.
//
// Every mbarrier wait is bounded (about two seconds): on expiry the kernel
// records PRISM_ERR_WAIT_TIMEOUT, all roles fall through to the common exit,
// tensor memory is released and the kernel returns.
#include "tcgen05.cuh"

namespace prism {
namespace tc {

constexpr int TILE_M = 128;          // weight rows per CTA tile (UMMA M)
constexpr int THREADS = 192;         // 6 warps

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2, EPI_PARTIAL = 3 };

template <int NTOK, int EPI> struct Cfg {
    static constexpr int W_TILES = EPI == EPI_SWIGLU ? 2 : 1;
    static constexpr int STAGE_BYTES = W_TILES * TILE_M * TILE_K * 2 + NTOK * TILE_K * 2;
    static constexpr int FIT = 208 * 1024 / STAGE_BYTES;
    static constexpr int STAGES = FIT >= 6 ? 6 : (FIT >= 2 ? FIT : 2);
    static constexpr int TMEM_COLS = (W_TILES * NTOK) <= 32 ? 32 : ((W_TILES * NTOK) <= 64 ? 64 : 128);
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int NTOK, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_swap_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 const void* __restrict__ bias, int bias_bf16, void* __restrict__ y, int ldy, int M, int N, int K,
                 int kblocks_per_split, int pair_offset, float* __restrict__ ws, int* __restrict__ counters, int* err) {
    using C = Cfg<NTOK, EPI>;
    constexpr int W_TILES = C::W_TILES;
    constexpr int STAGES = C::STAGES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * C::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    __shared__ int abort_flag;
    __shared__ int is_last;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * TILE_M;                    // first weight row (output feature) of this tile
    const int total_kb = (K + TILE_K - 1) / TILE_K;
    const int kb0 = blockIdx.y * kblocks_per_split;
    const int kb1 = min(total_kb, kb0 + kblocks_per_split);
    const int nkb = max(0, kb1 - kb0);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(C::TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    volatile int* abortp = &abort_flag;

    if (warp == 0) {
        // ---- TMA producer ---------------------------------------------------------
        // W does not depend on the kernels before this one: its first STAGES tiles are requested
        // at once; the activations x are requested after pdl_wait(), i.e. once they exist.
        if (lane == 0) {
            int issued = 0;
            const int pre = min(nkb, STAGES);
            for (int i = 0; i < pre; ++i) {
                unsigned char* st = tiles + (size_t)i * C::STAGE_BYTES;
                mbar_expect_tx(&full_bar[i], C::STAGE_BYTES);
                const int kc = (kb0 + i) * TILE_K;
#pragma unroll
                for (int w = 0; w < W_TILES; ++w)
                    tma_load_2d(st + w * TILE_M * TILE_K * 2, &map_w, &full_bar[i], kc, m0 + w * pair_offset);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i)
                tma_load_2d(tiles + (size_t)i * C::STAGE_BYTES + W_TILES * TILE_M * TILE_K * 2, &map_x, &full_bar[i],
                            (kb0 + i) * TILE_K, 0);
            issued = pre;
            for (int i = pre; i < nkb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1, abortp)) break;
                unsigned char* st = tiles + (size_t)s * C::STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
                const int kc = (kb0 + i) * TILE_K;
#pragma unroll
                for (int w = 0; w < W_TILES; ++w)
                    tma_load_2d(st + w * TILE_M * TILE_K * 2, &map_w, &full_bar[s], kc, m0 + w * pair_offset);
                tma_load_2d(st + W_TILES * TILE_M * TILE_K * 2, &map_x, &full_bar[s], kc, 0);
                issued = i + 1;
            }
            pdl_trigger_gemm();     // all of this CTA's loads are on their way: the next kernel may start its prologue
            if (*abortp) {
                // give the copies already in flight a bounded chance to land before the CTA's memory is reused
                for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(&full_bar[i % STAGES], (i / STAGES) & 1, abortp);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue ------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NTOK >> 3) << 17) |
                                       ((uint32_t)(TILE_M >> 4) << 24);
            bool ok = true;
            for (int i = 0; i < nkb && ok; ++i) {
                const int s = i % STAGES;
                ok = mbar_wait(&full_bar[s], (i / STAGES) & 1, abortp);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t st = smem_addr(tiles + (size_t)s * C::STAGE_BYTES);
                const uint64_t db = umma_desc(st + W_TILES * TILE_M * TILE_K * 2);
#pragma unroll
                for (int w = 0; w < W_TILES; ++w) {
                    const uint64_t da = umma_desc(st + w * TILE_M * TILE_K * 2);
#pragma unroll
                    for (int k = 0; k < TILE_K / UMMA_K; ++k)
                        umma_bf16(tmem_base + w * NTOK, da + (uint64_t)(k * UMMA_K * 2 >> 4), db + (uint64_t)(k * UMMA_K * 2 >> 4),
                                  idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty_bar[s]);          // the stage is free once these MMAs have read it
            }
            umma_commit(acc_bar);                    // the accumulator is complete (or as far as it got)
        }
    } else {
        // ---- epilogue: warps 2..5, TMEM lanes (warp % 4) * 32 .. + 31 -----------------
        const int q = warp & 3;
        const int m = m0 + q * 32 + lane;            // this thread's output feature
        pdl_wait();                                      // outputs, bias, workspace: ordered after earlier kernels
        if (nkb > 0) mbar_wait(acc_bar, 0, abortp);      // on expiry this sets the abort flag
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps agree on the flag
        const bool go = *abortp == 0;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (go) {
            float acc[W_TILES][NTOK];
            if (nkb > 0) {
#pragma unroll
                for (int w = 0; w < W_TILES; ++w)
                    tmem_load<NTOK>(tmem_base + ((uint32_t)(q * 32) << 16) + w * NTOK, acc[w]);
            } else {
#pragma unroll
                for (int w = 0; w < W_TILES; ++w)
#pragma unroll
                    for (int n = 0; n < NTOK; ++n) acc[w][n] = 0.f;
            }
            bool finish = true;
            if ((EPI == EPI_BF16 || EPI == EPI_F32) && gridDim.y > 1) {
                // K was split over gridDim.y CTAs: every CTA leaves its partial sums in the workspace and
                // the one that arrives last at the tile's counter adds them up, in split order, and
                // finishes the tile.  Nobody waits for anybody.
                if (m < N)
#pragma unroll
                    for (int n = 0; n < NTOK; ++n)
                        if (n < M) ws[((size_t)blockIdx.y * M + n) * N + m] = acc[0][n];
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");            // the four epilogue warps
                if (threadIdx.x == 64) {
                    const int old = atomicAdd(&counters[blockIdx.x], 1);
                    is_last = old == (int)gridDim.y - 1;
                    if (is_last) counters[blockIdx.x] = 0;                 // ready for the next launch
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                finish = is_last != 0;
                if (finish && m < N) {
                    __threadfence();
#pragma unroll
                    for (int n = 0; n < NTOK; ++n) {
                        if (n >= M) continue;
                        float v = 0.f;
                        for (int sp = 0; sp < (int)gridDim.y; ++sp) v += __ldcg(&ws[((size_t)sp * M + n) * N + m]);
                        acc[0][n] = v;
                    }
                }
            }
            if (finish && m < N) {
                const float b = (EPI == EPI_BF16 || EPI == EPI_F32) && bias != nullptr ? load_param(bias, bias_bf16, m) : 0.f;
#pragma unroll
                for (int n = 0; n < NTOK; ++n) {
                    if (n >= M) continue;
                    if (EPI == EPI_SWIGLU) {
                        const float g = acc[0][n], u = acc[W_TILES - 1][n];
                        reinterpret_cast<__nv_bfloat16*>(y)[(size_t)n * ldy + m] = __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
                    } else if (EPI == EPI_PARTIAL) {
                        reinterpret_cast<float*>(y)[((size_t)blockIdx.y * M + n) * ldy + m] = acc[0][n];
                    } else if (EPI == EPI_F32) {
                        reinterpret_cast<float*>(y)[(size_t)n * ldy + m] = acc[0][n] + b;
                    } else {
                        reinterpret_cast<__nv_bfloat16*>(y)[(size_t)n * ldy + m] = __float2bfloat16_rn(acc[0][n] + b);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag) report_error(err, PRISM_ERR_WAIT_TIMEOUT);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS));
    }
}

// ---- host side ----------------------------------------------------------------------

template <int NTOK, int EPI>
int launch(const void* W, int ldw, long long w_rows, const void* x, int ldx, const void* bias, int bias_bf16, void* y,
           int ldy, int M, int N, int K, int ksplit, int pair_offset, float* ws, int* counters, int* err,
           cudaStream_t stream) {
    using C = Cfg<NTOK, EPI>;
    CUtensorMap mw, mx;
    int rc = make_map(&mw, W, w_rows, K, ldw, TILE_M);
    if (rc) return rc;
    rc = make_map(&mx, x, M, K, ldx, NTOK);
    if (rc) return rc;
    const int total_kb = (K + TILE_K - 1) / TILE_K;
    const int per = (total_kb + ksplit - 1) / ksplit;
    auto kern = gemm_swap_kernel<NTOK, EPI>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
    dim3 grid((N + TILE_M - 1) / TILE_M, ksplit);
    return (int)launch_kernel(kern, grid, dim3(THREADS), C::SMEM, stream, mw, mx, bias, bias_bf16, y, ldy, M, N, K, per,
                              pair_offset, ws, counters, err);
}

}  // namespace tc
}  // namespace prism

// Programmatic dependent launch for every kernel of this library: 1 on (default), 0 off.
PRISM_EXPORT int prism_set_pdl(int on) {
    prism::pdl_enabled() = on ? 1 : 0;
    return prism::pdl_enabled();
}

// 1 if the kernel takes these sizes: up to 64 tokens, K a multiple of 8 (16-byte rows for TMA).
PRISM_EXPORT int prism_gemm_tcgen05_supported(int M, int N, int K) {
    return M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0;
}

// epi: 0 bf16 (+bias), 1 float32 (+bias), 2 paired SwiGLU (W is [2N, K]; bf16 out [M, N]),
// 3 partial sums: y is float32 [ksplit, M, N] (ldy = N), no bias.
// ksplit > 1 with epi 0 or 1 needs a workspace `ws` of ksplit * M * N floats and `counters`, one int per
// 128-row tile of N, zero before the first launch (the kernel leaves them zero); the last CTA of each
// tile adds the partial sums in split order, so the result does not depend on timing.  Not with epi 2.
PRISM_EXPORT int prism_gemm_tcgen05(const void* W, int ldw, const void* x, int ldx, const void* bias, int bias_dtype,
                                    void* y, int ldy, int M, int N, int K, int epi, int ksplit, float* ws,
                                    int* counters, int* err, cudaStream_t stream) {
    using namespace prism::tc;
    if (M <= 0 || N <= 0) return 0;
    if (!prism_gemm_tcgen05_supported(M, N, K) || ldw % 8 || ldx % 8 || ksplit < 1 || (ksplit > 1 && epi == EPI_SWIGLU) ||
        (ksplit > 1 && epi != EPI_PARTIAL && (ws == nullptr || counters == nullptr)) ||
        ((uintptr_t)W & 15) || ((uintptr_t)x & 15))
        return (int)cudaErrorInvalidValue;
    const int bb = bias_dtype == PRISM_DTYPE_BF16;
    const int ntok = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    const long long w_rows = epi == EPI_SWIGLU ? 2LL * N : N;
    const int pair = epi == EPI_SWIGLU ? N : 0;
#define ARGS W, ldw, w_rows, x, ldx, bias, bb, y, ldy, M, N, K, ksplit, pair, ws, counters, err, stream
#define BY_N(E) (ntok == 16 ? launch<16, E>(ARGS) : ntok == 32 ? launch<32, E>(ARGS) : launch<64, E>(ARGS))
    switch (epi) {
        case EPI_BF16: return BY_N(EPI_BF16);
        case EPI_F32: return BY_N(EPI_F32);
        case EPI_SWIGLU: return BY_N(EPI_SWIGLU);
        case EPI_PARTIAL: return BY_N(EPI_PARTIAL);
    }
#undef BY_N
#undef ARGS
    return (int)cudaErrorInvalidValue;
}
