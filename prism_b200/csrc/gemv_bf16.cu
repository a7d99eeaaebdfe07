// Weight-streaming matrix product for decode: y[M, N] = x[M, K] @ W[N, K]^T
// with M small (<= 32 tokens), bf16 in, float32 accumulate.  This is the
// F.linear of andre-fu/prism's decode path (engine/executor.py:142,155,158,160,162)
// at the sizes where it is bound by reading W once from HBM.
//
// A warp owns 16 rows of W (features) and a range of K.  W is the A operand
// of m16n8k16 MMAs and the tokens are the 8 columns of the B operand, so a
// weight is read once, straight from global memory into registers, with
// 16-byte loads: a thread loads 8 consecutive k of its row, and the same 8
// consecutive k of its token's activations, and uses them as the fragment
// elements of two MMAs.  The contraction index is permuted the same way in
// both operands, which a sum does not notice.  No shared memory on the
// streaming path; loads for the next 128 k are in flight while the current
// ones are multiplied.
//
// Eight warps per CTA are arranged as (8 / WK) row groups x WK splits of K;
// the WK partial sums meet in shared memory (fixed order: deterministic).
// Epilogues: + bias, store bf16 or float32; or "paired SwiGLU": the warp
// streams row m (gate) and row m + I (up) of the fused gate_up weight
// (engine/weight_pool.py:194-197) and stores silu(gate) * up
// (executor.py:127), so the [M, 2I] intermediate never exists.
#include "common.cuh"
#include "mma_helpers.cuh"

namespace prism {

constexpr int GEMV_WARPS = 8;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;
constexpr int GEMV_U = 4;            // 32-k steps per unrolled iteration

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2 };

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

template <int NT, int EPI>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_kernel(const __nv_bfloat16* __restrict__ W, int ldw, const __nv_bfloat16* __restrict__ x, int ldx,
            const void* __restrict__ bias, int bias_bf16, void* __restrict__ y, int ldy, int M, int N,
            int K, int WK, int pair_offset) {
    pdl_trigger();
    pdl_wait();
    constexpr int STREAMS = EPI == EPI_SWIGLU ? 2 : 1;    // weight rows streamed per output row
    extern __shared__ float red[];                         // [8 warps][STREAMS][16][NT * 8] when WK > 1
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int WR = GEMV_WARPS / WK;
    const int wk = warp % WK, wr = warp / WK;
    const int row0 = (blockIdx.x * WR + wr) * 16;
    const int r = lane >> 2, c = lane & 3;
    const int kper = ((K + 32 * WK - 1) / (32 * WK)) * 32;
    const int ks = wk * kper, ke = min(K, ks + kper);

    float acc[STREAMS][NT][4];
#pragma unroll
    for (int s = 0; s < STREAMS; ++s)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[s][j][0] = acc[s][j][1] = acc[s][j][2] = acc[s][j][3] = 0.f;

    if (row0 < N && ks < ke) {
        const __nv_bfloat16* pw[STREAMS][2];
#pragma unroll
        for (int s = 0; s < STREAMS; ++s) {
            pw[s][0] = W + (size_t)(min(row0 + r, N - 1) + s * pair_offset) * ldw + c * 8;
            pw[s][1] = W + (size_t)(min(row0 + r + 8, N - 1) + s * pair_offset) * ldw + c * 8;
        }
        const __nv_bfloat16* px[NT];
        bool xv[NT];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            xv[j] = j * 8 + r < M;
            px[j] = x + (size_t)(xv[j] ? j * 8 + r : 0) * ldx + c * 8;
        }
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        constexpr int U = GEMV_U / STREAMS;               // 32-k steps per block of loads
        uint4 wA[U][STREAMS][2], wB[U][STREAMS][2];       // two register buffers, indexed statically
        auto load_w = [&](uint4 (&w)[U][STREAMS][2], int k0) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int kk = k0 + 32 * u;
                const bool in = kk + c * 8 < ke;
#pragma unroll
                for (int s = 0; s < STREAMS; ++s) {
                    w[u][s][0] = in ? ldg_stream16(pw[s][0] + kk) : zero;
                    w[u][s][1] = in ? ldg_stream16(pw[s][1] + kk) : zero;
                }
            }
        };
        auto compute = [&](const uint4 (&w)[U][STREAMS][2], int k0) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int kk = k0 + 32 * u;
                const bool in = kk + c * 8 < ke;
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const uint4 xb = (in && xv[j]) ? __ldg(reinterpret_cast<const uint4*>(px[j] + kk)) : zero;
#pragma unroll
                    for (int s = 0; s < STREAMS; ++s) {
                        const uint4 wa = w[u][s][0], wb = w[u][s][1];
                        const uint32_t a1[4] = {wa.x, wb.x, wa.y, wb.y};
                        const uint32_t a2[4] = {wa.z, wb.z, wa.w, wb.w};
                        mma_bf16_16816(acc[s][j], a1, xb.x, xb.y);
                        mma_bf16_16816(acc[s][j], a2, xb.z, xb.w);
                    }
                }
            }
        };
        constexpr int STEP = 32 * U;
        load_w(wA, ks);
        for (int k0 = ks; k0 < ke; k0 += 2 * STEP) {
            if (k0 + STEP < ke) load_w(wB, k0 + STEP);
            compute(wA, k0);
            if (k0 + 2 * STEP < ke) load_w(wA, k0 + 2 * STEP);
            if (k0 + STEP < ke) compute(wB, k0 + STEP);
        }
    }

    // value of output (feature m, token n) from the summed accumulators
    auto finish = [&](float v0, float v1, int m, int n) {
        if (m >= N || n >= M) return;
        if (EPI == EPI_SWIGLU) {
            reinterpret_cast<__nv_bfloat16*>(y)[(size_t)n * ldy + m] = __float2bfloat16_rn(v0 / (1.f + expf(-v0)) * v1);
        } else {
            if (bias != nullptr) v0 += load_param(bias, bias_bf16, m);
            if (EPI == EPI_F32) reinterpret_cast<float*>(y)[(size_t)n * ldy + m] = v0;
            else reinterpret_cast<__nv_bfloat16*>(y)[(size_t)n * ldy + m] = __float2bfloat16_rn(v0);
        }
    };

    if (WK == 1) {
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                finish(acc[0][j][e], STREAMS == 2 ? acc[STREAMS - 1][j][e] : 0.f, row0 + r + (e >> 1) * 8,
                       j * 8 + c * 2 + (e & 1));
        return;
    }
    // partial sums of the WK splits meet in shared memory: red[warp][stream][row 16][token NT*8]
    constexpr int PER_WARP = STREAMS * 16 * NT * 8;
#pragma unroll
    for (int s = 0; s < STREAMS; ++s)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                red[warp * PER_WARP + (s * 16 + r + (e >> 1) * 8) * (NT * 8) + j * 8 + c * 2 + (e & 1)] = acc[s][j][e];
    __syncthreads();
    for (int i = threadIdx.x; i < WR * 16 * NT * 8; i += GEMV_THREADS) {
        const int m16 = i % 16, n = (i / 16) % (NT * 8), g = i / (16 * NT * 8);      // consecutive threads: consecutive features
        float v[2] = {0.f, 0.f};
#pragma unroll
        for (int s = 0; s < STREAMS; ++s)
            for (int w = 0; w < WK; ++w)
                v[s] += red[(g * WK + w) * PER_WARP + (s * 16 + m16) * (NT * 8) + n];
        finish(v[0], v[1], (blockIdx.x * WR + g) * 16 + m16, n);
    }
}

template <int NT, int EPI>
int launch_gemv(const __nv_bfloat16* W, int ldw, const __nv_bfloat16* x, int ldx, const void* bias, int bias_bf16,
                void* y, int ldy, int M, int N, int K, int pair_offset, cudaStream_t stream) {
    const int groups = (N + 15) / 16;
    int WK = 1;
    while (WK < GEMV_WARPS && (groups + (GEMV_WARPS / WK) - 1) / (GEMV_WARPS / WK) < 2 * 148) WK *= 2;
    while (WK > 1 && K / WK < 128) WK /= 2;
    const int WR = GEMV_WARPS / WK;
    const int grid = (groups + WR - 1) / WR;
    const size_t smem = WK > 1 ? (size_t)GEMV_WARPS * (EPI == EPI_SWIGLU ? 2 : 1) * 16 * NT * 8 * sizeof(float) : 0;
    auto kern = gemv_kernel<NT, EPI>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, GEMV_THREADS, smem, stream>>>(W, ldw, x, ldx, bias, bias_bf16, y, ldy, M, N, K, WK, pair_offset);
    return (int)cudaPeekAtLastError();
}

}  // namespace prism

// 1 if the kernel takes these sizes
PRISM_EXPORT int prism_gemv_bf16_supported(int M, int N, int K) {
    return M >= 1 && M <= 32 && K % 8 == 0 && K >= 32 && N >= 1;
}

// epi: 0 bf16 out (+bias), 1 float32 out (+bias), 2 paired SwiGLU (W is [2I, K]: gate rows then up rows;
// N = I output features; bf16 out, no bias).  ldw, ldx, ldy in elements.
PRISM_EXPORT int prism_gemv_bf16(const void* W, int ldw, const void* x, int ldx, const void* bias, int bias_dtype,
                                 void* y, int ldy, int M, int N, int K, int epi, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!prism_gemv_bf16_supported(M, N, K) || ldw % 8 || ldx % 8) return (int)cudaErrorInvalidValue;
    const int bb = bias_dtype == PRISM_DTYPE_BF16;
    const int nt = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
    const int pair = epi == prism::EPI_SWIGLU ? N : 0;
#define ARGS (const __nv_bfloat16*)W, ldw, (const __nv_bfloat16*)x, ldx, bias, bb, y, ldy, M, N, K, pair, stream
#define BY_NT(E) (nt == 1 ? prism::launch_gemv<1, E>(ARGS) : nt == 2 ? prism::launch_gemv<2, E>(ARGS) : prism::launch_gemv<4, E>(ARGS))
    if (epi == prism::EPI_BF16) return BY_NT(prism::EPI_BF16);
    if (epi == prism::EPI_F32) return BY_NT(prism::EPI_F32);
    if (epi == prism::EPI_SWIGLU) return BY_NT(prism::EPI_SWIGLU);
#undef BY_NT
#undef ARGS
    return (int)cudaErrorInvalidValue;
}
