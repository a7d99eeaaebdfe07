// Sampling over float32 logits, one block per row.
//
// Greedy: argmax, lowest index on ties (andre-fu/prism engine/scheduler.py:268,
// engine/executor.py:424).  Temperature: p = softmax(logits / T)
// (scheduler.py:270, executor.py:426) and, in place of torch.multinomial's
// unseeded draw (scheduler.py:271), the inverse CDF at a uniform number u the
// host supplies: the first index whose inclusive cumulative sum of
// exp((x - max) / T) exceeds u * total.  A row with temperature <= 0 is greedy.
#include "common.cuh"

namespace prism {

constexpr int SAMPLE_THREADS = 512;

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
              const float* __restrict__ u, int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    __shared__ float s_val[SAMPLE_THREADS];
    __shared__ int s_idx[SAMPLE_THREADS];
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = pdl_fresh(logits) + (size_t)row * ld;       // the previous kernel's output
    const float temp = temperature ? temperature[row] : 0.f;

    // argmax (needed by both branches: it is also the softmax's max)
    float best = -INFINITY;
    int besti = V;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float v = x[i];
        if (v > best || (v == best && i < besti)) { best = v; besti = i; }
    }
    s_val[tid] = best;
    s_idx[tid] = besti;
    __syncthreads();
    for (int o = SAMPLE_THREADS / 2; o > 0; o >>= 1) {
        if (tid < o) {
            const float v = s_val[tid + o];
            const int i = s_idx[tid + o];
            if (v > s_val[tid] || (v == s_val[tid] && i < s_idx[tid])) { s_val[tid] = v; s_idx[tid] = i; }
        }
        __syncthreads();
    }
    const float mx = s_val[0];
    const int amax = s_idx[0] < V ? s_idx[0] : 0;
    __syncthreads();
    if (!(temp > 0.f)) {
        if (tid == 0) out[row] = amax;
        return;
    }
    // each thread owns one contiguous chunk so that the cumulative sum has a fixed order
    const float inv_t = 1.f / temp;
    const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int c0 = min(tid * chunk, V), c1 = min(c0 + chunk, V);
    float part = 0.f;
    for (int i = c0; i < c1; ++i) part += expf((x[i] - mx) * inv_t);
    s_val[tid] = part;
    __syncthreads();
    if (tid == 0) {
        float run = 0.f;
        for (int i = 0; i < SAMPLE_THREADS; ++i) { const float p = s_val[i]; s_val[i] = run; run += p; }
        scratch[0] = run;
        s_idx[0] = -1;
    }
    __syncthreads();
    const float target = u[row] * scratch[0];
    const float before = s_val[tid];
    if (c0 < c1 && target >= before && (tid == SAMPLE_THREADS - 1 || c1 == V || target < s_val[tid + 1] )) {
        float run = before;
        int pick = c1 - 1;
        for (int i = c0; i < c1; ++i) {
            run += expf((x[i] - mx) * inv_t);
            if (run > target) { pick = i; break; }
        }
        // rounding can push the crossing past this chunk's end; the last index of the chunk stands
        atomicMax(&s_idx[0], pick);
    }
    __syncthreads();
    if (tid == 0) out[row] = s_idx[0] >= 0 ? s_idx[0] : amax;
}

// Greedy only, many blocks per row: block (b, row) finds the best of its slice of the
// vocabulary and leaves (value, index) in `part`; the block that arrives last at the row's
// counter reduces the slices (lowest index on ties) and writes the token.  Nobody waits.
constexpr int ARGMAX_THREADS = 256;

__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_split_kernel(const float* __restrict__ logits, int ld, int V, float* __restrict__ part_val,
                    int* __restrict__ part_idx, int* __restrict__ counters, int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ float s_val[ARGMAX_THREADS];
    __shared__ int s_idx[ARGMAX_THREADS];
    __shared__ int s_last;
    const int nb = gridDim.x, b = blockIdx.x, row = blockIdx.y, tid = threadIdx.x;
    const int per = ((V + nb - 1) / nb + 3) & ~3;
    const int c0 = min(b * per, V), c1 = min(c0 + per, V);
    const float* x = pdl_fresh(logits) + (size_t)row * ld;       // the previous kernel's output
    float best = -INFINITY;
    int besti = V;
    for (int i = c0 + tid; i < c1; i += ARGMAX_THREADS) {
        const float v = x[i];
        if (v > best || (v == best && i < besti)) { best = v; besti = i; }
    }
    auto reduce = [&]() {
        s_val[tid] = best;
        s_idx[tid] = besti;
        __syncthreads();
        for (int o = ARGMAX_THREADS / 2; o > 0; o >>= 1) {
            if (tid < o) {
                const float v = s_val[tid + o];
                const int i = s_idx[tid + o];
                if (v > s_val[tid] || (v == s_val[tid] && i < s_idx[tid])) { s_val[tid] = v; s_idx[tid] = i; }
            }
            __syncthreads();
        }
    };
    reduce();
    if (tid == 0) {
        part_val[(size_t)row * nb + b] = s_val[0];
        part_idx[(size_t)row * nb + b] = s_idx[0];
        __threadfence();
        const int old = atomicAdd(&counters[row], 1);
        s_last = old == nb - 1;
        if (s_last) counters[row] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    best = -INFINITY;
    besti = V;
    if (tid < nb) {
        best = __ldcg(&part_val[(size_t)row * nb + tid]);
        besti = __ldcg(&part_idx[(size_t)row * nb + tid]);
    }
    reduce();
    if (tid == 0) out[row] = s_idx[0] < V ? s_idx[0] : 0;
}

}  // namespace prism

// All rows greedy, several blocks per row.  part_val/part_idx: R * nb entries; counters: R ints, zero
// before the first launch (the kernel leaves them zero).  nb <= 256.
PRISM_EXPORT int prism_argmax_split(const float* logits, int ld, int R, int V, int nb, float* part_val,
                                    int* part_idx, int* counters, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (nb < 1 || nb > prism::ARGMAX_THREADS || R > 65535) return (int)cudaErrorInvalidValue;
    return (int)prism::launch_kernel(prism::argmax_split_kernel, dim3(nb, R), dim3(prism::ARGMAX_THREADS), 0, stream,
                                     logits, ld, V, part_val, part_idx, counters, out);
}

// temperature and u may be null: all rows greedy.
PRISM_EXPORT int prism_sample(const float* logits, int ld, int R, int V, const float* temperature,
                              const float* u, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    prism::sample_kernel<<<R, prism::SAMPLE_THREADS, 0, stream>>>(logits, ld, V, temperature, u, out);
    return (int)cudaPeekAtLastError();
}
