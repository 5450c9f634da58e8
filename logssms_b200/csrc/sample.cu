// Next-token choice from float32 logits, one CTA per row, all steps fused in one launch:
//   greedy rows (temperature <= 0): argmax, lowest index on ties;
//   other rows: softmax(logits / max(T, 1e-6)) -> keep the top_k most likely -> keep the smallest
//   set whose mass reaches top_p (of what top_k kept) -> draw one token from what is left.
// The reference does the same chain with four library calls (softmax, top_k_renorm_probs,
// top_p_renorm_probs, sampling_from_probs; python/logssms/engine/sample.py:31-72, 83-133).
//
// Probabilities are never stored: p_i = exp((l_i - max) / T) is recomputed from the logits in every
// pass (the row stays in L1/L2), so any vocabulary size works with a few bytes of shared memory.
// The k-th largest probability and the top-p threshold are found by bisection on the bit pattern of
// p (monotonic for non-negative floats).  Ties at a threshold are kept together.  The draw uses a
// Philox-4x32-10 counter RNG keyed by (seed, row counter), so a request's stream of draws depends
// only on its seed and how many tokens it has drawn, not on the batch it is in.
#include "lb200/common.cuh"
using namespace lb200;

namespace {
constexpr int kThreads = 1024;

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t (&k)[2]) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
    const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
    const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k[0], n2 = hi0 ^ c[3] ^ k[1];
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
    k[0] += 0x9E3779B9u; k[1] += 0xBB67AE85u;
}

__device__ float philox_uniform(unsigned long long seed, unsigned long long counter) {
    uint32_t c[4] = {(uint32_t)counter, (uint32_t)(counter >> 32), 0x5AD0F00Du, 0u};
    uint32_t k[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
#pragma unroll
    for (int i = 0; i < 10; ++i) philox_round(c, k);
    return (float)(c[0] >> 8) * (1.0f / 16777216.0f);      // [0, 1)
}

__device__ __forceinline__ float block_sum_all(float v, float* red) { return block_sum(v, red); }

__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, long row_stride, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ counters,
              int* __restrict__ out, const int* __restrict__ status, int rows) {
    // `status`: a word on the device (the error word of the kernels with bounded waits) that travels to the host
    // behind the sampled ids, out[rows], in the same copy
    if (status != nullptr && blockIdx.x == 0 && threadIdx.x == 0) out[rows] = *status;
    __shared__ float red[32];
    __shared__ int red_i[32];
    __shared__ float scan[kThreads];
    __shared__ int chosen;
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* l = logits + (size_t)row * row_stride;
    const float T = temperature ? temperature[row] : 0.f;

    // max and argmax (lowest index among equal maxima)
    float best = -INFINITY; int best_i = V;
    for (int i = tid; i < V; i += kThreads) {
        const float v = l[i];
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if ((tid & 31) == 0) { red[tid >> 5] = best; red_i[tid >> 5] = best_i; }
    __syncthreads();
    if (tid < 32) {
        best = red[tid]; best_i = red_i[tid];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (tid == 0) { red[0] = best; red_i[0] = best_i; }
    }
    __syncthreads();
    const float m = red[0];
    const int arg = red_i[0];
    __syncthreads();
    if (!(T > 0.f)) {                                   // greedy (also NaN temperature)
        if (tid == 0) out[row] = arg;
        return;
    }
    const float invT = 1.f / fmaxf(T, 1e-6f);
#define LB_P(i) expf((l[i] - m) * invT)

    // threshold as a bit pattern: keep p with bits >= thr
    unsigned thr = 0u;
    const int k = top_k ? top_k[row] : 0;
    if (k >= 1 && k < V) {
        unsigned lo = 0u, hi = 0x3F800000u;             // p in [0, 1]; find largest t with count(p >= t) >= k
        while (lo < hi) {
            const unsigned mid = lo + (hi - lo + 1u) / 2u;
            float cnt = 0.f;
            for (int i = tid; i < V; i += kThreads) cnt += (__float_as_uint(LB_P(i)) >= mid) ? 1.f : 0.f;
            cnt = block_sum_all(cnt, red);
            if (cnt >= (float)k) lo = mid; else hi = mid - 1u;
        }
        thr = lo;
    }
    float Z = 0.f;
    for (int i = tid; i < V; i += kThreads) { const float p = LB_P(i); if (__float_as_uint(p) >= thr) Z += p; }
    Z = block_sum_all(Z, red);
    const float P = top_p ? top_p[row] : 1.f;
    if (P < 1.f) {
        const float need = fmaxf(P, 1e-6f) * Z;         // largest t with mass(p >= t) >= need
        unsigned lo = thr, hi = 0x3F800000u;
        while (lo < hi) {
            const unsigned mid = lo + (hi - lo + 1u) / 2u;
            float mass = 0.f;
            for (int i = tid; i < V; i += kThreads) { const float p = LB_P(i); if (__float_as_uint(p) >= mid) mass += p; }
            mass = block_sum_all(mass, red);
            if (mass >= need) lo = mid; else hi = mid - 1u;
        }
        thr = lo;
    }

    // inverse CDF over the kept set, in index order: thread t owns indices [t*chunk, (t+1)*chunk)
    const int chunk = (V + kThreads - 1) / kThreads;
    const int i0 = min(tid * chunk, V), i1 = min(i0 + chunk, V);
    float mine = 0.f;
    for (int i = i0; i < i1; ++i) { const float p = LB_P(i); if (__float_as_uint(p) >= thr) mine += p; }
    scan[tid] = mine;
    if (tid == 0) chosen = -1;
    __syncthreads();
    for (int o = 1; o < kThreads; o <<= 1) {            // inclusive scan
        const float add = tid >= o ? scan[tid - o] : 0.f;
        __syncthreads();
        scan[tid] += add;
        __syncthreads();
    }
    const float total = scan[kThreads - 1];
    const unsigned long long seed = seeds ? seeds[row] : 0ull;
    const unsigned long long ctr = counters ? counters[row] : 0ull;
    const float target = philox_uniform(seed, ctr) * total;
    const float before = scan[tid] - mine;
    if (mine > 0.f && target >= before && target < scan[tid]) {
        float acc = before; int pick = -1;
        for (int i = i0; i < i1; ++i) {
            const float p = LB_P(i);
            if (__float_as_uint(p) >= thr) { acc += p; pick = i; if (target < acc) break; }
        }
        atomicMax(&chosen, pick);
    }
    __syncthreads();
    if (tid == 0) out[row] = chosen >= 0 ? chosen : arg;   // rounding left nobody: the most likely token
#undef LB_P
}
}  // namespace

extern "C" int lb_sample(const float* logits, long row_stride, int rows, int V, const float* temperature,
                         const int* top_k, const float* top_p, const unsigned long long* seeds,
                         const unsigned long long* counters, int* out, const int* status, void* stream) {
    if (rows <= 0) return kOk;
    if (V <= 0) return kBadSize;
    sample_kernel<<<rows, kThreads, 0, (cudaStream_t)stream>>>(logits, row_stride, V, temperature, top_k, top_p,
                                                               seeds, counters, out, status, rows);
    return launch_status();
}
