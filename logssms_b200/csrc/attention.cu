// Causal grouped-query attention over a paged key/value cache: the general kernel.
//
// One warp per (token, query head).  It serves every case the step function can produce with one
// code path: portions of prompts (each token sees the cache up to its own position, which includes
// earlier portions and the keys this step stored), single decoded tokens, any mix of them, an
// optional sliding window.  Softmax statistics and the output accumulator are 32-bit; exp is the
// accurate expf.  It takes any head size that is a multiple of 16 up to 256, any number of heads and
// groups, any page size.  It is the kernel of the float32 path and the fall-back of the bfloat16
// path for shapes the tensor-core kernels refuse.
//
// Formula: softmax(q k^T * scale + causal) v per query head h with key/value head h / (Hq/Hkv),
// causal over absolute positions (python/logssms/layers/attention_backend/fi.py:175-190;
// oracle in tests/hybrid/test_falcon_h1.py:24-37 of the reference).
#include "lb200/common.cuh"
using namespace lb200;

namespace {
constexpr int kWarps = 4;
constexpr int kMaxHd = 256;
constexpr int kDpl = kMaxHd / 32;

template <typename T> struct Vec;
template <> struct Vec<float> { using type = float4; static constexpr int n = 4; };
template <> struct Vec<__nv_bfloat16> { using type = uint4; static constexpr int n = 8; };

__device__ __forceinline__ void unpack(const float4& v, float* f) { f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
__device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 p = __bfloat1622float2(h[i]); f[2 * i] = p.x; f[2 * i + 1] = p.y; }
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
paged_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                       T* __restrict__ out, const int* __restrict__ block_table, int bt_stride,
                       const int* __restrict__ token_req, const int* __restrict__ positions, int Hq, int Hkv,
                       int hd, int page_size, float scale, int window) {
    __shared__ float q_s[kWarps][kMaxHd];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t t = blockIdx.x;
    const int h = blockIdx.y * kWarps + warp;
    if (h >= Hq) return;
    const int kvh = h / (Hq / Hkv);
    const int req = token_req[t];
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* bt = block_table + (size_t)req * bt_stride;

    const T* qp = q + (t * Hq + h) * hd;
    for (int d = lane; d < hd; d += 32) q_s[warp][d] = to_f32(qp[d]) * scale;
    __syncwarp();

    float o[kDpl];
#pragma unroll
    for (int i = 0; i < kDpl; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    constexpr int VN = Vec<T>::n;
    using V = typename Vec<T>::type;

    for (int j0 = lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j <= pos;
        long row = 0;
        float s = -INFINITY;
        if (valid) {
            const int page = bt[j / page_size];
            row = (long)page * page_size + (j % page_size);
            const T* kp = k_cache + ((size_t)row * Hkv + kvh) * hd;
            float acc = 0.f;
            for (int d = 0; d < hd; d += VN) {
                float f[VN];
                unpack(*reinterpret_cast<const V*>(kp + d), f);
#pragma unroll
                for (int e = 0; e < VN; ++e) acc += q_s[warp][d + e] * f[e];
            }
            s = acc;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float alpha = expf(m - m_new);         // m = -inf on the first tile: exp(-inf) = 0
        const float p = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < kDpl; ++i) o[i] *= alpha;
        const int count = min(32, pos - j0 + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long rj = __shfl_sync(0xffffffffu, row, jj);
            const T* vp = v_cache + ((size_t)rj * Hkv + kvh) * hd;
#pragma unroll
            for (int i = 0; i < kDpl; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) o[i] += pj * to_f32(vp[d]);
            }
        }
    }
    const float inv = 1.f / l;
    T* op = out + (t * Hq + h) * hd;
#pragma unroll
    for (int i = 0; i < kDpl; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) op[d] = from_f32<T>(o[i] * inv);
    }
}
}  // namespace

extern "C" int lb_paged_attention(const void* q, const void* k_cache, const void* v_cache, void* out,
                                  const int* block_table, int bt_stride, const int* token_req, const int* positions,
                                  int tokens, int Hq, int Hkv, int hd, int page_size, float scale, int window,
                                  int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (hd <= 0 || hd > kMaxHd || hd % 16 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || page_size <= 0) return kBadSize;
    dim3 grid(tokens, (Hq + kWarps - 1) / kWarps);
    LB_DISPATCH_DTYPE(dtype, paged_attention_kernel<T><<<grid, kWarps * 32, 0, (cudaStream_t)stream>>>(
        (const T*)q, (const T*)k_cache, (const T*)v_cache, (T*)out, block_table, bt_stride, token_req, positions,
        Hq, Hkv, hd, page_size, scale, window));
    return launch_status();
}
