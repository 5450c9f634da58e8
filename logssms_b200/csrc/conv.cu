// Depthwise causal conv1d over packed portions, with per-request history kept in state slots.
//
//   u_t[ch]  = round(xBC_t[ch] * region_scale(ch))                (three regions: x | B | C)
//   c_t[ch]  = sum_{j<K} w[ch, j] * u_{t-(K-1)+j}[ch] (+ bias[ch])  ; inputs before the portion come
//              from the request's conv state (zeros when the request starts at position 0)
//   out_t    = round(silu(round(c_t)))
//   state'   = the last K-1 scaled inputs u, oldest first
// (python/logssms/kernel/linear_attention/packed_conv.py:96-140; decode form
// python/logssms/kernel/linear_attention/conv_decode.py:112-278.)
//
// Long portions take two launches: the forward kernel only READS the state (grid over token chunks, so
// a long prompt spreads over many CTAs), the update kernel then rewrites it, one thread per (request,
// channel).  When no portion is longer than one chunk (every decode step) a thread is the only reader
// of its (request, channel) state, so the forward kernel rewrites it itself and the step is one launch.
#include "lb200/common.cuh"
using namespace lb200;

namespace {
constexpr int kChunk = 64;

struct ConvArgs {
    const void* x; long x_stride;          // [tokens, C] view, row stride in elements
    const float* weight;                   // [C, K]
    const float* bias;                     // [C] or null
    void* state;                           // [slots, C, K-1]
    void* out;                             // [tokens, C] contiguous
    const int* cu_seqlens; const int* start_pos; const int* slots;
    int C; int end0; int end1; float s0; float s1; float s2;
};

template <typename T>
__device__ __forceinline__ float scaled_input(const ConvArgs& a, long token, int c, float scale) {
    return round_to<T>(to_f32(((const T*)a.x)[token * a.x_stride + c]) * scale);
}

template <typename T, int K, bool UPDATE>
__global__ void conv_forward_kernel(ConvArgs a) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.C) return;
    const int b = blockIdx.z;
    const int begin = a.cu_seqlens[b], len = a.cu_seqlens[b + 1] - begin;
    const int t0 = blockIdx.y * kChunk;
    if (t0 >= len) return;
    const int t1 = min(len, t0 + kChunk);
    const float scale = c < a.end0 ? a.s0 : (c < a.end1 ? a.s1 : a.s2);
    const bool has_history = a.start_pos[b] > 0;
    const T* st = (const T*)a.state + ((size_t)a.slots[b] * a.C + c) * (K - 1);
    float w[K], win[K];
#pragma unroll
    for (int j = 0; j < K; ++j) w[j] = a.weight[(size_t)c * K + j];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
        const int idx = t0 - (K - 1) + j;                 // relative to the portion's first token
        win[j] = idx >= 0 ? scaled_input<T>(a, begin + idx, c, scale)
                          : (has_history ? to_f32(st[K - 1 + idx]) : 0.f);
    }
    const float bias = a.bias ? a.bias[c] : 0.f;
    for (int t = t0; t < t1; ++t) {
        win[K - 1] = scaled_input<T>(a, begin + t, c, scale);
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < K; ++j) acc += win[j] * w[j];
        acc = round_to<T>(acc + bias);
        ((T*)a.out)[(size_t)(begin + t) * a.C + c] = from_f32<T>(silu_f(acc));
#pragma unroll
        for (int j = 0; j < K - 1; ++j) win[j] = win[j + 1];
    }
    if (UPDATE) {                                         // single chunk: win holds the last K-1 inputs
        T* st_w = (T*)a.state + ((size_t)a.slots[b] * a.C + c) * (K - 1);
#pragma unroll
        for (int j = 0; j < K - 1; ++j) st_w[j] = from_f32<T>(win[j]);
    }
}

template <typename T, int K>
__global__ void conv_state_update_kernel(ConvArgs a) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.C) return;
    const int b = blockIdx.y;
    const int begin = a.cu_seqlens[b], len = a.cu_seqlens[b + 1] - begin;
    if (len <= 0) return;
    const float scale = c < a.end0 ? a.s0 : (c < a.end1 ? a.s1 : a.s2);
    const bool has_history = a.start_pos[b] > 0;
    T* st = (T*)a.state + ((size_t)a.slots[b] * a.C + c) * (K - 1);
    float next[K];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
        const int idx = len - (K - 1) + j;
        next[j] = idx >= 0 ? scaled_input<T>(a, begin + idx, c, scale)
                           : (has_history ? to_f32(st[K - 1 + idx]) : 0.f);
    }
#pragma unroll
    for (int j = 0; j < K - 1; ++j) st[j] = from_f32<T>(next[j]);
}

// The same for bfloat16 with eight channels per thread and 16-byte loads and stores: channels, the region
// edges and the row stride must be multiples of 8 and the input 16-byte aligned.  A thread walks
// kVecChunk tokens; their rows are fetched in batches so that several loads are in flight.
constexpr int kVecChunk = 8;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 p = __bfloat1622float2(h[i]); f[2 * i] = p.x; f[2 * i + 1] = p.y; }
}

template <int K, bool UPDATE>
__global__ void __launch_bounds__(128) conv_forward_vec_kernel(ConvArgs a) {
    typedef __nv_bfloat16 T;
    static_assert(K - 1 <= kVecChunk, "only a portion's first chunk may reach back into the saved inputs");
    const int cg = blockIdx.x * blockDim.x + threadIdx.x;
    const int c = cg * 8;
    if (c >= a.C) return;
    const int b = blockIdx.z;
    const int begin = a.cu_seqlens[b], len = a.cu_seqlens[b + 1] - begin;
    const int t0 = blockIdx.y * kVecChunk;
    if (t0 >= len) return;
    const int n = min(len - t0, kVecChunk);
    const float scale = c < a.end0 ? a.s0 : (c < a.end1 ? a.s1 : a.s2);
    const bool has_history = a.start_pos[b] > 0;
    const T* x = (const T*)a.x;
    T* st = (T*)a.state + ((size_t)a.slots[b] * a.C + c) * (K - 1);
    // The rows of the chunk, the thread's taps (8 * K consecutive floats) and its biases are fetched as 16-byte
    // pieces up front, so that all of them are in flight together: one after the other, each waited for,
    // they were most of the kernel's time.
    uint4 rows[kVecChunk];
#pragma unroll
    for (int i = 0; i < kVecChunk; ++i)
        if (i < n) rows[i] = *reinterpret_cast<const uint4*>(x + (size_t)(begin + t0 + i) * a.x_stride + c);
    float w[8][K], win[8][K], bias[8];
    {
        float4 raw[2 * K];
        const float4* wp = reinterpret_cast<const float4*>(a.weight + (size_t)c * K);
#pragma unroll
        for (int i = 0; i < 2 * K; ++i) raw[i] = __ldg(wp + i);
        float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
        if (a.bias) { b0 = __ldg(reinterpret_cast<const float4*>(a.bias + c)); b1 = __ldg(reinterpret_cast<const float4*>(a.bias + c) + 1); }
        bias[0] = b0.x; bias[1] = b0.y; bias[2] = b0.z; bias[3] = b0.w; bias[4] = b1.x; bias[5] = b1.y; bias[6] = b1.z; bias[7] = b1.w;
        const float* flat = reinterpret_cast<const float*>(raw);
#pragma unroll
        for (int e = 0; e < 8; ++e)
#pragma unroll
            for (int j = 0; j < K; ++j) w[e][j] = flat[e * K + j];
    }
    // the thread's 8 channels' saved inputs are 8 * (K - 1) consecutive values: K - 1 pieces of 16 bytes, asked for
    // together (one 2-byte load per value made a decode step's conv a chain of dependent loads)
    __align__(16) T hist[8 * (K - 1)];
    if (has_history && t0 == 0) {
#pragma unroll
        for (int j = 0; j < K - 1; ++j) reinterpret_cast<uint4*>(hist)[j] = reinterpret_cast<const uint4*>(st)[j];
    }
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
        const int idx = t0 - (K - 1) + j;
        if (idx >= 0) {
            float f[8];
            unpack8(*reinterpret_cast<const uint4*>(x + (size_t)(begin + idx) * a.x_stride + c), f);
#pragma unroll
            for (int e = 0; e < 8; ++e) win[e][j] = round_to<T>(f[e] * scale);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e)                  // idx < 0 only in the portion's first chunk: idx = j - (K - 1)
                win[e][j] = has_history ? __bfloat162float(hist[e * (K - 1) + j]) : 0.f;
        }
    }
#pragma unroll
    for (int i = 0; i < kVecChunk; ++i) {
        if (i < n) {
            float f[8];
            unpack8(rows[i], f);
            __nv_bfloat162 o[4];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                win[e][K - 1] = round_to<T>(f[e] * scale);
                float acc = 0.f;
#pragma unroll
                for (int j = 0; j < K; ++j) acc += win[e][j] * w[e][j];
                acc = round_to<T>(acc + bias[e]);
                acc = silu_fast(acc);                            // the result is rounded to bfloat16 next
                if (e & 1) o[e >> 1].y = __float2bfloat16_rn(acc); else o[e >> 1].x = __float2bfloat16_rn(acc);
#pragma unroll
                for (int j = 0; j < K - 1; ++j) win[e][j] = win[e][j + 1];
            }
            *reinterpret_cast<uint4*>((T*)a.out + (size_t)(begin + t0 + i) * a.C + c) = *reinterpret_cast<uint4*>(o);
        }
    }
    if (UPDATE) {
        __align__(16) T next[8 * (K - 1)];
#pragma unroll
        for (int e = 0; e < 8; ++e)
#pragma unroll
            for (int j = 0; j < K - 1; ++j) next[e * (K - 1) + j] = __float2bfloat16_rn(win[e][j]);
#pragma unroll
        for (int j = 0; j < K - 1; ++j) reinterpret_cast<uint4*>(st)[j] = reinterpret_cast<const uint4*>(next)[j];
    }
}

// Long portions (bfloat16, the same alignment rules): a CTA of 256 threads stages kTileTokens + K - 1 rows of 256
// channels in shared memory, already scaled and rounded, each row fetched once with 16-byte loads that are all in
// flight together; a thread then walks 4 consecutive tokens of 8 channels.  One thread per 32 outputs instead of
// per 64 with the rows shared through shared memory: four times the warps of the register form above, which at
// 2,048 tokens left the SMs a dozen warps each.
constexpr int kTileTokens = 64, kTileGroups = 32, kTileThreads = 256;

template <int K>
__global__ void __launch_bounds__(kTileThreads, 3) conv_forward_tile_kernel(ConvArgs a) {
    typedef __nv_bfloat16 T;
    constexpr int kRows = kTileTokens + K - 1;
    __shared__ __align__(16) T tile[kRows][kTileGroups * 8];
    const int b = blockIdx.z;
    const int begin = a.cu_seqlens[b], len = a.cu_seqlens[b + 1] - begin;
    const int t0 = blockIdx.y * kTileTokens;
    if (t0 >= len) return;
    const int c0 = blockIdx.x * kTileGroups * 8;
    const bool has_history = a.start_pos[b] > 0;
    const T* x = (const T*)a.x;
    const T* st = (const T*)a.state + (size_t)a.slots[b] * a.C * (K - 1);
    const int g = threadIdx.x % kTileGroups, ts = threadIdx.x / kTileGroups;
    const int c = c0 + g * 8;
    const bool live = c < a.C;
    // The CTA's taps and biases go through shared memory: its 256 channels are one contiguous run of K * 256 floats,
    // fetched coalesced.  (A thread fetching its own 8 * K floats makes every load instruction of a warp touch 32
    // different lines; that was most of this kernel's time.)  A thread's 8 channels lie 8 * K + 4 floats from the
    // next thread's, so that the 16-byte reads below spread over all banks.
    constexpr int kWPitch = 8 * K + 4;
    __shared__ __align__(16) float w_s[kTileGroups * kWPitch];
    __shared__ __align__(16) float bias_s[kTileGroups * 8];
    for (int f = threadIdx.x; f < kTileGroups * 8 * K; f += kTileThreads) {
        const int ch = f / K, j = f - ch * K;
        w_s[(ch >> 3) * kWPitch + (ch & 7) * K + j] = c0 + ch < a.C ? __ldg(a.weight + (size_t)c0 * K + f) : 0.f;
    }
    bias_s[threadIdx.x] = (a.bias != nullptr && c0 + (int)threadIdx.x < a.C) ? __ldg(a.bias + c0 + threadIdx.x) : 0.f;
    // rows t0 - (K - 1) .. t0 + kTileTokens - 1 of the portion; row rr of the tile, channel group g
    constexpr int kPer = (kRows + kTileThreads / kTileGroups - 1) / (kTileThreads / kTileGroups);
    const float scale = c < a.end0 ? a.s0 : (c < a.end1 ? a.s1 : a.s2);
    uint4 fetched[kPer];
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        const int rr = ts + i * (kTileThreads / kTileGroups), idx = t0 - (K - 1) + rr;
        if (live && rr < kRows && idx >= 0 && idx < len)
            fetched[i] = *reinterpret_cast<const uint4*>(x + (size_t)(begin + idx) * a.x_stride + c);
    }
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        const int rr = ts + i * (kTileThreads / kTileGroups), idx = t0 - (K - 1) + rr;
        if (!live || rr >= kRows) continue;
        __nv_bfloat162 o[4];
        if (idx >= 0 && idx < len) {
            float f[8];
            unpack8(fetched[i], f);
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = __floats2bfloat162_rn(f[2 * e] * scale, f[2 * e + 1] * scale);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) {                 // before the portion: the saved inputs, or zeros
                const T v = (idx < 0 && has_history) ? st[(size_t)(c + e) * (K - 1) + K - 1 + idx] : __float2bfloat16_rn(0.f);
                if (e & 1) o[e >> 1].y = v; else o[e >> 1].x = v;
            }
        }
        *reinterpret_cast<uint4*>(&tile[rr][g * 8]) = *reinterpret_cast<uint4*>(o);
    }
    __syncthreads();
    if (!live) return;
    float w[8][K], bias[8];
    {
        const float* flat = w_s + g * kWPitch;            // K * 8 floats: 16-byte reads when K is even, else single ones
#pragma unroll
        for (int e = 0; e < 8; ++e)
#pragma unroll
            for (int j = 0; j < K; ++j) w[e][j] = flat[e * K + j];
#pragma unroll
        for (int e = 0; e < 8; ++e) bias[e] = bias_s[g * 8 + e];
    }
    constexpr int kWalk = kTileTokens / (kTileThreads / kTileGroups);      // 4 consecutive tokens per thread
    const int first = ts * kWalk;
    float win[8][K];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(&tile[first + j][g * 8]), f);
#pragma unroll
        for (int e = 0; e < 8; ++e) win[e][j] = f[e];
    }
#pragma unroll
    for (int i = 0; i < kWalk; ++i) {
        const int t = t0 + first + i;
        if (t >= len) break;
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(&tile[first + i + K - 1][g * 8]), f);
        __nv_bfloat162 o[4];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            win[e][K - 1] = f[e];
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < K; ++j) acc += win[e][j] * w[e][j];
            acc = round_to<T>(acc + bias[e]);
            acc = silu_fast(acc);                            // the result is rounded to bfloat16 next
            if (e & 1) o[e >> 1].y = __float2bfloat16_rn(acc); else o[e >> 1].x = __float2bfloat16_rn(acc);
#pragma unroll
            for (int j = 0; j < K - 1; ++j) win[e][j] = win[e][j + 1];
        }
        *reinterpret_cast<uint4*>((T*)a.out + (size_t)(begin + t) * a.C + c) = *reinterpret_cast<uint4*>(o);
    }
}

template <int K>
void launch_vec(const ConvArgs& a, int B, int max_len, cudaStream_t s) {
    const int threads = 128, groups = a.C / 8;
    dim3 grid_f((groups + threads - 1) / threads, (max_len + kVecChunk - 1) / kVecChunk, B);
    if (max_len <= kVecChunk) {
        conv_forward_vec_kernel<K, true><<<grid_f, threads, 0, s>>>(a);
    } else {
        dim3 grid_u((a.C + threads - 1) / threads, B);
        dim3 grid_t((groups + kTileGroups - 1) / kTileGroups, (max_len + kTileTokens - 1) / kTileTokens, B);
        conv_forward_tile_kernel<K><<<grid_t, kTileThreads, 0, s>>>(a);
        conv_state_update_kernel<__nv_bfloat16, K><<<grid_u, threads, 0, s>>>(a);
    }
}

inline bool vec_ok(const ConvArgs& a, int dtype) {
    return dtype == kBF16 && a.C % 8 == 0 && a.end0 % 8 == 0 && a.end1 % 8 == 0 && a.x_stride % 8 == 0 &&
           ((uintptr_t)a.x & 15) == 0 && ((uintptr_t)a.out & 15) == 0 && ((uintptr_t)a.weight & 15) == 0 &&
           ((uintptr_t)a.state & 15) == 0 &&
           (a.bias == nullptr || ((uintptr_t)a.bias & 15) == 0);
}

template <typename T>
int launch(const ConvArgs& a, int B, int K, int max_len, cudaStream_t s) {
    const int threads = 128;
    dim3 grid_f((a.C + threads - 1) / threads, (max_len + kChunk - 1) / kChunk, B);
    dim3 grid_u((a.C + threads - 1) / threads, B);
#define LB_CONV_K(KK)                                                         \
    case KK:                                                                  \
        if (max_len <= kChunk) {                                              \
            conv_forward_kernel<T, KK, true><<<grid_f, threads, 0, s>>>(a);   \
        } else {                                                              \
            conv_forward_kernel<T, KK, false><<<grid_f, threads, 0, s>>>(a);  \
            conv_state_update_kernel<T, KK><<<grid_u, threads, 0, s>>>(a);    \
        }                                                                     \
        break;
    switch (K) {
        LB_CONV_K(2) LB_CONV_K(3) LB_CONV_K(4) LB_CONV_K(5) LB_CONV_K(6) LB_CONV_K(7) LB_CONV_K(8)
        default: return kBadSize;
    }
#undef LB_CONV_K
    return launch_status();
}
}  // namespace

extern "C" int lb_causal_conv1d(const void* x, long x_stride, const float* weight, const float* bias, void* state,
                                void* out, const int* cu_seqlens, const int* start_pos, const int* slots, int B,
                                int max_len, int C, int K, int end0, int end1, float s0, float s1, float s2,
                                int dtype, void* stream) {
    if (B <= 0 || max_len <= 0) return kOk;
    if (C <= 0 || K < 2 || K > 8) return kBadSize;
    ConvArgs a{x, x_stride, weight, bias, state, out, cu_seqlens, start_pos, slots, C, end0, end1, s0, s1, s2};
    if (vec_ok(a, dtype) && K <= 5) {
        switch (K) {
            case 2: launch_vec<2>(a, B, max_len, (cudaStream_t)stream); break;
            case 3: launch_vec<3>(a, B, max_len, (cudaStream_t)stream); break;
            case 4: launch_vec<4>(a, B, max_len, (cudaStream_t)stream); break;
            default: launch_vec<5>(a, B, max_len, (cudaStream_t)stream); break;
        }
        return launch_status();
    }
    LB_DISPATCH_DTYPE(dtype, return launch<T>(a, B, K, max_len, (cudaStream_t)stream));
    return kOk;
}
