// Split-KV attention over the paged cache for decoded tokens and short prompt portions.
//
// A decode step is bound by reading keys and values: every (token, key/value head) pair has to
// stream its whole context once.  This kernel packs the query heads that share a key/value head
// into one CTA (keys and values are read once for all of them) and cuts each context into
// `splits` ranges so that a handful of tokens still fills the 148 SMs; a second small kernel
// merges the ranges' partial results.
//
//   grid  (tokens, kv heads x head tiles, splits), 128 threads = 4 warps
//   warp  32-key tiles of the CTA's range, round robin.  Scores: lane = key, the key row is read in
//         16-byte pieces and multiplied with the (pre-scaled, float32) queries held in shared
//         memory.  Softmax is the online form per warp (max by shuffles, the running sum per lane).
//         Values: the 32 x head_dim tile is read in 16-byte pieces, lane = (key, piece), and each
//         lane keeps 8 output columns per query head; lanes that hold the same columns are summed
//         at the end.
//   end   the four warps' (max, sum, output) are merged in shared memory; with one split the
//         normalised output is written, otherwise the unnormalised output and (max, sum) go to
//         scratch for `attn_merge_kernel`.
//
// Each token is handled on its own (causal over absolute positions, optional sliding window), so
// the kernel serves any mix of requests; `token_list` restricts it to some tokens of the batch.
// All statistics and accumulators are 32-bit, exp is expf.  Head sizes: multiples of 16 up to 256.
// Formula: python/logssms/layers/attention_backend/fi.py:175-190 (causal, scale head_dim^-1/2).
#include "lb200/common.cuh"
using namespace lb200;

namespace {
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;

struct DecodeArgs {
    const void* q; const void* k_cache; const void* v_cache; void* out;
    const int* block_table; int bt_stride;
    const int* token_req; const int* positions; const int* token_list;
    float* part_o; float* part_ml;
    int Hq, Hkv, hd, page_size, window, splits, head_tiles;
    float scale;
};

// eight consecutive elements as floats
__device__ __forceinline__ void load8(const float* p, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

// GT: query heads per CTA.  CHP: 8-element pieces per value row, rounded up to a power of two (2..32).
template <typename T, int GT, int CHP>
__global__ void __launch_bounds__(kThreads) attn_split_kernel(DecodeArgs a) {
    extern __shared__ float smem[];
    const int hd = a.hd;
    float* q_s = smem;                                   // [GT][hd]
    float* mrg = smem + GT * hd;                         // [kWarps][GT][hd + 2]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sel = blockIdx.x;
    const size_t t = a.token_list ? a.token_list[sel] : sel;
    const int kvh = blockIdx.y / a.head_tiles, ht = blockIdx.y % a.head_tiles;
    const int G = a.Hq / a.Hkv;
    const int h0 = kvh * G + ht * GT;
    const int nheads = min(GT, G - ht * GT);
    const int split = blockIdx.z;
    const int pos = a.positions[t];
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int n = pos - lo + 1;
    const int chunk = (((n + a.splits - 1) / a.splits) + 31) / 32 * 32;
    const int begin = lo + split * chunk;
    const int end = min(begin + chunk, pos + 1);
    const int* bt = a.block_table + (size_t)a.token_req[t] * a.bt_stride;
    const T* qp = (const T*)a.q + (t * a.Hq + h0) * hd;
    for (int i = threadIdx.x; i < GT * hd; i += kThreads)
        q_s[i] = (i / hd) < nheads ? to_f32(qp[i]) * a.scale : 0.f;
    __syncthreads();

    constexpr int KPI = 32 / CHP;                        // keys per value-load instruction
    const int piece = lane % CHP, ksub = lane / CHP;
    const bool piece_ok = piece * 8 < hd;
    float acc[GT][8];
    float m[GT], l[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
    }
    const T* kc = (const T*)a.k_cache;
    const T* vc = (const T*)a.v_cache;
    const int pieces = hd / 8;

    for (int j0 = begin + warp * 32; j0 < end; j0 += kWarps * 32) {
        const int j = j0 + lane;
        const bool valid = j < end;
        long row = 0;
        float s[GT];
#pragma unroll
        for (int g = 0; g < GT; ++g) s[g] = 0.f;
        if (valid) {
            row = (long)bt[j / a.page_size] * a.page_size + (j % a.page_size);
            const T* kp = kc + ((size_t)row * a.Hkv + kvh) * hd;
#pragma unroll 4
            for (int c = 0; c < pieces; ++c) {
                float f[8];
                load8(kp + c * 8, f);
#pragma unroll
                for (int g = 0; g < GT; ++g) {
                    const float* qg = q_s + g * hd + c * 8;
#pragma unroll
                    for (int e = 0; e < 8; ++e) s[g] = fmaf(qg[e], f[e], s[g]);
                }
            }
        }
        float p[GT];
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            const float m_new = fmaxf(m[g], warp_max(valid ? s[g] : -INFINITY));
            const float alpha = expf(m[g] - m_new);          // m = -inf at first: exp(-inf) = 0
            p[g] = valid ? expf(s[g] - m_new) : 0.f;
            l[g] = l[g] * alpha + p[g];
            m[g] = m_new;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] *= alpha;
        }
        const int count = min(32, end - j0);
#pragma unroll 4
        for (int i = 0; i < CHP; ++i) {
            const int key = i * KPI + ksub;
            const long rj = __shfl_sync(0xffffffffu, row, key);
            float pj[GT];
#pragma unroll
            for (int g = 0; g < GT; ++g) pj[g] = __shfl_sync(0xffffffffu, p[g], key);
            if (key < count && piece_ok) {
                float f[8];
                load8(vc + ((size_t)rj * a.Hkv + kvh) * hd + piece * 8, f);
#pragma unroll
                for (int g = 0; g < GT; ++g)
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pj[g], f[e], acc[g][e]);
            }
        }
    }
    // lanes that hold the same columns -> lane `piece`
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        l[g] = warp_sum(l[g]);
#pragma unroll
        for (int o = CHP; o < 32; o <<= 1)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], o);
    }
    const int stride = hd + 2;
    if (lane < CHP && piece_ok) {
#pragma unroll
        for (int g = 0; g < GT; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) mrg[(warp * GT + g) * stride + piece * 8 + e] = acc[g][e];
    }
    if (lane == 0) {
#pragma unroll
        for (int g = 0; g < GT; ++g) { mrg[(warp * GT + g) * stride + hd] = m[g]; mrg[(warp * GT + g) * stride + hd + 1] = l[g]; }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nheads * hd; i += kThreads) {
        const int g = i / hd, d = i % hd;
        float mt = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mt = fmaxf(mt, mrg[(w * GT + g) * stride + hd]);
        float lt = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float mw = mrg[(w * GT + g) * stride + hd];
            const float f = mw == -INFINITY ? 0.f : expf(mw - mt);
            lt += mrg[(w * GT + g) * stride + hd + 1] * f;
            o += mrg[(w * GT + g) * stride + d] * f;
        }
        const int h = h0 + g;
        if (a.splits == 1) {
            ((T*)a.out)[(t * a.Hq + h) * hd + d] = from_f32<T>(o / lt);
        } else {
            const size_t slot = ((size_t)sel * a.Hq + h) * a.splits + split;
            a.part_o[slot * hd + d] = o;
            if (d == 0) { a.part_ml[slot * 2] = mt; a.part_ml[slot * 2 + 1] = lt; }
        }
    }
}

// grid (selected tokens, query heads); one thread per output column.  The ranges' (max, sum) pairs are
// read once into shared memory, where every range gets its weight exp(max_s - max); the columns are then
// weighted sums of independent, coalesced loads.
constexpr int kMaxMergeSplits = 1024;

template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  T* __restrict__ out, const int* __restrict__ token_list, int Hq, int hd, int splits) {
    pdl_trigger();
    extern __shared__ float w_s[];                     // [splits] weights, then [32] for the reductions
    float* red = w_s + splits;
    const int sel = blockIdx.x, h = blockIdx.y;
    const size_t t = token_list ? token_list[sel] : sel;
    const size_t base = ((size_t)sel * Hq + h) * splits;
    float mt = -INFINITY;
    for (int s = threadIdx.x; s < splits; s += blockDim.x) mt = fmaxf(mt, part_ml[(base + s) * 2]);
    mt = block_max(mt, red);
    float lt = 0.f;
    for (int s = threadIdx.x; s < splits; s += blockDim.x) {
        const float ms = part_ml[(base + s) * 2];
        const float f = ms == -INFINITY ? 0.f : expf(ms - mt);      // an empty range has weight 0
        w_s[s] = f;
        lt += part_ml[(base + s) * 2 + 1] * f;
    }
    lt = block_sum(lt, red);                           // (its barriers also publish w_s)
    const float inv = 1.f / lt;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) o = fmaf(part_o[(base + s) * hd + d], w_s[s], o);
        out[(t * Hq + h) * hd + d] = from_f32<T>(o * inv);
    }
}

template <typename T, int GT>
int launch_chp(const DecodeArgs& a, int sel_tokens, cudaStream_t s) {
    const int pieces = a.hd / 8;
    dim3 grid(sel_tokens, a.Hkv * a.head_tiles, a.splits);
    const size_t smem = (size_t)(GT * a.hd + kWarps * GT * (a.hd + 2)) * sizeof(float);
#define LB_CHP(N)                                                                                          \
    {                                                                                                      \
        if (smem > 48 * 1024)                                                                              \
            cudaFuncSetAttribute(attn_split_kernel<T, GT, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        attn_split_kernel<T, GT, N><<<grid, kThreads, smem, s>>>(a);                                       \
    }
    if (pieces <= 2) LB_CHP(2)
    else if (pieces <= 4) LB_CHP(4)
    else if (pieces <= 8) LB_CHP(8)
    else if (pieces <= 16) LB_CHP(16)
    else LB_CHP(32)
#undef LB_CHP
    return launch_status();
}

template <typename T>
int launch(DecodeArgs a, int sel_tokens, cudaStream_t s) {
    const int G = a.Hq / a.Hkv;
    const int gt = G >= 8 ? 8 : (G > 2 ? 4 : (G == 2 ? 2 : 1));
    a.head_tiles = (G + gt - 1) / gt;
    int rc;
    switch (gt) {
        case 1: rc = launch_chp<T, 1>(a, sel_tokens, s); break;
        case 2: rc = launch_chp<T, 2>(a, sel_tokens, s); break;
        case 4: rc = launch_chp<T, 4>(a, sel_tokens, s); break;
        default: rc = launch_chp<T, 8>(a, sel_tokens, s); break;
    }
    if (rc != 0 || a.splits == 1) return rc;
    dim3 grid(sel_tokens, a.Hq);
    const int threads = a.hd <= 32 ? 32 : (a.hd <= 64 ? 64 : 128);
    attn_merge_kernel<T><<<grid, threads, (a.splits + 32) * sizeof(float), s>>>(a.part_o, a.part_ml, (T*)a.out, a.token_list,
                                                                                a.Hq, a.hd, a.splits);
    return launch_status();
}
}  // namespace

// `part_o`: float32 [sel_tokens, Hq, splits, hd]; `part_ml`: float32 [sel_tokens, Hq, splits, 2];
// both may be null when splits == 1.  `token_list`: the tokens to run (null: the first `sel_tokens`).
extern "C" int lb_attention_decode(const void* q, const void* k_cache, const void* v_cache, void* out,
                                   const int* block_table, int bt_stride, const int* token_req,
                                   const int* positions, const int* token_list, int sel_tokens, int Hq, int Hkv,
                                   int hd, int page_size, float scale, int window, int splits, float* part_o,
                                   float* part_ml, int dtype, void* stream) {
    if (sel_tokens <= 0) return kOk;
    if (hd <= 0 || hd > 256 || hd % 16 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || page_size <= 0 || splits < 1)
        return kBadSize;
    if (splits > 1 && (part_o == nullptr || part_ml == nullptr)) return kBadSize;
    if (splits > kMaxMergeSplits || (long)Hkv * ((Hq / Hkv + 7) / 8 + 1) > 65535) return kTooLarge;
    DecodeArgs a{q, k_cache, v_cache, out, block_table, bt_stride, token_req, positions, token_list, part_o, part_ml,
                 Hq, Hkv, hd, page_size, window, splits, 1, scale};
    LB_DISPATCH_DTYPE(dtype, return launch<T>(a, sel_tokens, (cudaStream_t)stream));
    return kOk;
}

// ------------------------------------------------------------------------------------------------
// The same attention without any allocation: the ranges' partial results live in a fixed array of
// this library's device data segment.  Declaration, limits and rules: lb200/attention_decode_static.h.
// No counterpart in the reference.
#include <mutex>
#include <stdio.h>

#include "lb200/attention_decode_static.h"

namespace {
// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_static_scratch[LB_ATTN_STATIC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_static_scratch_addr[kMaxDevices] = {};
std::mutex g_static_scratch_mutex;

int refuse(char* err, size_t err_len, int code, const char* fmt, long a = 0, long b = 0) {
    if (err != nullptr && err_len > 0) snprintf(err, err_len, fmt, a, b);
    return code;
}

// Device address of the array on the current device; looked up once per device.
int static_scratch_address(float** addr, char* err, size_t err_len) {
    int device = -1;
    cudaError_t rc = cudaGetDevice(&device);
    if (rc != cudaSuccess) return refuse(err, err_len, (int)rc, "cudaGetDevice failed: CUDA error %ld", (long)rc);
    if (device < 0 || device >= kMaxDevices)
        return refuse(err, err_len, kTooLarge, "device index %ld is beyond the %ld this entry point tracks", device, kMaxDevices);
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_addr[device] == nullptr) {
        float* p = nullptr;
        rc = cudaGetSymbolAddress((void**)&p, g_static_scratch);
        if (rc != cudaSuccess || p == nullptr)
            return refuse(err, err_len, rc != cudaSuccess ? (int)rc : (int)cudaErrorInvalidSymbol,
                          "cudaGetSymbolAddress of the static scratch failed: CUDA error %ld", (long)rc);
        g_static_scratch_addr[device] = p;
    }
    *addr = g_static_scratch_addr[device];
    return kOk;
}
}  // namespace

extern "C" int lb_attention_decode_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                          const int* block_table, int bt_stride, const int* token_req,
                                          const int* positions, const int* token_list, int sel_tokens, int Hq,
                                          int Hkv, int hd, int page_size, float scale, int window, int splits,
                                          int dtype, void* stream, char* err, size_t err_len) {
    if (err != nullptr && err_len > 0) err[0] = '\0';
    if (sel_tokens <= 0) return kOk;
    if (hd <= 0 || hd > 256 || hd % 16 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || page_size <= 0 || splits < 1)
        return refuse(err, err_len, kBadSize, "a size the kernel does not take (head_dim %ld in steps of 16 up to 256, "
                      "query heads a multiple of key/value heads, splits %ld >= 1)", hd, splits);
    if (splits > kMaxMergeSplits || (long)Hkv * ((Hq / Hkv + 7) / 8 + 1) > 65535)
        return refuse(err, err_len, kTooLarge, "too many ranges (%ld) or key/value heads (%ld) for one grid", splits, Hkv);
    if (dtype != kF32 && dtype != kBF16) return refuse(err, err_len, kBadDType, "dtype code %ld is neither float32 (0) nor bfloat16 (1)", dtype);
    const size_t slots = (size_t)sel_tokens * (size_t)Hq * (size_t)splits;
    const size_t need = slots * (size_t)(hd + 2);
    if (need > (size_t)LB_ATTN_STATIC_SCRATCH_FLOATS)
        return refuse(err, err_len, LB_ERR_STATIC_SCRATCH,
                      "this call needs %ld floats of scratch, the static array holds %ld: use fewer ranges or tokens per call",
                      (long)need, (long)LB_ATTN_STATIC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    const int rc = static_scratch_address(&scratch, err, err_len);
    if (rc != kOk) return rc;
    // partial outputs first (slots * hd floats, 256-byte aligned start), then the (max, sum) pairs
    float* part_o = scratch;
    float* part_ml = scratch + slots * (size_t)hd;
    DecodeArgs a{q, k_cache, v_cache, out, block_table, bt_stride, token_req, positions, token_list, part_o, part_ml,
                 Hq, Hkv, hd, page_size, window, splits, 1, scale};
    int launched = kOk;
    if (dtype == kF32) launched = launch<float>(a, sel_tokens, (cudaStream_t)stream);
    else launched = launch<__nv_bfloat16>(a, sel_tokens, (cudaStream_t)stream);
    if (launched != kOk) return refuse(err, err_len, launched, "kernel launch failed: CUDA error %ld", launched);
    return kOk;
}
