// Rotary position encoding fused with the key multiplier and the paged key/value store.
//
// cos/sin table: row p = [cos(p * inv_freq) | sin(p * inv_freq)] in float32, the angle being the
// float32 product (python/logssms/layers/rotary.py:27-32).  Per (token, head): keys are scaled by the
// key multiplier and rounded BEFORE the rotation; half-split pairing; columns >= rotary_dim pass
// through; keys and values are scattered into the page cache at the token's slot, skipped when the
// slot is negative (python/logssms/kernel/fused.py:161-256).
#include "lb200/common.cuh"
using namespace lb200;

__global__ void rope_table_kernel(float* __restrict__ table, const float* __restrict__ inv_freq, int rows, int half) {
    const int p = blockIdx.x;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float angle = (float)p * inv_freq[i];
        float s, c;
        sincosf(angle, &s, &c);
        table[(size_t)p * 2 * half + i] = c;
        table[(size_t)p * 2 * half + half + i] = s;
    }
}

extern "C" int lb_rope_table(float* table, const float* inv_freq, int rows, int half, void* stream) {
    if (rows <= 0 || half <= 0) return kBadSize;
    rope_table_kernel<<<rows, 64, 0, (cudaStream_t)stream>>>(table, inv_freq, rows, half);
    return launch_status();
}

// grid: (tokens, Hq + 2*Hkv); q/k/v are views with a common row stride (one projection buffer).
template <typename T>
__global__ void rope_kv_store_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                     long row_stride, const int* __restrict__ positions,
                                     const int* __restrict__ slot_mapping, const float* __restrict__ cos_sin,
                                     int table_rows, T* __restrict__ q_out, T* __restrict__ k_cache,
                                     T* __restrict__ v_cache, int Hq, int Hkv, int hd, int rotary_dim,
                                     float key_scale, int write_kv) {
    const size_t t = blockIdx.x;
    int head = blockIdx.y;
    const int half = rotary_dim >> 1;
    int pos = positions[t];
    pos = min(max(pos, 0), table_rows - 1);          // the table has a row for every position the cache manager admits; the clamp only keeps a bad index in bounds
    const float* cs = cos_sin + (size_t)pos * rotary_dim;
    if (head < Hq) {
        const T* src = q + t * row_stride + (size_t)head * hd;
        T* dst = q_out + (t * Hq + head) * hd;
        for (int c = threadIdx.x; c < hd; c += blockDim.x) {
            float val = to_f32(src[c]);
            if (c < rotary_dim) {
                const int f = c < half ? c : c - half;
                const float partner = to_f32(src[c < half ? c + half : c - half]);
                val = val * cs[f] + (c < half ? -partner : partner) * cs[half + f];
            }
            dst[c] = from_f32<T>(val);
        }
        return;
    }
    if (!write_kv) return;
    head -= Hq;
    const long slot = slot_mapping[t];
    if (slot < 0) return;
    if (head < Hkv) {
        const T* src = k + t * row_stride + (size_t)head * hd;
        T* dst = k_cache + ((size_t)slot * Hkv + head) * hd;
        for (int c = threadIdx.x; c < hd; c += blockDim.x) {
            float val = round_to<T>(to_f32(src[c]) * key_scale);
            if (c < rotary_dim) {
                const int f = c < half ? c : c - half;
                const float partner = round_to<T>(to_f32(src[c < half ? c + half : c - half]) * key_scale);
                val = val * cs[f] + (c < half ? -partner : partner) * cs[half + f];
            }
            dst[c] = from_f32<T>(val);
        }
    } else {
        head -= Hkv;
        const T* src = v + t * row_stride + (size_t)head * hd;
        T* dst = v_cache + ((size_t)slot * Hkv + head) * hd;
        for (int c = threadIdx.x; c < hd; c += blockDim.x) dst[c] = src[c];
    }
}

// The same for bfloat16 with 16-byte accesses: a thread owns 8 consecutive columns of one head of one token
// and reads its partner's 8 columns beside them.  Needs hd and rotary_dim / 2 in multiples of 8 and
// 16-byte-aligned rows; the launcher falls back to the kernel above otherwise.
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 p = __bfloat1622float2(h[i]); f[2 * i] = p.x; f[2 * i + 1] = p.y; }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
}

__global__ void __launch_bounds__(256) rope_kv_store_vec_kernel(
        const __nv_bfloat16* __restrict__ qkv, long row_stride, const int* __restrict__ positions,
        const int* __restrict__ slot_mapping, const float* __restrict__ cos_sin, int table_rows,
        __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
        int tokens, int Hq, int Hkv, int hd, int rotary_dim, float key_scale, int write_kv) {
    const int pieces = hd >> 3, heads = Hq + 2 * Hkv;
    const long item = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= (long)tokens * heads * pieces) return;
    const int piece = (int)(item % pieces);
    const int head = (int)((item / pieces) % heads);
    const size_t t = (size_t)(item / ((long)pieces * heads));
    const int c = piece * 8, half = rotary_dim >> 1;
    const __nv_bfloat16* src = qkv + t * row_stride + (size_t)head * hd;
    __nv_bfloat16* dst;
    bool rotate = c < rotary_dim;
    float scale = 1.f;
    if (head < Hq) {
        dst = q_out + (t * Hq + head) * hd;
    } else {
        if (!write_kv) return;
        const long slot = slot_mapping[t];
        if (slot < 0) return;
        if (head < Hq + Hkv) {
            dst = k_cache + ((size_t)slot * Hkv + (head - Hq)) * hd;
            scale = key_scale;
        } else {
            dst = v_cache + ((size_t)slot * Hkv + (head - Hq - Hkv)) * hd;
            rotate = false;
        }
    }
    const uint4 own = *reinterpret_cast<const uint4*>(src + c);
    if (!rotate && scale == 1.f) { *reinterpret_cast<uint4*>(dst + c) = own; return; }
    float x[8];
    unpack8(own, x);
    if (scale != 1.f) {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = round_to<__nv_bfloat16>(x[i] * scale);       // keys: scaled and rounded first
    }
    if (rotate) {
        const bool low = c < half;
        float y[8];
        unpack8(*reinterpret_cast<const uint4*>(src + (low ? c + half : c - half)), y);
        if (scale != 1.f) {
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = round_to<__nv_bfloat16>(y[i] * scale);
        }
        const int pos = min(max(positions[t], 0), table_rows - 1);
        const float* cs = cos_sin + (size_t)pos * rotary_dim + (low ? c : c - half);
        const float4 c0 = *reinterpret_cast<const float4*>(cs), c1 = *reinterpret_cast<const float4*>(cs + 4);
        const float4 s0 = *reinterpret_cast<const float4*>(cs + half), s1 = *reinterpret_cast<const float4*>(cs + half + 4);
        const float co[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float si[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = x[i] * co[i] + (low ? -y[i] : y[i]) * si[i];
    }
    *reinterpret_cast<uint4*>(dst + c) = pack8(x);
}

extern "C" int lb_rope_kv_store(const void* q, const void* k, const void* v, long row_stride, const int* positions,
                                const int* slot_mapping, const float* cos_sin, int table_rows, void* q_out,
                                void* k_cache, void* v_cache, int tokens, int Hq, int Hkv, int hd, int rotary_dim,
                                float key_scale, int write_kv, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (hd <= 0 || rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1) || Hq <= 0 || Hkv <= 0) return kBadSize;
    if (dtype == kBF16 && q == (const char*)k - (size_t)Hq * hd * 2 && v == (const char*)k + (size_t)Hkv * hd * 2 &&
        hd % 8 == 0 && rotary_dim % 16 == 0 && row_stride % 8 == 0 && ((uintptr_t)q & 15) == 0 &&
        ((uintptr_t)q_out & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 &&
        ((uintptr_t)cos_sin & 15) == 0) {
        const long items = (long)tokens * (Hq + 2 * Hkv) * (hd / 8);
        rope_kv_store_vec_kernel<<<(unsigned)((items + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)q, row_stride, positions, slot_mapping, cos_sin, table_rows, (__nv_bfloat16*)q_out,
            (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, tokens, Hq, Hkv, hd, rotary_dim, key_scale, write_kv);
        return launch_status();
    }
    dim3 grid(tokens, Hq + 2 * Hkv);
    const int threads = hd <= 32 ? 32 : (hd <= 64 ? 64 : 128);
    LB_DISPATCH_DTYPE(dtype, rope_kv_store_kernel<T><<<grid, threads, 0, (cudaStream_t)stream>>>(
        (const T*)q, (const T*)k, (const T*)v, row_stride, positions, slot_mapping, cos_sin, table_rows,
        (T*)q_out, (T*)k_cache, (T*)v_cache, Hq, Hkv, hd, rotary_dim, key_scale, write_kv));
    return launch_status();
}
