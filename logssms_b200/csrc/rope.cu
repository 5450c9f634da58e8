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
    pos = min(max(pos, 0), table_rows - 1);          // the host refuses positions beyond the table
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

extern "C" int lb_rope_kv_store(const void* q, const void* k, const void* v, long row_stride, const int* positions,
                                const int* slot_mapping, const float* cos_sin, int table_rows, void* q_out,
                                void* k_cache, void* v_cache, int tokens, int Hq, int Hkv, int hd, int rotary_dim,
                                float key_scale, int write_kv, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (hd <= 0 || rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1) || Hq <= 0 || Hkv <= 0) return kBadSize;
    dim3 grid(tokens, Hq + 2 * Hkv);
    const int threads = hd <= 32 ? 32 : (hd <= 64 ? 64 : 128);
    LB_DISPATCH_DTYPE(dtype, rope_kv_store_kernel<T><<<grid, threads, 0, (cudaStream_t)stream>>>(
        (const T*)q, (const T*)k, (const T*)v, row_stride, positions, slot_mapping, cos_sin, table_rows,
        (T*)q_out, (T*)k_cache, (T*)v_cache, Hq, Hkv, hd, rotary_dim, key_scale, write_kv));
    return launch_status();
}
