// Embedding row gather fused with the embedding multiplier.
//   out[t, :] = round(table[ids[t], :] * multiplier)
// Replaces the reference's gather kernel (csrc/jit/index.cu) plus the separate multiply of
// python/logssms/models/falcon_h1.py:213.  Ids outside [0, vocab) are clamped and counted in
// `bad_ids` (a device int the host may read); they never index out of the table.
#include "lb200/common.cuh"
using namespace lb200;

template <typename T>
__global__ void embed_gather_kernel(T* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                    int H, int V, float mult, int* bad_ids) {
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0 && bad_ids) atomicAdd(bad_ids, 1);
        id = min(max(id, 0), V - 1);
    }
    const T* src = table + (size_t)id * H;
    T* dst = out + (size_t)t * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) dst[c] = from_f32<T>(to_f32(src[c]) * mult);
}

// Row gather without scaling: out[i, :] = src[rows[i], :] (used to pick the positions whose logits are wanted).
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ src, const int* __restrict__ rows, int H) {
    pdl_trigger();
    const T* s = src + (size_t)rows[blockIdx.x] * H;
    T* d = out + (size_t)blockIdx.x * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) d[c] = s[c];
}

extern "C" int lb_embed_gather(void* out, const void* table, const int* ids, int T_, int H, int V, float mult,
                               int* bad_ids, int dtype, void* stream) {
    if (T_ <= 0) return kOk;
    if (H <= 0 || V <= 0) return kBadSize;
    const int threads = H >= 1024 ? 256 : 128;
    LB_DISPATCH_DTYPE(dtype, embed_gather_kernel<T><<<T_, threads, 0, (cudaStream_t)stream>>>(
        (T*)out, (const T*)table, ids, H, V, mult, bad_ids));
    return launch_status();
}

extern "C" int lb_gather_rows(void* out, const void* src, const int* rows, int n, int H, int dtype, void* stream) {
    if (n <= 0) return kOk;
    const int threads = H >= 1024 ? 256 : 128;
    LB_DISPATCH_DTYPE(dtype, gather_rows_kernel<T><<<n, threads, 0, (cudaStream_t)stream>>>(
        (T*)out, (const T*)src, rows, H));
    return launch_status();
}
