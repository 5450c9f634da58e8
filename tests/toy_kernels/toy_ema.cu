// A kernel that lives outside the package: the scan of the test suite's toy mixer,
//     s_t = a * s_{t-1} + x_t     (a = sigmoid(decay_logit), per channel; s is the request's state)
// one thread per (request, channel), walking the request's tokens of this step.  A part names this file in its
// `kernels` attribute and the package's build module compiles and loads it like its own sources.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

template <typename T> __device__ float load(const T* p);
template <> __device__ float load<float>(const float* p) { return *p; }
template <> __device__ float load<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__global__ void toy_ema_kernel(const T* x, float* y, float* state, const float* decay_logit, const int* cu_seqlens,
                               const int* start_pos, const int* slots, int H) {
    const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= H) return;
    const int begin = cu_seqlens[b], end = cu_seqlens[b + 1];
    const float a = 1.f / (1.f + expf(-decay_logit[c]));
    float* sp = state + (size_t)slots[b] * H + c;
    float s = start_pos[b] > 0 ? *sp : 0.f;          // a request at position 0 starts from zero whatever the slot holds
    for (int t = begin; t < end; ++t) {
        s = a * s + load<T>(x + (size_t)t * H + c);
        y[(size_t)t * H + c] = s;
    }
    if (end > begin) *sp = s;
}

extern "C" int toy_ema_scan(const void* x, float* y, float* state, const float* decay_logit, const int* cu_seqlens,
                            const int* start_pos, const int* slots, int requests, int H, int is_bf16, void* stream) {
    if (requests <= 0 || H <= 0) return 0;
    const dim3 grid(requests, (H + 127) / 128);
    if (is_bf16) toy_ema_kernel<__nv_bfloat16><<<grid, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, y, state, decay_logit, cu_seqlens, start_pos, slots, H);
    else toy_ema_kernel<float><<<grid, 128, 0, (cudaStream_t)stream>>>((const float*)x, y, state, decay_logit, cu_seqlens, start_pos, slots, H);
    return (int)cudaGetLastError();
}
