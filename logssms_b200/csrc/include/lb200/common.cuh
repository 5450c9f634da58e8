// Shared device/host helpers of the logssms_b200 kernels (sm_100a).
//
// Every kernel file exports plain C launchers (`extern "C" int lb_*`) that take raw device
// pointers, sizes and a stream, and return 0 or an error code; the Python side checks shapes,
// dtypes and contiguity before the call and turns a non-zero code into an exception.  The same
// division of labour as the reference's host-side TensorMatcher + LaunchKernel helpers
// (csrc/include/logssms/tensor.hpp:475, csrc/include/logssms/utils.hpp:189-264), without tvm-ffi.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <utility>

namespace lb200 {

enum DType : int { kF32 = 0, kBF16 = 1 };

// error codes of the launchers (negative: refused before launch; positive: cudaError_t)
enum : int { kOk = 0, kBadDType = -1, kBadSize = -2, kTooLarge = -3 };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// value after a store in T and a load back: the "rounded to the activation dtype" of the formulas
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32(from_f32<T>(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a whole block; `scratch` is >= 32 floats of shared memory.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
// the same by the fast exponential and division (a few units in the last place of float32): for bfloat16 kernels that
// round the result to bfloat16 next and whose time the accurate form would set
__device__ __forceinline__ float silu_fast(float v) { return __fdividef(v, 1.f + __expf(-v)); }

// Programmatic dependent launch.  A kernel that is launched with `launch_pdl` may start while the kernel
// before it on the stream still runs; everything it does before `pdl_wait()` must not depend on that
// kernel (it may fetch weights), everything after sees all of its writes.  `pdl_trigger()` in the
// earlier kernel says "the next kernel may start now"; without it the next kernel starts at its end.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }

inline int launch_status() { return (int)cudaGetLastError(); }

// Raise a kernel's dynamic shared-memory limit, once per size: the attribute call costs the host tens of microseconds,
// which a step that is launched kernel by kernel pays at every launch otherwise.  `have` is a static of the calling
// launcher (one per kernel instantiation; the engine drives one device per process).
template <typename Kernel>
inline void ensure_dynamic_smem(Kernel kernel, size_t smem, size_t& have) {
    if (smem > 48 * 1024 && smem > have) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        have = smem;
    }
}

// `allow` false: plain stream order for this launch.
template <typename... KArgs, typename... Args>
inline int launch_pdl_if(bool allow, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                         Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = allow ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    return launch_pdl_if(true, kernel, grid, block, smem, stream, std::forward<Args>(args)...);
}
// Rows (tokens of a step) up to which a kernel starts under the one before it: with more rows the kernels are
// long enough to fill the GPU by themselves, and an early start only takes SM space from the one that runs
// (measured on a 36-layer decode step: 1-4 % faster at 1 and 8 rows, 4-10 % slower at 16, 32 and 64).
constexpr int kPdlMaxRows = 8;

}  // namespace lb200

#define LB_DISPATCH_DTYPE(dtype, ...)                                   \
    switch (dtype) {                                                    \
        case lb200::kF32: { using T = float; __VA_ARGS__; break; }      \
        case lb200::kBF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
        default: return lb200::kBadDType;                               \
    }
