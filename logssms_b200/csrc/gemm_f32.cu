// True 32-bit matrix product for the float32 path: C[M, N] = A[M, K] * W[N, K]^T (+ bias[N]) (* out_scale).
//
// Plain FFMA accumulation in float32; no tensor cores, so no reduced-precision matrix mode can
// sneak in whatever the library defaults are.  A may be a row-strided view.  64x64 tile per CTA,
// 256 threads, 4x4 outputs per thread, K in steps of 16 through shared memory.  Slow by design:
// it exists to show faults that bfloat16 hides.
#include "lb200/common.cuh"
using namespace lb200;

namespace {
constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, long lda, const float* __restrict__ W, const float* __restrict__ bias,
                float* __restrict__ C, long ldc, int M, int N, int K, float out_scale) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * BK; i += 256) {
            const int r = i / BK, c = i % BK;
            const int m = m0 + r, k = k0 + c;
            As[c][r] = (m < M && k < K) ? A[(size_t)m * lda + k] : 0.f;
        }
        for (int i = threadIdx.x; i < BN * BK; i += 256) {
            const int r = i / BK, c = i % BK;
            const int n = n0 + r, k = k0 + c;
            Ws[c][r] = (n < N && k < K) ? W[(size_t)n * K + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[k][ty * 4 + i]; w[i] = Ws[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            C[(size_t)m * ldc + n] = v * out_scale;
        }
    }
}
}  // namespace

extern "C" int lb_gemm_f32(const float* A, long lda, const float* W, const float* bias, float* C, long ldc, int M,
                           int N, int K, float out_scale, void* stream) {
    if (M <= 0 || N <= 0) return kOk;
    if (K <= 0) return kBadSize;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(A, lda, W, bias, C, ldc, M, N, K, out_scale);
    return launch_status();
}
