// Row-wise normalisation and gating kernels: statistics in 32-bit, one CTA per row (or row group).
//
//  add_rmsnorm_branches : residual add + RMSNorm with one or two scaled outputs
//                         (formula of python/logssms/kernel/norm.py:16-35)
//  gated_rmsnorm        : grouped RMSNorm with SiLU gate, before or after the gate, or the plain
//                         y * silu(gate) product when the mixer has no norm
//                         (python/logssms/kernel/norm.py:55-86, python/logssms/kernel/fused.py:9-19)
//  swiglu               : silu(gate * s) * up on a packed [gate | up] row
//                         (python/logssms/kernel/fused.py:32-50)
#include "lb200/common.cuh"
using namespace lb200;

// r = round(round(x*in0) + round(other*in1)) when `other` is given; else r = round(x*in0) (in0 = 1: r = x)
// r += residual ; residual_out = round(r) ; n = round(r * rsqrt(mean(r^2)+eps) * w)
// out0 = round(n*s0) ; out1 = round(n*s1)
template <typename T>
__global__ void add_rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ other, const T* residual_in,
                                   T* residual_out, const float* __restrict__ weight, T* __restrict__ out0,
                                   T* __restrict__ out1, int H, float eps, float in0, float in1, float s0, float s1) {
    pdl_trigger();
    extern __shared__ float row[];          // H floats
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = to_f32(x[base + c]);
        if (other != nullptr) {
            v = round_to<T>(round_to<T>(v * in0) + round_to<T>(to_f32(other[base + c]) * in1));
        } else if (in0 != 1.f) {
            v = round_to<T>(v * in0);                 // the output multiplier of the product that made x, applied here
        }
        if (residual_in != nullptr) v += to_f32(residual_in[base + c]);
        row[c] = v;
        ss += v * v;
        if (residual_out != nullptr) residual_out[base + c] = from_f32<T>(v);
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float n = round_to<T>(row[c] * inv * weight[c]);
        out0[base + c] = from_f32<T>(n * s0);
        if (out1 != nullptr) out1[base + c] = from_f32<T>(n * s1);
    }
}

// The same for bfloat16 rows whose length is a multiple of 8 (up to 128 threads * 4 pieces * 8), in 16-byte
// pieces that stay in registers between the two passes: one load per tensor and thread where the kernel above
// makes eight, each waited for.
constexpr int kVecThreads = 128, kVecPieces = 4;
__global__ void __launch_bounds__(kVecThreads) add_rmsnorm_vec_kernel(
        const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ other, const __nv_bfloat16* residual_in,
        __nv_bfloat16* residual_out, const float* __restrict__ weight, __nv_bfloat16* __restrict__ out0,
        __nv_bfloat16* __restrict__ out1, int H, float eps, float in0, float in1, float s0, float s1) {
    typedef __nv_bfloat16 T;
    pdl_trigger();
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * H;
    const int pieces = H >> 3;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    uint4 xv[kVecPieces], ov[kVecPieces], rv[kVecPieces];
#pragma unroll
    for (int i = 0; i < kVecPieces; ++i) {
        const int pc = threadIdx.x + i * kVecThreads;
        xv[i] = ov[i] = rv[i] = zero;
        if (pc < pieces) {
            xv[i] = *reinterpret_cast<const uint4*>(x + base + pc * 8);
            if (other != nullptr) ov[i] = *reinterpret_cast<const uint4*>(other + base + pc * 8);
            if (residual_in != nullptr) rv[i] = *reinterpret_cast<const uint4*>(residual_in + base + pc * 8);
        }
    }
    float v[kVecPieces][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kVecPieces; ++i) {
        const int pc = threadIdx.x + i * kVecThreads;
        if (pc < pieces) {
            const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv[i]);
            const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&ov[i]);
            const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv[i]);
            uint4 packed;
            __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float2 f = __bfloat1622float2(x2[e]);
                if (other != nullptr) {
                    const float2 o = __bfloat1622float2(o2[e]);
                    f.x = round_to<T>(round_to<T>(f.x * in0) + round_to<T>(o.x * in1));
                    f.y = round_to<T>(round_to<T>(f.y * in0) + round_to<T>(o.y * in1));
                } else if (in0 != 1.f) {
                    f.x = round_to<T>(f.x * in0); f.y = round_to<T>(f.y * in0);
                }
                if (residual_in != nullptr) { const float2 r = __bfloat1622float2(r2[e]); f.x += r.x; f.y += r.y; }
                v[i][2 * e] = f.x; v[i][2 * e + 1] = f.y;
                ss += f.x * f.x + f.y * f.y;
                p2[e] = __floats2bfloat162_rn(f.x, f.y);
            }
            if (residual_out != nullptr) *reinterpret_cast<uint4*>(residual_out + base + pc * 8) = packed;
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int i = 0; i < kVecPieces; ++i) {
        const int pc = threadIdx.x + i * kVecThreads;
        if (pc < pieces) {
            const float4 w0 = __ldg(reinterpret_cast<const float4*>(weight + pc * 8));
            const float4 w1 = __ldg(reinterpret_cast<const float4*>(weight + pc * 8) + 1);
            const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            uint4 a, b;
            __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&a);
            __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float n0 = round_to<T>(v[i][2 * e] * inv * w[2 * e]), n1 = round_to<T>(v[i][2 * e + 1] * inv * w[2 * e + 1]);
                a2[e] = __floats2bfloat162_rn(n0 * s0, n1 * s0);
                b2[e] = __floats2bfloat162_rn(n0 * s1, n1 * s1);
            }
            *reinterpret_cast<uint4*>(out0 + base + pc * 8) = a;
            if (out1 != nullptr) *reinterpret_cast<uint4*>(out1 + base + pc * 8) = b;
        }
    }
}

extern "C" int lb_add_rmsnorm(const void* x, const void* other, const void* residual_in, void* residual_out,
                              const float* weight, void* out0, void* out1, int rows, int H, float eps,
                              float in0, float in1, float s0, float s1, int dtype, void* stream) {
    if (rows <= 0) return kOk;
    if (H <= 0) return kBadSize;
    auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if (dtype == kBF16 && H % 8 == 0 && H <= kVecThreads * kVecPieces * 8 && aligned(x) && aligned(other) &&
        aligned(residual_in) && aligned(residual_out) && aligned(weight) && aligned(out0) && aligned(out1)) {
        typedef __nv_bfloat16 B;
        add_rmsnorm_vec_kernel<<<rows, kVecThreads, 0, (cudaStream_t)stream>>>(
            (const B*)x, (const B*)other, (const B*)residual_in, (B*)residual_out, weight, (B*)out0, (B*)out1,
            H, eps, in0, in1, s0, s1);
        return launch_status();
    }
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return kTooLarge;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    LB_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_rmsnorm_kernel<T><<<rows, threads, smem, (cudaStream_t)stream>>>(
            (const T*)x, (const T*)other, (const T*)residual_in, (T*)residual_out, weight, (T*)out0, (T*)out1,
            H, eps, in0, in1, s0, s1);
    });
    return launch_status();
}

// RMSNorm of rows that are already the 32-bit residual sums (left by a product that joined the residual in its
// epilogue): n = round(v * rsqrt(mean(v^2)+eps) * w); out_k = round(n * s_k).  The rounding points of the kernel above.
template <typename T>
__global__ void summed_rmsnorm_kernel(const float* __restrict__ v, const float* __restrict__ weight,
                                      T* __restrict__ out0, T* __restrict__ out1, int H, float eps, float s0, float s1) {
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) { const float f = v[base + c]; ss += f * f; }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float n = round_to<T>(v[base + c] * inv * weight[c]);
        out0[base + c] = from_f32<T>(n * s0);
        if (out1 != nullptr) out1[base + c] = from_f32<T>(n * s1);
    }
}

extern "C" int lb_summed_rmsnorm(const float* v, const float* weight, void* out0, void* out1, int rows, int H,
                                 float eps, float s0, float s1, int dtype, void* stream) {
    if (rows <= 0) return kOk;
    if (H <= 0) return kBadSize;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    LB_DISPATCH_DTYPE(dtype, {
        summed_rmsnorm_kernel<T><<<rows, threads, 0, (cudaStream_t)stream>>>(v, weight, (T*)out0, (T*)out1, H, eps, s0, s1);
    });
    return launch_status();
}

// mode 0: out = y * round(silu(round(gate*s)))               (no norm)
// mode 1: norm before gate: out = y*rsqrt(mean_g(y^2)+eps)*w * silu(round(gate*s))
// mode 2: norm after gate : t = y*silu(round(gate*s)); out = t*rsqrt(mean_g(t^2)+eps)*w
// grid (rows, groups); y row stride = groups*width (contiguous), gate row stride given (a view).
template <typename T>
__global__ void gated_rmsnorm_kernel(const T* __restrict__ y, const T* __restrict__ gate, long gate_stride,
                                     const float* __restrict__ weight, T* __restrict__ out, int width, int groups,
                                     float eps, float gate_scale, int mode) {
    pdl_trigger();
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const int g = blockIdx.y;
    const T* yr = y + row * (size_t)groups * width + (size_t)g * width;
    const T* gr = gate + row * (size_t)gate_stride + (size_t)g * width;
    T* orow = out + row * (size_t)groups * width + (size_t)g * width;
    if (mode == 0) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            const float z = round_to<T>(silu_f(round_to<T>(to_f32(gr[c]) * gate_scale)));
            orow[c] = from_f32<T>(to_f32(yr[c]) * z);
        }
        return;
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = to_f32(yr[c]);
        if (mode == 2) v *= silu_f(round_to<T>(to_f32(gr[c]) * gate_scale));
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float z = silu_f(round_to<T>(to_f32(gr[c]) * gate_scale));
        float v = to_f32(yr[c]);
        if (mode == 2) v *= z;
        v = v * inv * weight[g * width + c];
        if (mode == 1) v *= z;
        orow[c] = from_f32<T>(v);
    }
}

extern "C" int lb_gated_rmsnorm(const void* y, const void* gate, long gate_stride, const float* weight, void* out,
                                int rows, int width, int groups, float eps, float gate_scale, int mode, int dtype,
                                void* stream) {
    if (rows <= 0) return kOk;
    if (width <= 0 || groups <= 0 || mode < 0 || mode > 2) return kBadSize;
    const int threads = width >= 1024 ? 256 : 128;
    dim3 grid(rows, groups);
    LB_DISPATCH_DTYPE(dtype, gated_rmsnorm_kernel<T><<<grid, threads, 0, (cudaStream_t)stream>>>(
        (const T*)y, (const T*)gate, gate_stride, weight, (T*)out, width, groups, eps, gate_scale, mode));
    return launch_status();
}

// out[r, c] = round(silu(round(gate*s))) * up, gate = in[r, c], up = in[r, I + c]; in row stride 2*I.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ in, T* __restrict__ out, int I, float act_scale) {
    const size_t r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= I) return;
    const float g = round_to<T>(to_f32(in[r * 2 * I + c]) * act_scale);
    const float a = round_to<T>(silu_f(g));
    out[r * I + c] = from_f32<T>(a * to_f32(in[r * 2 * I + I + c]));
}

// the same for bfloat16 rows whose width is a multiple of 8: eight columns per thread, 16-byte accesses
__global__ void swiglu_vec_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int I, float act_scale) {
    typedef __nv_bfloat16 T;
    const size_t r = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= I) return;
    const uint4 gv = *reinterpret_cast<const uint4*>(in + r * 2 * I + c);
    const uint4 uv = *reinterpret_cast<const uint4*>(in + r * 2 * I + I + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
        const float a0 = round_to<T>(silu_fast(round_to<T>(g.x * act_scale)));
        const float a1 = round_to<T>(silu_fast(round_to<T>(g.y * act_scale)));
        o2[e] = __floats2bfloat162_rn(a0 * u.x, a1 * u.y);
    }
    *reinterpret_cast<uint4*>(out + r * I + c) = ov;
}

extern "C" int lb_swiglu(const void* in, void* out, int rows, int I, float act_scale, int dtype, void* stream) {
    if (rows <= 0) return kOk;
    if (I <= 0) return kBadSize;
    if (dtype == kBF16 && I % 8 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
        dim3 grid((I / 8 + 127) / 128, rows);
        swiglu_vec_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, I, act_scale);
        return launch_status();
    }
    dim3 grid((I + 255) / 256, rows);
    LB_DISPATCH_DTYPE(dtype, swiglu_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>((const T*)in, (T*)out, I, act_scale));
    return launch_status();
}

// out = round(x * s): the output multiplier of a projection when it cannot ride in the product's epilogue.
template <typename T>
__global__ void scale_kernel(const T* __restrict__ x, T* __restrict__ out, size_t n, float s) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f32<T>(to_f32(x[i]) * s);
}

// out_f32 = float(x) * s: logits leave the model in 32-bit.
template <typename T>
__global__ void scale_to_f32_kernel(const T* __restrict__ x, float* __restrict__ out, size_t n, float s) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = to_f32(x[i]) * s;
}

__global__ void scale_vec_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, size_t n8, float s) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const uint4 v = reinterpret_cast<const uint4*>(x)[i];
    const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(v2[e]); o2[e] = __floats2bfloat162_rn(f.x * s, f.y * s); }
    reinterpret_cast<uint4*>(out)[i] = o;
}

extern "C" int lb_scale(const void* x, void* out, long n, float s, int to_f32_out, int dtype, void* stream) {
    if (n <= 0) return kOk;
    if (dtype == kBF16 && !to_f32_out && n % 8 == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
        const size_t n8 = (size_t)n / 8;
        scale_vec_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)x, (__nv_bfloat16*)out, n8, s);
        return launch_status();
    }
    const unsigned blocks = (unsigned)((n + 255) / 256);
    LB_DISPATCH_DTYPE(dtype, {
        if (to_f32_out) scale_to_f32_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>((const T*)x, (float*)out, (size_t)n, s);
        else scale_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>((const T*)x, (T*)out, (size_t)n, s);
    });
    return launch_status();
}
