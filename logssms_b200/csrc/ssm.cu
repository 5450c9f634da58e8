// Selective state-space scan (Mamba2), token by token.  The state is held in 32-bit while a portion runs and is kept
// between steps in 32-bit (the default) or, for bfloat16 models, in bfloat16 as the reference keeps it
// (python/logssms/cache/naive/manager.py:445-451: the state pool has the engine's dtype): half the bytes of a decode step's
// state update, one rounding of the state per step.
//
//   dt_h   = softplus(round(dt_raw_h * dt_scale) + dt_bias_h)        softplus(v) = v if v > 20 else log1p(e^v)
//   dA_h   = -exp(A_log_h) * dt_h
//   S_h   <- e^{dA_h} S_h + B_{g(h)} (x) (x_h * dt_h)                 S_h in R^{P x N}
//   y_h    = S_h C_{g(h)} + D_h x_h                                   (uses the updated state)
//   y_h   <- round(y_h) * round(silu(round(z_h * gate_scale)))          (optional: the gate of a mixer without norm)
// (python/logssms/kernel/linear_attention/mamba2.py:27-36 and :261-292; recurrence oracle
// tests/kernel/test_mamba2.py:22-38 of the reference.)
//
// This kernel runs a portion of any length from the request's saved state and writes the state back
// in place; a request whose portion starts at position 0 starts from zeros whatever the slot holds.
// A single decoded token is a portion of length one.  `req_list` restricts the launch to some requests of
// the batch (B then counts the list).  Grid (head, request, P tile of 16); 128 threads
// = 16 values of p x 8 lanes over N; each lane owns N/8 state values in registers (float4 strided),
// the sum over N ends with three shuffles.
// A second form (`beside`) walks the same items with a grid that is resident at once; see ssm_scan_persistent_kernel.
#include "lb200/common.cuh"
using namespace lb200;

namespace {
constexpr int kPTile = 16;
constexpr int kLanesN = 8;

struct SsmArgs {
    const void* conv; int C; long conv_stride;   // [tokens, C] (row stride in elements): x | B | C after the conv
    const void* dt; long dt_stride;              // [tokens, nh] view
    const float* A_log; const float* dt_bias; const float* D;
    void* state;                                 // [slots, nh, P, N], float or (state_bf16) bfloat16
    void* y;                                     // [tokens, nh * P]
    const int* cu_seqlens; const int* start_pos; const int* slots;
    int nh, P, N, G; float dt_scale;
    const void* gate; long gate_stride; float gate_scale;   // optional [tokens, nh * P] view: y *= silu(gate * scale)
    const int* req_list;                         // optional: the requests (indices in the batch) to run
    int beside;                                  // the launch shares the GPU with other kernels of the step: leave them SM slots
    int state_bf16;
};

template <typename T> __device__ __forceinline__ void load4(const T* p, float* f);
template <> __device__ __forceinline__ void load4<float>(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// four consecutive state values, from or to the dtype the state is kept in
__device__ __forceinline__ void state_load4(const float* p, float* f) { load4<float>(p, f); }
__device__ __forceinline__ void state_load4(const __nv_bfloat16* p, float* f) { load4<__nv_bfloat16>(p, f); }
__device__ __forceinline__ void state_store4(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
__device__ __forceinline__ void state_store4(__nv_bfloat16* p, const float* f) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&a);
    v.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = v;
}

// The tokens of one portion through the state values S that the thread holds (thread (pi, nl): row p of head h, the
// state columns i * 32 + nl * 4 .. + 3): y for its row, S updated.
template <typename T, int NPT, bool ALIGNED>
__device__ __forceinline__ void scan_tokens(const SsmArgs& a, int h, int p, bool p_ok, int nl, int begin, int len, float (&S)[NPT]) {
    const int g = h / (a.nh / a.G);
    const int inner = a.nh * a.P;
    const int N = a.N;
    const float negA = -expf(a.A_log[h]);
    const float dt_bias = a.dt_bias[h], Dh = a.D[h];
    const T* conv = (const T*)a.conv;
    const T* dtp = (const T*)a.dt;
#pragma unroll 2
    for (int t = 0; t < len; ++t) {
        const size_t tok = (size_t)(begin + t);
        const T* row = conv + tok * a.conv_stride;
        float dt = round_to<T>(to_f32(dtp[tok * a.dt_stride + h]) * a.dt_scale) + dt_bias;
        dt = dt > 20.f ? dt : log1pf(expf(dt));
        const float decay = expf(negA * dt);
        const float xv = p_ok ? to_f32(row[h * a.P + p]) : 0.f;
        const float u = xv * dt;
        const T* Bp = row + inner + g * N;
        const T* Cp = Bp + a.G * N;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < NPT / 4; ++i) {
            const int n0 = i * 32 + nl * 4;
            if (n0 < N) {
                float Bv[4], Cv[4];
                if (ALIGNED) {
                    load4<T>(Bp + n0, Bv);
                    load4<T>(Cp + n0, Cv);
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) { Bv[e] = to_f32(Bp[n0 + e]); Cv[e] = to_f32(Cp[n0 + e]); }
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    S[4 * i + e] = S[4 * i + e] * decay + Bv[e] * u;
                    acc += S[4 * i + e] * Cv[e];
                }
            }
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        if (nl == 0 && p_ok) {
            float yv = acc + Dh * xv;
            if (a.gate != nullptr) {                      // the mixer's gate when it has no norm (fused.py:9-19)
                const float zg = round_to<T>(to_f32(((const T*)a.gate)[tok * a.gate_stride + h * a.P + p]) * a.gate_scale);
                yv = round_to<T>(yv) * round_to<T>(silu_f(zg));
            }
            ((T*)a.y)[tok * inner + h * a.P + p] = from_f32<T>(yv);
        }
    }
}

// NPT: state values per thread (N <= 8 * NPT).  ALIGNED: 4-element vector loads of B and C are legal.
template <typename T, typename ST, int NPT, bool ALIGNED>
__global__ void __launch_bounds__(kPTile * kLanesN) ssm_scan_kernel(SsmArgs a) {
    pdl_trigger();
    const int h = blockIdx.x, b = a.req_list ? a.req_list[blockIdx.y] : blockIdx.y;
    const int pi = threadIdx.x / kLanesN, nl = threadIdx.x % kLanesN;
    const int p = blockIdx.z * kPTile + pi;
    const bool p_ok = p < a.P;
    const int begin = a.cu_seqlens[b], len = a.cu_seqlens[b + 1] - begin;
    if (len <= 0) return;
    const int N = a.N;
    ST* sp = (ST*)a.state + (((size_t)a.slots[b] * a.nh + h) * a.P + (p_ok ? p : 0)) * N;

    float S[NPT];
    const bool fresh = a.start_pos[b] <= 0;
#pragma unroll
    for (int i = 0; i < NPT / 4; ++i) {
        const int n0 = i * 32 + nl * 4;
        if (!fresh && p_ok && n0 < N) {
            state_load4(sp + n0, &S[4 * i]);
        } else {
            S[4 * i] = S[4 * i + 1] = S[4 * i + 2] = S[4 * i + 3] = 0.f;
        }
    }
    // Up to here only step tables, constants and the saved state were read: with a programmatic launch that runs
    // under the kernel before (the projection and conv that make x, B, C and dt), whose results are read from here on.
    pdl_wait();
    scan_tokens<T, NPT, ALIGNED>(a, h, p, p_ok, nl, begin, len, S);
    if (p_ok) {
#pragma unroll
        for (int i = 0; i < NPT / 4; ++i) {
            const int n0 = i * 32 + nl * 4;
            if (n0 < N) state_store4(sp + n0, &S[4 * i]);
        }
    }
}

// The same work as a grid that is resident all at once: every CTA walks (request, head, tile of p) items, the state of
// its next item on its way while it works on this one.  For the listed requests of a step that also holds prompt
// portions: the one-CTA-per-item grid above is thousands of CTAs that take every SM slot that frees up before any
// kernel launched after it gets one, so nothing could run beside it; this form leaves the other kernels of the step
// (the chunked kernels of the prompt portion, on another stream) their share of the SMs, while it streams the states.
constexpr int kPersistCtasPerSm = 3, kSmCount = 148;

template <typename T, typename ST, int NPT, bool ALIGNED>
__global__ void __launch_bounds__(kPTile * kLanesN) ssm_scan_persistent_kernel(SsmArgs a, int B, int ptiles) {
    extern __shared__ int facts[];                       // per listed request: state slot, starts from zeros?, first token, tokens
    pdl_trigger();
    for (int i = threadIdx.x; i < B; i += blockDim.x) {
        const int b = a.req_list ? a.req_list[i] : i;
        const int begin = b >= 0 ? a.cu_seqlens[b] : 0;
        facts[4 * i] = b >= 0 ? a.slots[b] : 0;
        facts[4 * i + 1] = b >= 0 ? (a.start_pos[b] <= 0) : 1;
        facts[4 * i + 2] = begin;
        facts[4 * i + 3] = b >= 0 ? a.cu_seqlens[b + 1] - begin : 0;      // an entry that names no request: no tokens
    }
    __syncthreads();
    const int pi = threadIdx.x / kLanesN, nl = threadIdx.x % kLanesN;
    const int N = a.N, per_request = a.nh * ptiles, total = B * per_request;
    // item -> (request index in the list, head, tile of p): tiles of a head, heads of a request follow one another, as
    // the state lies in memory
    auto state_of = [&](int item, int& bi, int& h, int& p, bool& p_ok) -> ST* {
        bi = item / per_request;
        const int r = item - bi * per_request;
        h = r / ptiles;
        p = (r - h * ptiles) * kPTile + pi;
        p_ok = p < a.P;
        return (ST*)a.state + (((size_t)facts[4 * bi] * a.nh + h) * a.P + (p_ok ? p : 0)) * N;
    };
    auto fetch = [&](int item, float (&S)[NPT]) {
        int bi, h, p; bool p_ok;
        const ST* sp = state_of(item, bi, h, p, p_ok);
        const bool read = p_ok && !facts[4 * bi + 1] && facts[4 * bi + 3] > 0;
#pragma unroll
        for (int i = 0; i < NPT / 4; ++i) {
            const int n0 = i * 32 + nl * 4;
            S[4 * i] = S[4 * i + 1] = S[4 * i + 2] = S[4 * i + 3] = 0.f;
            if (read && n0 < N) state_load4(sp + n0, &S[4 * i]);
        }
    };
    float S[NPT], Sn[NPT];
    int item = blockIdx.x;
    if (item < total) fetch(item, S);
    pdl_wait();
    while (item < total) {
        const int next = item + gridDim.x;
        if (next < total) fetch(next, Sn);               // on its way while this item is worked on
        int bi, h, p; bool p_ok;
        ST* sp = state_of(item, bi, h, p, p_ok);
        const int len = facts[4 * bi + 3];
        if (len > 0) {
            scan_tokens<T, NPT, ALIGNED>(a, h, p, p_ok, nl, facts[4 * bi + 2], len, S);
            if (p_ok) {
#pragma unroll
                for (int i = 0; i < NPT / 4; ++i) {
                    const int n0 = i * 32 + nl * 4;
                    if (n0 < N) state_store4(sp + n0, &S[4 * i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < NPT; ++i) S[i] = Sn[i];
        item = next;
    }
}

template <typename T, typename ST, int NPT>
void launch_npt(const SsmArgs& a, int B, bool aligned, cudaStream_t s) {
    const int ptiles = (a.P + kPTile - 1) / kPTile;
    if (a.beside && (long)B * a.nh * ptiles > kPersistCtasPerSm * kSmCount && B <= 4096) {
        const int ctas = kPersistCtasPerSm * kSmCount;
        const size_t smem = (size_t)B * 4 * sizeof(int);
        if (aligned) ssm_scan_persistent_kernel<T, ST, NPT, true><<<ctas, kPTile * kLanesN, smem, s>>>(a, B, ptiles);
        else ssm_scan_persistent_kernel<T, ST, NPT, false><<<ctas, kPTile * kLanesN, smem, s>>>(a, B, ptiles);
        return;
    }
    dim3 grid(a.nh, B, ptiles);
    // few requests: the kernel starts under the one before it and has its state in registers when that one ends
    const bool early = B <= kPdlMaxRows;
    if (aligned) launch_pdl_if(early, ssm_scan_kernel<T, ST, NPT, true>, grid, dim3(kPTile * kLanesN), 0, s, a);
    else launch_pdl_if(early, ssm_scan_kernel<T, ST, NPT, false>, grid, dim3(kPTile * kLanesN), 0, s, a);
}

template <typename T, typename ST>
int launch_state(const SsmArgs& a, int B, cudaStream_t s) {
    const int inner = a.nh * a.P;
    const bool aligned = (inner % 4 == 0) && (a.C % 4 == 0) && (a.conv_stride % 4 == 0) && (((uintptr_t)a.conv & 15) == 0) && (a.N % 4 == 0) &&
                         (sizeof(T) == 4 || (inner % 4 == 0));
    if (a.N <= 32) launch_npt<T, ST, 4>(a, B, aligned, s);
    else if (a.N <= 64) launch_npt<T, ST, 8>(a, B, aligned, s);
    else if (a.N <= 128) launch_npt<T, ST, 16>(a, B, aligned, s);
    else if (a.N <= 256) launch_npt<T, ST, 32>(a, B, aligned, s);
    else return kTooLarge;
    return launch_status();
}

template <typename T>
int launch(const SsmArgs& a, int B, cudaStream_t s) { return launch_state<T, float>(a, B, s); }
template <>
int launch<__nv_bfloat16>(const SsmArgs& a, int B, cudaStream_t s) {
    return a.state_bf16 ? launch_state<__nv_bfloat16, __nv_bfloat16>(a, B, s) : launch_state<__nv_bfloat16, float>(a, B, s);
}
}  // namespace

// `state_bf16`: the state tensor is bfloat16 (bfloat16 models only), else float32.
extern "C" int lb_ssm_scan(const void* conv, int C, long conv_stride, const void* dt, long dt_stride, const float* A_log,
                           const float* dt_bias, const float* D, void* state, void* y, const int* cu_seqlens,
                           const int* start_pos, const int* slots, int B, int nh, int P, int N, int G,
                           float dt_scale, const void* gate, long gate_stride, float gate_scale,
                           const int* req_list, int beside, int state_bf16, int dtype, void* stream) {
    if (B <= 0) return kOk;
    if (nh <= 0 || P <= 0 || N <= 0 || G <= 0 || nh % G || N % 4) return kBadSize;
    if (C != nh * P + 2 * G * N) return kBadSize;
    if (state_bf16 && dtype != kBF16) return kBadSize;
    SsmArgs a{conv, C, conv_stride, dt, dt_stride, A_log, dt_bias, D, state, y, cu_seqlens, start_pos, slots, nh, P, N, G, dt_scale,
              gate, gate_stride, gate_scale, req_list, beside, state_bf16};
    LB_DISPATCH_DTYPE(dtype, return launch<T>(a, B, (cudaStream_t)stream));
    return kOk;
}
