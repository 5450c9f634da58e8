// Projections of a decode step: y[M, N] = x[M, K] W[N, K]^T for a handful of rows (M <= 64), bfloat16.
//
// With so few rows the product is bound by reading W once from HBM, so the kernel is built as a weight
// streamer: every CTA owns 16 output features (16 rows of W; 16 gate + 16 up rows for the SwiGLU form),
// its 8 warps split K between them, and every thread pulls its share of W straight from global memory
// into registers with 16-byte loads that bypass L1 (each byte of W is used once).  The rows of x are a
// few KB shared by all CTAs; they are read through L1/L2 as needed.  The arithmetic rides on the
// warp-level tensor-core instruction (mma.sync m16n8k16, bfloat16 in, float32 accumulate) with W as the
// 16-row operand and x as the 8-column operand ("swap A/B"), so 8 batch rows cost one instruction per
// 16 x 16 block of W.  tcgen05 has nothing to offer here: its smallest tile has 64 rows and needs W in
// shared memory first, while this kernel's limit is the HBM stream.
//
// K order inside an instruction is free as long as both operands agree: a thread loads 8 consecutive
// k (16 bytes) of its W row and of its x row and feeds them to two instructions, so all loads are
// 16-byte vectors.
//
// Epilogues (all on the float32 sums, rounding where the unfused chain rounds):
//   plain : out = round(round(acc + bias) * out_scale)                      bfloat16
//   f32   : out = float(round(acc + bias)) * out_scale                      float32 (logits)
//   swiglu: g = round(acc_gate), u = round(acc_up);
//           out = round(round(silu(round(g * act_scale))) * u)              bfloat16
// (python/logssms/layers/linear.py:26, python/logssms/kernel/fused.py:32-50 for the gate chain.)
#include "lb200/common.cuh"
using namespace lb200;

namespace {
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kFeat = 16;            // output features per CTA (per half for swiglu)
constexpr int kChunk = 32;           // k per load step: 4 lanes x 8 elements
constexpr int kUnroll = 4;           // chunks in flight per warp

struct SkinnyArgs {
    const __nv_bfloat16* x; long ldx;
    const __nv_bfloat16* w;                      // [N (or 2*N for swiglu: gate rows then up rows), K]
    const __nv_bfloat16* bias;                   // [N] or null
    void* out; long ldo;
    int M, N, K;
    float out_scale, act_scale;
    // optional prologue: x is not given but made here, as the RMSNorm of a residual sum
    //   v = [round(round(nx * in0) + round(nother * in1))  or  round(nx * in0)] + nres ; residual_out = round(v) (one CTA writes it)
    //   x = round(round(v * rsqrt(mean(v^2) + eps) * nweight) * nscale)
    const __nv_bfloat16* nx; const __nv_bfloat16* nother; const __nv_bfloat16* nres; __nv_bfloat16* nres_out;
    const float* nweight; float neps, nin0, nin1, nscale;
    // optional epilogue for output features [conv_c0, conv_c1): a depthwise causal conv step per row, each row
    // being the single new token of its own request (a decode step).  For channel c = n - conv_c0:
    //   u = round(y * region scale) ; c_out = round(sum_j w[c][j] * window_j + bias[c]) with window = state | u ;
    //   y <- round(silu(c_out)) ; state <- window without its oldest entry
    // (python/logssms/kernel/linear_attention/conv_decode.py:112-278; the thread that owns (row, feature) is the
    // only reader and writer of that row's state for the channel.)
    const float* conv_w; const float* conv_b; __nv_bfloat16* conv_state;     // [C, Kc] float32, [C] or null, [slots, C, Kc-1]
    const int* conv_slots; const int* conv_start;                             // per row: state slot, tokens before this one
    int conv_c0, conv_c1, conv_k, conv_e0, conv_e1; float conv_s0, conv_s1, conv_s2;
    // optional: the product joins the residual stream in its epilogue (plain epilogue, j_vsum given).  With y the
    // bfloat16 output the unfused chain would store,
    //   v = [round(round(y * j_in0) + round(j_other * j_in1))  or  y] + j_res          (float32)
    //   j_vsum = v ; j_res_out = round(v) ; j_partial[this CTA][row] = sum of v^2 over the CTA's 16 features
    // which is everything the next RMSNorm needs (python/logssms/kernel/norm.py:16-35): a consumer in mode
    // NORM == 2 takes s_vsum = j_vsum and the s_nparts partial sums per row, finds each row's factor with
    // s_nparts / 4 loads per thread, and norms its own columns where it loads them - no pass over whole rows and
    // no barrier before its main loop, with the rounding points of the norm kernel.
    const __nv_bfloat16* j_other; const __nv_bfloat16* j_res; float j_in0, j_in1;
    float* j_vsum; __nv_bfloat16* j_res_out; float* j_partial;
    const float* s_vsum; const float* s_partial; int s_nparts;
};

__device__ __forceinline__ uint4 load_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

enum Epilogue : int { kPlain = 0, kOutF32 = 1, kSwiglu = 2 };

// MT: tiles of 8 batch rows.  HALVES: 1, or 2 for swiglu (gate and up rows of the same feature).
// NORM 1: x is produced in shared memory by the fused residual-add + RMSNorm prologue (K <= 2048, M <= 16).
// NORM 2: x is the RMSNorm of rows already summed by the product before (see SkinnyArgs), made where it is loaded.
template <int MT, int EPI, int NORM>
__global__ void __launch_bounds__(kThreads) skinny_linear_kernel(SkinnyArgs a) {
    constexpr int HALVES = EPI == kSwiglu ? 2 : 1;
    constexpr int MP = MT * 8 + 1;
    extern __shared__ float red_raw[];
    float (*red)[HALVES][kFeat][MP] = reinterpret_cast<float (*)[HALVES][kFeat][MP]>(red_raw);
    // normalised rows, bfloat16, row stride K + 8 (behind the reduction buffer, 16-byte aligned)
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(red_raw + ((kWarps * HALVES * kFeat * MP + 3) / 4) * 4);
    const int ldxs = a.K + 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * kFeat;
    const int K = a.K;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    // rows of W this thread reads (clamped at the edge; masked at the store)
    const __nv_bfloat16* wrow[HALVES][2];
#pragma unroll
    for (int h = 0; h < HALVES; ++h)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int n = min(n0 + g + 8 * r, a.N - 1);
            wrow[h][r] = a.w + ((size_t)h * a.N + n) * K;
        }
    const __nv_bfloat16* xrow[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m)
        xrow[m] = NORM == 1 ? xs + (size_t)(m * 8 + g) * ldxs : (NORM == 2 ? nullptr : a.x + (size_t)min(m * 8 + g, a.M - 1) * a.ldx);

    float acc[HALVES][MT][4];
#pragma unroll
    for (int h = 0; h < HALVES; ++h)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[h][m][e] = 0.f;

    const int chunks = (K + kChunk - 1) / kChunk;
    const int per_warp = (chunks + kWarps - 1) / kWarps;
    const int c_begin = warp * per_warp, c_end = min(chunks, c_begin + per_warp);
    // two batches of weights in registers: one is multiplied while the other is on its way
    uint4 wa[kUnroll][HALVES][2], wb[kUnroll][HALVES][2];
    auto load_w = [&](uint4 (&wv)[kUnroll][HALVES][2], int c0) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int k = (c0 + u) * kChunk + t * 8;
            const bool ok = (c0 + u) < c_end && k < K;
#pragma unroll
            for (int h = 0; h < HALVES; ++h)
#pragma unroll
                for (int r = 0; r < 2; ++r) wv[u][h][r] = ok ? load_stream(wrow[h][r] + k) : zero;
        }
    };
    // The weights do not depend on the kernel before this one: their first two batches (all of them up to
    // K = 2048) are on their way while that kernel still runs; x (its output) is touched only after the wait.
    load_w(wa, c_begin);
    load_w(wb, c_begin + kUnroll);
    pdl_wait();
    if (NORM == 1) {
        // one warp per row; a lane keeps its 8-element pieces of the row in registers between the two passes
        constexpr int kMaxPieces = 8;                     // K <= 32 lanes * 8 pieces * 8 elements = 2048
        const int pieces = K / 8;
        for (int r = warp; r < MT * 8; r += kWarps) {
            __nv_bfloat16* dst = xs + (size_t)r * ldxs;
            if (r >= a.M) {
                for (int pc = lane; pc < pieces; pc += 32) *reinterpret_cast<uint4*>(dst + pc * 8) = zero;
                continue;
            }
            float v[kMaxPieces][8];
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < kMaxPieces; ++i) {
                const int pc = lane + 32 * i;
                if (pc < pieces) {
                    const size_t off = (size_t)r * K + pc * 8;
                    const uint4 xv = *reinterpret_cast<const uint4*>(a.nx + off);
                    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
                    uint4 ov = zero, rv = zero;
                    if (a.nother != nullptr) ov = *reinterpret_cast<const uint4*>(a.nother + off);
                    if (a.nres != nullptr) rv = *reinterpret_cast<const uint4*>(a.nres + off);
                    const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&ov);
                    const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
                    uint4 outv;
                    __nv_bfloat162* out2 = reinterpret_cast<__nv_bfloat162*>(&outv);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float2 f = __bfloat1622float2(x2[e]);
                        if (a.nother != nullptr) {
                            const float2 fo = __bfloat1622float2(o2[e]);
                            f.x = round_to<__nv_bfloat16>(round_to<__nv_bfloat16>(f.x * a.nin0) + round_to<__nv_bfloat16>(fo.x * a.nin1));
                            f.y = round_to<__nv_bfloat16>(round_to<__nv_bfloat16>(f.y * a.nin0) + round_to<__nv_bfloat16>(fo.y * a.nin1));
                        } else if (a.nin0 != 1.f) {
                            f.x = round_to<__nv_bfloat16>(f.x * a.nin0); f.y = round_to<__nv_bfloat16>(f.y * a.nin0);
                        }
                        if (a.nres != nullptr) { const float2 fr = __bfloat1622float2(r2[e]); f.x += fr.x; f.y += fr.y; }
                        v[i][2 * e] = f.x; v[i][2 * e + 1] = f.y;
                        ss += f.x * f.x + f.y * f.y;
                        out2[e] = __floats2bfloat162_rn(f.x, f.y);
                    }
                    if (a.nres_out != nullptr && blockIdx.x == 0) *reinterpret_cast<uint4*>(a.nres_out + off) = outv;
                }
            }
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / (float)K + a.neps);
#pragma unroll
            for (int i = 0; i < kMaxPieces; ++i) {
                const int pc = lane + 32 * i;
                if (pc < pieces) {
                    const float4 w0 = *reinterpret_cast<const float4*>(a.nweight + pc * 8);
                    const float4 w1 = *reinterpret_cast<const float4*>(a.nweight + pc * 8 + 4);
                    const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                    uint4 outv;
                    __nv_bfloat162* out2 = reinterpret_cast<__nv_bfloat162*>(&outv);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float n0 = round_to<__nv_bfloat16>(v[i][2 * e] * inv * w[2 * e]);
                        const float n1 = round_to<__nv_bfloat16>(v[i][2 * e + 1] * inv * w[2 * e + 1]);
                        out2[e] = __floats2bfloat162_rn(n0 * a.nscale, n1 * a.nscale);
                    }
                    *reinterpret_cast<uint4*>(dst + pc * 8) = outv;
                }
            }
        }
        __syncthreads();
    }
    // a joining product: the values of the residual and of the other branch that this thread's outputs meet in the
    // epilogue are fetched now, under the weight stream (thread i of the epilogue loop owns row i / 16, feature i % 16)
    constexpr int kJoinPer = (MT * 8 * kFeat + kThreads - 1) / kThreads;
    float j_res_v[kJoinPer], j_other_v[kJoinPer];
    if (EPI == kPlain && a.j_vsum != nullptr) {
#pragma unroll
        for (int q = 0; q < kJoinPer; ++q) {
            const int i = threadIdx.x + q * kThreads, m = i / kFeat, n = n0 + i % kFeat;
            const bool in = m < a.M && n < a.N;
            j_res_v[q] = (in && a.j_res != nullptr) ? __bfloat162float(a.j_res[(size_t)m * a.N + n]) : 0.f;
            j_other_v[q] = (in && a.j_other != nullptr) ? __bfloat162float(a.j_other[(size_t)m * a.N + n]) : 0.f;
        }
    }
    float inv_row[MT];
    if (NORM == 2) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const int row = min(m * 8 + g, a.M - 1);
            float ss = 0.f;
            for (int p = t; p < a.s_nparts; p += 4) ss += __ldg(a.s_partial + (size_t)p * a.M + row);
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            inv_row[m] = rsqrtf(ss / (float)K + a.neps);
        }
    }
    auto summed = [&](int m, int k) -> uint4 {
        const int row = m * 8 + g;
        if (row >= a.M) return zero;
        const float4* vp = reinterpret_cast<const float4*>(a.s_vsum + (size_t)row * K + k);
        const float4 v0 = __ldg(vp), v1 = __ldg(vp + 1);
        const float4 w0 = __ldg(reinterpret_cast<const float4*>(a.nweight + k));
        const float4 w1 = __ldg(reinterpret_cast<const float4*>(a.nweight + k) + 1);
        const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        const float gw[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        uint4 outv;
        __nv_bfloat162* out2 = reinterpret_cast<__nv_bfloat162*>(&outv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float n0 = round_to<__nv_bfloat16>(v[2 * e] * inv_row[m] * gw[2 * e]);
            const float n1 = round_to<__nv_bfloat16>(v[2 * e + 1] * inv_row[m] * gw[2 * e + 1]);
            out2[e] = __floats2bfloat162_rn(n0 * a.nscale, n1 * a.nscale);
        }
        return outv;
    };
    auto multiply = [&](const uint4 (&wv)[kUnroll][HALVES][2], int c0) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int k = (c0 + u) * kChunk + t * 8;
            const bool ok = (c0 + u) < c_end && k < K;
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const uint4 xv = !ok ? zero : (NORM == 2 ? summed(m, k) : (NORM == 1 ? *reinterpret_cast<const uint4*>(xrow[m] + k)
                                                                                       : __ldg(reinterpret_cast<const uint4*>(xrow[m] + k))));
#pragma unroll
                for (int h = 0; h < HALVES; ++h) {
                    mma_bf16(acc[h][m], wv[u][h][0].x, wv[u][h][1].x, wv[u][h][0].y, wv[u][h][1].y, xv.x, xv.y);
                    mma_bf16(acc[h][m], wv[u][h][0].z, wv[u][h][1].z, wv[u][h][0].w, wv[u][h][1].w, xv.z, xv.w);
                }
            }
        }
    };
    for (int c0 = c_begin; c0 < c_end; c0 += 2 * kUnroll) {
        multiply(wa, c0);
        if (c0 + 2 * kUnroll < c_end) load_w(wa, c0 + 2 * kUnroll);
        if (c0 + kUnroll < c_end) multiply(wb, c0 + kUnroll);
        if (c0 + 3 * kUnroll < c_end) load_w(wb, c0 + 3 * kUnroll);
    }
    // The next kernel may start once every CTA here has streamed its weights: it fetches its own under this
    // kernel's reduction and stores.  (A trigger at the start lets a whole chain of waiting kernels pile up
    // on the SMs; measured slower.)
    pdl_trigger();
    // accumulator element e of tile m: feature g + 8*(e/2), batch row m*8 + 2t + (e&1)
#pragma unroll
    for (int h = 0; h < HALVES; ++h)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int e = 0; e < 4; ++e) red[warp][h][g + 8 * (e >> 1)][m * 8 + 2 * t + (e & 1)] = acc[h][m][e];
    __syncthreads();
    const bool joins = EPI == kPlain && a.j_vsum != nullptr;      // then N is a multiple of 16 (the launcher checks)
    const int bound = joins ? (a.M * kFeat + 31) / 32 * 32 : a.M * kFeat;
#pragma unroll
    for (int q = 0; q < kJoinPer; ++q) {
        const int i = threadIdx.x + q * kThreads;
        if (i >= bound) break;
        const int m = i / kFeat, f = i % kFeat;
        const int n = n0 + f;
        float joined_sq = 0.f;
        if (m < a.M && n < a.N) {
        float s[HALVES];
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) v += red[w][h][f][m];
            s[h] = v;
        }
        if (EPI == kSwiglu) {
            const float gate = round_to<__nv_bfloat16>(round_to<__nv_bfloat16>(s[0]) * a.act_scale);
            const float act = round_to<__nv_bfloat16>(silu_f(gate));
            const float up = round_to<__nv_bfloat16>(s[HALVES - 1]);
            ((__nv_bfloat16*)a.out)[(size_t)m * a.ldo + n] = __float2bfloat16_rn(act * up);
        } else {
            float v = s[0];
            if (a.bias != nullptr) v += __bfloat162float(a.bias[n]);
            v = round_to<__nv_bfloat16>(v);
            if (EPI == kPlain && a.conv_w != nullptr && n >= a.conv_c0 && n < a.conv_c1) {
                const int c = n - a.conv_c0, C = a.conv_c1 - a.conv_c0, taps = a.conv_k;
                const float scale = c < a.conv_e0 ? a.conv_s0 : (c < a.conv_e1 ? a.conv_s1 : a.conv_s2);
                const float u = round_to<__nv_bfloat16>(v * scale);
                __nv_bfloat16* st = a.conv_state + ((size_t)a.conv_slots[m] * C + c) * (taps - 1);
                const bool history = a.conv_start[m] > 0;
                const float* w = a.conv_w + (size_t)c * taps;
                float acc2 = w[taps - 1] * u;
                for (int j = 0; j < taps - 1; ++j) {
                    const float win = history ? __bfloat162float(st[j]) : 0.f;
                    acc2 += w[j] * win;
                    if (j > 0) st[j - 1] = __float2bfloat16_rn(win);          // shift: entry j moves to j - 1
                }
                st[taps - 2] = __float2bfloat16_rn(u);
                if (a.conv_b != nullptr) acc2 += a.conv_b[c];
                acc2 = round_to<__nv_bfloat16>(acc2);
                v = round_to<__nv_bfloat16>(silu_f(acc2));
            }
            if (EPI == kOutF32) ((float*)a.out)[(size_t)m * a.ldo + n] = v * a.out_scale;
            else if (!joins) ((__nv_bfloat16*)a.out)[(size_t)m * a.ldo + n] =
                a.out_scale == 1.f ? __float2bfloat16_rn(v) : __float2bfloat16_rn(v * a.out_scale);
            else {
                float y = a.out_scale == 1.f ? v : round_to<__nv_bfloat16>(v * a.out_scale);
                const size_t at = (size_t)m * a.N + n;
                if (a.j_other != nullptr)
                    y = round_to<__nv_bfloat16>(round_to<__nv_bfloat16>(y * a.j_in0) + round_to<__nv_bfloat16>(j_other_v[q] * a.j_in1));
                if (a.j_res != nullptr) y += j_res_v[q];
                a.j_vsum[at] = y;
                a.j_res_out[at] = __float2bfloat16_rn(y);
                joined_sq = y * y;
            }
        }
        }
        if (joins) {                                              // 16 consecutive lanes hold one row's 16 features
            joined_sq += __shfl_xor_sync(0xffffffffu, joined_sq, 8);
            joined_sq += __shfl_xor_sync(0xffffffffu, joined_sq, 4);
            joined_sq += __shfl_xor_sync(0xffffffffu, joined_sq, 2);
            joined_sq += __shfl_xor_sync(0xffffffffu, joined_sq, 1);
            if (f == 0 && m < a.M) a.j_partial[(size_t)blockIdx.x * a.M + m] = joined_sq;
        }
    }
}

template <int EPI, int NORM>
int launch_mt(const SkinnyArgs& a, cudaStream_t s) {
    const dim3 grid((a.N + kFeat - 1) / kFeat);
    const int mt = (a.M + 7) / 8;
    constexpr int halves = EPI == kSwiglu ? 2 : 1;
#define LB_SKINNY(MT)                                                                                       \
    {                                                                                                       \
        size_t smem = sizeof(float) * ((kWarps * halves * kFeat * (MT * 8 + 1) + 3) / 4 * 4);               \
        if (NORM == 1) smem += (size_t)MT * 8 * (a.K + 8) * sizeof(__nv_bfloat16);                          \
        if (smem > 48 * 1024)                                                                               \
            cudaFuncSetAttribute(skinny_linear_kernel<MT, EPI, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        rc = launch_pdl_if(a.M <= kPdlMaxRows, skinny_linear_kernel<MT, EPI, NORM>, grid, dim3(kThreads), smem, s, a); \
    }
    int rc = 0;
    if (mt <= 1) LB_SKINNY(1)
    else if (mt <= 2) LB_SKINNY(2)
    else if constexpr (NORM != 0) return kTooLarge;
    else if (mt <= 4) LB_SKINNY(4)
    else LB_SKINNY(8)
#undef LB_SKINNY
    return rc != 0 ? rc : launch_status();
}

template <int NORM>
int launch_epi(const SkinnyArgs& a, int epilogue, cudaStream_t s) {
    switch (epilogue) {
        case kPlain: return launch_mt<kPlain, NORM>(a, s);
        case kOutF32: return launch_mt<kOutF32, NORM>(a, s);
        case kSwiglu: return launch_mt<kSwiglu, NORM>(a, s);
        default: return kBadSize;
    }
}
}  // namespace

// x: [M, K] bfloat16 rows (row stride ldx, a multiple of 8 elements, 16-byte aligned base);
// w: [N, K] bfloat16 contiguous ([2N, K] for the swiglu epilogue: gate rows, then up rows); K a
// multiple of 8; M <= 64.  epilogue: 0 plain (bfloat16 out), 1 float32 out, 2 swiglu (bfloat16 out).
extern "C" int lb_linear_skinny(const void* x, long ldx, const void* w, const void* bias, void* out, long ldo, int M,
                                int N, int K, float out_scale, float act_scale, int epilogue, void* stream) {
    if (M <= 0 || N <= 0) return kOk;
    if (K <= 0 || K % 8 || ldx % 8) return kBadSize;
    if (M > 64) return kTooLarge;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return kBadSize;
    SkinnyArgs a{(const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, out, ldo,
                 M, N, K, out_scale, act_scale, nullptr, nullptr, nullptr, nullptr, nullptr, 0.f, 1.f, 1.f, 1.f,
                 nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0, 0, 1.f, 1.f, 1.f};
    return launch_epi<0>(a, epilogue, (cudaStream_t)stream);
}

// The same product with x made on the fly: x = round(rmsnorm(v; norm_weight, eps) * norm_scale) with
// v = [round(round(nx * in0) + round(nother * in1)) or round(nx * in0)] + nres.  nx / nother / nres / res_out: contiguous
// [M, K] bfloat16 (nother, nres, res_out may be null); res_out (the new residual, round(v)) must not alias
// nres: other CTAs still read it.  M <= 16, K a multiple of 8 up to 2048, norm_weight float32 [K].
extern "C" int lb_linear_skinny_normed(const void* nx, const void* nother, const void* nres, void* res_out,
                                       const float* norm_weight, float eps, float in0, float in1, float norm_scale,
                                       const void* w, const void* bias, void* out, long ldo, int M, int N, int K,
                                       float out_scale, float act_scale, int epilogue, void* stream) {
    if (M <= 0 || N <= 0) return kOk;
    if (K <= 0 || K % 8) return kBadSize;
    if (M > 16 || K > 2048) return kTooLarge;
    if (((uintptr_t)nx | (uintptr_t)w | (uintptr_t)nother | (uintptr_t)nres | (uintptr_t)res_out | (uintptr_t)norm_weight) & 15) return kBadSize;
    if (res_out != nullptr && res_out == nres) return kBadSize;
    SkinnyArgs a{nullptr, 0, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, out, ldo, M, N, K, out_scale, act_scale,
                 (const __nv_bfloat16*)nx, (const __nv_bfloat16*)nother, (const __nv_bfloat16*)nres, (__nv_bfloat16*)res_out,
                 norm_weight, eps, in0, in1, norm_scale,
                 nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0, 0, 1.f, 1.f, 1.f};
    return launch_epi<1>(a, epilogue, (cudaStream_t)stream);
}

// The plain product (x given, or made by the norm prologue when `nx` is not null) with the conv step of a
// decode batch on the output features [c0, c1): see SkinnyArgs.  conv_w: float32 [c1 - c0, taps]; conv_b: float32
// [c1 - c0] or null; conv_state: bfloat16 [slots, c1 - c0, taps - 1], updated in place; slots / start: int32 per row;
// e0, e1: channel indices (relative to c0) where the second and third input scale begin.
extern "C" int lb_linear_skinny_conv(const void* x, long ldx, const void* nx, const void* nother, const void* nres,
                                     void* res_out, const float* norm_weight, float eps, float in0, float in1,
                                     float norm_scale, const void* w, const void* bias, void* out, long ldo, int M, int N,
                                     int K, const float* conv_w, const float* conv_b, void* conv_state,
                                     const int* slots, const int* start, int c0, int c1, int taps, int e0, int e1,
                                     float s0, float s1, float s2, void* stream) {
    if (M <= 0 || N <= 0) return kOk;
    if (K <= 0 || K % 8 || taps < 2 || taps > 8 || c0 < 0 || c1 > N || c0 > c1) return kBadSize;
    const bool normed = nx != nullptr;
    if (normed ? (M > 16 || K > 2048) : (M > 64)) return kTooLarge;
    if (!normed && (ldx % 8 || ((uintptr_t)x & 15))) return kBadSize;
    if (((uintptr_t)nx | (uintptr_t)w | (uintptr_t)nother | (uintptr_t)nres | (uintptr_t)res_out | (uintptr_t)norm_weight) & 15) return kBadSize;
    if (res_out != nullptr && res_out == nres) return kBadSize;
    SkinnyArgs a{(const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, out, ldo, M, N, K, 1.f, 1.f,
                 (const __nv_bfloat16*)nx, (const __nv_bfloat16*)nother, (const __nv_bfloat16*)nres, (__nv_bfloat16*)res_out,
                 norm_weight, eps, in0, in1, norm_scale,
                 conv_w, conv_b, (__nv_bfloat16*)conv_state, slots, start, c0, c1, taps, e0, e1, s0, s1, s2};
    return normed ? launch_epi<1>(a, kPlain, (cudaStream_t)stream) : launch_epi<0>(a, kPlain, (cudaStream_t)stream);
}

// The plain product whose epilogue joins the residual stream (see SkinnyArgs): instead of its bfloat16 output y it
// leaves v = [round(round(y * in0) + round(other * in1)) or y] + res as float32 in vsum [M, N], round(v) in res_out
// [M, N] and per CTA and row the sum of v^2 over its 16 features in partial [N / 16, M].  other, res: contiguous
// [M, N] bfloat16 or null; N a multiple of 16; M <= 64.
extern "C" int lb_linear_skinny_join(const void* x, long ldx, const void* w, const void* bias, int M, int N, int K,
                                     float out_scale, const void* other, const void* res, float in0, float in1,
                                     float* vsum, void* res_out, float* partial, void* stream) {
    if (M <= 0 || N <= 0) return kOk;
    if (K <= 0 || K % 8 || ldx % 8 || N % kFeat || vsum == nullptr || res_out == nullptr || partial == nullptr) return kBadSize;
    if (M > 64) return kTooLarge;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return kBadSize;
    SkinnyArgs a{};
    a.x = (const __nv_bfloat16*)x; a.ldx = ldx; a.w = (const __nv_bfloat16*)w; a.bias = (const __nv_bfloat16*)bias;
    a.out = nullptr; a.ldo = N; a.M = M; a.N = N; a.K = K; a.out_scale = out_scale; a.act_scale = 1.f;
    a.j_other = (const __nv_bfloat16*)other; a.j_res = (const __nv_bfloat16*)res; a.j_in0 = in0; a.j_in1 = in1;
    a.j_vsum = vsum; a.j_res_out = (__nv_bfloat16*)res_out; a.j_partial = partial;
    return launch_epi<0>(a, kPlain, (cudaStream_t)stream);
}

// A product (any epilogue; with conv_w given, the conv step on the features [c0, c1) as in lb_linear_skinny_conv)
// whose x is the RMSNorm of rows that lb_linear_skinny_join left: x = round(round(v * rsqrt(mean(v^2) + eps) *
// norm_weight) * norm_scale), v = vsum [M, K] float32, mean(v^2) from the nparts partial sums per row.  M <= 16.
extern "C" int lb_linear_skinny_summed(const float* vsum, const float* partial, int nparts, const float* norm_weight,
                                       float eps, float norm_scale, const void* w, const void* bias, void* out, long ldo,
                                       int M, int N, int K, float out_scale, float act_scale, int epilogue,
                                       const float* conv_w, const float* conv_b, void* conv_state, const int* slots,
                                       const int* start, int c0, int c1, int taps, int e0, int e1, float s0, float s1,
                                       float s2, void* stream) {
    if (M <= 0 || N <= 0) return kOk;
    if (K <= 0 || K % 8 || nparts <= 0 || vsum == nullptr || partial == nullptr || norm_weight == nullptr) return kBadSize;
    if (M > 16) return kTooLarge;
    if (((uintptr_t)vsum | (uintptr_t)w | (uintptr_t)norm_weight) & 15) return kBadSize;
    if (conv_w != nullptr && (epilogue != kPlain || taps < 2 || taps > 8 || c0 < 0 || c1 > N || c0 > c1)) return kBadSize;
    SkinnyArgs a{};
    a.w = (const __nv_bfloat16*)w; a.bias = (const __nv_bfloat16*)bias; a.out = out; a.ldo = ldo;
    a.M = M; a.N = N; a.K = K; a.out_scale = out_scale; a.act_scale = act_scale;
    a.nweight = norm_weight; a.neps = eps; a.nin0 = 1.f; a.nin1 = 1.f; a.nscale = norm_scale;
    a.s_vsum = vsum; a.s_partial = partial; a.s_nparts = nparts;
    if (conv_w != nullptr) {
        a.conv_w = conv_w; a.conv_b = conv_b; a.conv_state = (__nv_bfloat16*)conv_state; a.conv_slots = slots; a.conv_start = start;
        a.conv_c0 = c0; a.conv_c1 = c1; a.conv_k = taps; a.conv_e0 = e0; a.conv_e1 = e1;
        a.conv_s0 = s0; a.conv_s1 = s1; a.conv_s2 = s2;
    }
    return launch_epi<2>(a, epilogue, (cudaStream_t)stream);
}
