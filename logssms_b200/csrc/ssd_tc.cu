// The chunk-scan step of the chunked selective scan (ssd.cu, kernel 3) on the 5th-generation tensor cores:
// head size a multiple of 64 (a CTA takes 64 dims of a head), state size a multiple of 64 up to 256, chunks of 128
// tokens, bfloat16.  Other sizes stay on the mma.sync kernel.
//
//   y_t = e^{a_t} C_t . S_in + sum_{s<=t} [(C_t . B_s) e^{a_t - a_s} dt_s] x_s + D x_t       (t, s: tokens of one chunk)
//
// (python/logssms/kernel/linear_attention/mamba2.py:148-194, vendor/fla/chunk_o.py:79-136 of the reference.)
// One CTA per (chunk, 64 dims of a head), 10 warps, two CTAs per SM:
//   warp 0    one thread: TMA loads (128-byte swizzle) of the chunk's rows of C and B (128 tokens x N, 64 columns
//             per box), of x (128 x 64) and of the state the chunk starts from (64 x N, bfloat16)
//   warp 1    allocates 256 columns of tensor memory; one thread issues
//                 G  = C B^T      M 128 tokens t, N 128 tokens s, K = state size     -> columns   0..127
//                 Y2 = C S_in^T   M 128, N 64 head dims, K = state size              -> columns 128..191
//                 Y1 = W x        M 128, N 64, K 128 tokens s (x as an MN-major operand) -> columns 192..255
//   warps 2-9 two threads per token t (a warp reads its own quarter of tensor memory's lanes, so warps w and w + 4
//             share 32 tokens and split the columns): dt (softplus) and the running sum of dA over the chunk
//             (float32, a prefix sum over the chunk) while the loads are under way; then their halves of the row of
//             G from tensor memory, times the decay and dt_s, zero above the diagonal, rounded to bfloat16 into
//             shared memory as W (over the tile of B, which G has consumed by then); at the end
//             y_t = e^{a_t} Y2 + Y1 + D x_t, the gate, the store.
// Rows of a last, shorter chunk: the loads bring whatever follows in the step (other requests' rows, zeros beyond
// the end), all finite; dt_s = 0 for them, so they add nothing, and their own rows are not stored.
//
// Every wait on an mbarrier is bounded; a wait that gives up records itself in `error`, every role then runs out of
// its own bounded waits, tensor memory is freed and the kernel returns.
#include "lb200/common.cuh"
#include "lb200/tcgen05.cuh"
using namespace lb200;
using namespace lb200::tc;

namespace {
typedef __nv_bfloat16 bf16;
constexpr int kL = 128, kP = 64;
constexpr int kRowThreads = 256;                          // two threads per token of the chunk
constexpr int kThreads = 64 + kRowThreads;
constexpr uint32_t kRowTile = kL * 128;                    // a 128-row tile of 64 bfloat16 columns
constexpr uint32_t kSinTile = kP * 128;
constexpr uint32_t kTmemCols = 256;
constexpr float kLog2e = 1.4426950408889634f;

struct ScanArgs {
    const bf16* dt; long dt_stride;
    const float* A_log; const float* dt_bias; const float* D;
    bf16* y;
    const int* cu_seqlens; const int* chunks;
    int nh, P, N, G;                                      // P: the head size, a multiple of 64 (a CTA takes 64 dims of it)
    float dt_scale;
    const bf16* gate; long gate_stride; float gate_scale;
    int gate16;                                           // the gate's rows start on 16-byte boundaries
    int* error;
};

__device__ __forceinline__ void report(int* error, int role) {
    if (error != nullptr) atomicCAS(error, 0, 0x20000000 | (role << 24) | ((blockIdx.y & 0xFFF) << 12) | (blockIdx.x & 0xFFF));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int NB>                                          // state size / 64
__global__ void __launch_bounds__(kThreads, 2)
ssd_chunk_scan_tc_kernel(const __grid_constant__ CUtensorMap map_conv, const __grid_constant__ CUtensorMap map_sin, ScanArgs a) {
    constexpr int kBTiles = NB > 2 ? NB : 2;              // W (128 x 128) lies over the tile of B
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* c_s = base;                                  // NB x [128][128 B]
    uint8_t* b_s = c_s + NB * kRowTile;                   // NB x [128][128 B]; later W: 2 x [128][128 B]
    uint8_t* x_s = b_s + kBTiles * kRowTile;              // [128][128 B]
    uint8_t* sin_s = x_s + kRowTile;                      // NB x [64][128 B]
    float2* ad_s = reinterpret_cast<float2*>(sin_s + NB * kSinTile);  // [128]  (running sum of dA times log2(e), dt) of a token
    float* tot = reinterpret_cast<float*>(ad_s + kL);     // [4]
    uint64_t* full_cb = reinterpret_cast<uint64_t*>(tot + 4);
    uint64_t* full_sx = full_cb + 1;
    uint64_t* g_ready = full_sx + 1;                      // G is in tensor memory (and B has been read)
    uint64_t* w_ready = g_ready + 1;                      // W is in shared memory (128 arrivals)
    uint64_t* y_ready = w_ready + 1;                      // Y1 and Y2 are in tensor memory
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(y_ready + 1);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // a head of more than 64 dims is run as pieces of 64 with a CTA each: they share the head's B, C, dt and decay
    // (and each computes G = C B^T again), and own their columns of x, of the start state and of y
    const int chunk = blockIdx.x, pieces = a.P / kP, h = blockIdx.y / pieces, col0 = h * a.P + (blockIdx.y % pieces) * kP;
    const int b = a.chunks[2 * chunk], t0 = a.chunks[2 * chunk + 1];
    if (b < 0) return;                                  // a list entry without work: the lists of a step that was filled up to fixed sizes end in such entries
    const int begin = a.cu_seqlens[b], len = a.cu_seqlens[b + 1] - begin;
    const int Lc = min(kL, len - t0);
    const int tok0 = begin + t0;
    const int g = h / (a.nh / a.G), inner = a.nh * a.P;

    if (threadIdx.x == 0) {
        mbar_init(full_cb, 1); mbar_init(full_sx, 1); mbar_init(g_ready, 1); mbar_init(y_ready, 1);
        mbar_init(w_ready, kRowThreads);
        *failed = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc<kTmemCols>(tmem_slot);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(full_cb, 2 * NB * kRowTile);
#pragma unroll
            for (int kb = 0; kb < NB; ++kb) {
                tma_load_2d(c_s + kb * kRowTile, &map_conv, full_cb, inner + (a.G + g) * a.N + kb * 64, tok0);
                tma_load_2d(b_s + kb * kRowTile, &map_conv, full_cb, inner + g * a.N + kb * 64, tok0);
            }
            mbar_expect_tx(full_sx, kRowTile + NB * kSinTile);
            tma_load_2d(x_s, &map_conv, full_sx, col0, tok0);
#pragma unroll
            for (int kb = 0; kb < NB; ++kb)
                tma_load_2d(sin_s + kb * kSinTile, &map_sin, full_sx, kb * 64, chunk * inner + col0);
            // the CTA does not leave before its copies have landed, whatever the other roles do
            if (!mbar_wait(full_cb, 0)) { report(a.error, 1); *failed = 1; }
            if (!mbar_wait(full_sx, 0)) { report(a.error, 1); *failed = 1; }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = mbar_wait(full_cb, 0);
            if (!ok) { report(a.error, 2); *failed = 1; }
            if (ok) {
                fence_after_sync();
                const uint32_t idesc_g = umma_idesc(kL, kL);
#pragma unroll
                for (int kb = 0; kb < NB; ++kb) {
                    const uint64_t cdesc = umma_desc(c_s + kb * kRowTile), bdesc = umma_desc(b_s + kb * kRowTile);
#pragma unroll
                    for (int k = 0; k < 4; ++k) umma_bf16(tmem, cdesc + 2 * k, bdesc + 2 * k, idesc_g, (kb | k) != 0);
                }
                umma_commit(g_ready);
                ok = mbar_wait(full_sx, 0);
                if (!ok) { report(a.error, 3); *failed = 1; }
            }
            const uint32_t idesc_y = umma_idesc(kL, kP);
            if (ok) {
                fence_after_sync();
#pragma unroll
                for (int kb = 0; kb < NB; ++kb) {
                    const uint64_t cdesc = umma_desc(c_s + kb * kRowTile), sdesc = umma_desc(sin_s + kb * kSinTile);
#pragma unroll
                    for (int k = 0; k < 4; ++k) umma_bf16(tmem + 128, cdesc + 2 * k, sdesc + 2 * k, idesc_y, (kb | k) != 0);
                }
                ok = mbar_wait(w_ready, 0);
                if (!ok) { report(a.error, 4); *failed = 1; }
            }
            if (ok && !*failed) {
                fence_after_sync();
                const uint64_t xdesc = umma_desc(x_s);
#pragma unroll
                for (int k = 0; k < kL / 16; ++k) {        // 16 tokens s: 32 bytes along a row of W, two 8-row groups of x
                    const uint64_t wdesc = umma_desc(b_s + (k / 4) * kRowTile) + 2 * (k % 4);
                    umma_bf16(tmem + 192, wdesc, xdesc + (uint64_t)(2048 >> 4) * k, idesc_y | kBMnMajor, k != 0);
                }
                umma_commit(y_ready);
            }
        }
    } else {
        const int wq = warp & 3;                           // the quarter of tensor memory's lanes this warp may read
        const int hf = (warp - 2) >> 2;                    // which of the row's two threads
        const int r = wq * 32 + lane;                      // the token of the chunk this thread works on
        const uint32_t lane_addr = tmem + ((uint32_t)(wq * 32) << 16);
        // dt, dA and the running sum over the chunk (both threads of a row compute it; one writes it)
        float dtv = 0.f, dA = 0.f;
        if (r < Lc) {
            dtv = round_to<bf16>(__bfloat162float(a.dt[(size_t)(tok0 + r) * a.dt_stride + h]) * a.dt_scale) + a.dt_bias[h];
            dtv = dtv > 20.f ? dtv : log1pf(expf(dtv));
            dA = -expf(a.A_log[h]) * dtv;
        }
        float run = dA;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, run, o);
            if (lane >= o) run += up;
        }
        if (lane == 31 && hf == 0) tot[wq] = run;
        asm volatile("bar.sync 1, %0;" ::"n"(kRowThreads) : "memory");
        float before = 0.f;
        for (int w = 0; w < wq; ++w) before += tot[w];
        const float at = (run + before) * kLog2e;
        if (hf == 0) ad_s[r] = make_float2(at, dtv);
        asm volatile("bar.sync 1, %0;" ::"n"(kRowThreads) : "memory");
        // this thread's half of the gate's row is asked for now and used at the end
        uint4 zrow[4];
        const bool gated = a.gate != nullptr && r < Lc;
        if (gated) {
            const bf16* zr = a.gate + (size_t)(tok0 + r) * a.gate_stride + col0 + hf * 32;
            if (a.gate16) {
                const uint4* zp = reinterpret_cast<const uint4*>(zr);
#pragma unroll
                for (int j = 0; j < 4; ++j) zrow[j] = __ldg(zp + j);
            } else {                                       // a view whose rows start on no 16-byte boundary
                const unsigned short* zp = reinterpret_cast<const unsigned short*>(zr);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t* zw = reinterpret_cast<uint32_t*>(&zrow[j]);
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        zw[e] = (uint32_t)__ldg(zp + j * 8 + 2 * e) | ((uint32_t)__ldg(zp + j * 8 + 2 * e + 1) << 16);
                }
            }
        }
        bool ok = mbar_wait(g_ready, 0);
        if (!ok && lane == 0) { report(a.error, 5); *failed = 1; }
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            fence_after_sync();
            // 32 tokens s at a time, the row's two threads in turn; blocks above this warp's rows are zeros, the block
            // on the diagonal is masked, those below are not
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int cb = 2 * i + hf;
                uint8_t* w_row = b_s + i * kRowTile + (size_t)r * 128;
                if (cb > wq) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        *reinterpret_cast<uint4*>(w_row + (((hf * 4 + j) ^ (r & 7)) * 16)) = make_uint4(0u, 0u, 0u, 0u);
                } else {
                    uint32_t gv[32];
                    tmem_ld32(lane_addr + cb * 32, gv);
                    if (cb < wq) {                         // below the diagonal block: every token s counts
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint4 piece;
                            uint32_t* pw = reinterpret_cast<uint32_t*>(&piece);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int c = j * 8 + 2 * e;
                                const float4 ad = *reinterpret_cast<const float4*>(ad_s + cb * 32 + c);     // (a, dt) of two tokens
                                pw[e] = pack2(__uint_as_float(gv[c]) * ex2_approx(at - ad.x) * ad.y,
                                              __uint_as_float(gv[c + 1]) * ex2_approx(at - ad.z) * ad.w);
                            }
                            *reinterpret_cast<uint4*>(w_row + (((hf * 4 + j) ^ (r & 7)) * 16)) = piece;
                        }
                    } else {                               // the diagonal block: tokens s <= r
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint4 piece;
                            uint32_t* pw = reinterpret_cast<uint32_t*>(&piece);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int c = j * 8 + 2 * e, s0 = cb * 32 + c;
                                const float4 ad = *reinterpret_cast<const float4*>(ad_s + s0);
                                const float w0 = s0 <= r ? __uint_as_float(gv[c]) * ex2_approx(at - ad.x) * ad.y : 0.f;
                                const float w1 = s0 + 1 <= r ? __uint_as_float(gv[c + 1]) * ex2_approx(at - ad.z) * ad.w : 0.f;
                                pw[e] = pack2(w0, w1);
                            }
                            *reinterpret_cast<uint4*>(w_row + (((hf * 4 + j) ^ (r & 7)) * 16)) = piece;
                        }
                    }
                }
            }
            fence_async_smem();
            fence_before_sync();
            mbar_arrive(w_ready);
            ok = mbar_wait(y_ready, 0);
            if (!ok && lane == 0) { report(a.error, 6); *failed = 1; }
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            fence_after_sync();
            // this thread's 32 of the row's 64 head dims
            uint32_t y2[32], y1[32];
            tmem_ld32(lane_addr + 128 + hf * 32, y2);
            tmem_ld32(lane_addr + 192 + hf * 32, y1);
            if (r < Lc) {
                const float ea = exp2f(at), Dh = a.D[h];
                bf16* dst = a.y + (size_t)(tok0 + r) * inner + col0 + hf * 32;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 xv = *reinterpret_cast<const uint4*>(x_s + (size_t)r * 128 + (((hf * 4 + j) ^ (r & 7)) * 16));
                    const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv);
                    const __nv_bfloat162* zh = reinterpret_cast<const __nv_bfloat162*>(&zrow[j]);
                    uint4 piece;
                    uint32_t* pw = reinterpret_cast<uint32_t*>(&piece);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int c = j * 8 + 2 * e;
                        const float2 xf = __bfloat1622float2(xh[e]);
                        float v0 = fmaf(ea, __uint_as_float(y2[c]), __uint_as_float(y1[c])) + Dh * xf.x;
                        float v1 = fmaf(ea, __uint_as_float(y2[c + 1]), __uint_as_float(y1[c + 1])) + Dh * xf.y;
                        if (gated) {
                            const float2 zf = __bfloat1622float2(zh[e]);
                            const float z0 = round_to<bf16>(zf.x * a.gate_scale), z1 = round_to<bf16>(zf.y * a.gate_scale);
                            // SiLU by the fast exponential and division: its result is rounded to bfloat16 next
                            v0 = round_to<bf16>(v0) * round_to<bf16>(silu_fast(z0));
                            v1 = round_to<bf16>(v1) * round_to<bf16>(silu_fast(z1));
                        }
                        pw[e] = pack2(v0, v1);
                    }
                    *reinterpret_cast<uint4*>(dst + j * 8) = piece;
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    __syncwarp();
    if (warp == 1) tmem_free<kTmemCols>(tmem);
}

template <int NB>
int launch(const CUtensorMap& map_conv, const CUtensorMap& map_sin, const ScanArgs& a, int n_chunks, cudaStream_t s) {
    constexpr int kBTiles = NB > 2 ? NB : 2;
    const size_t smem = (size_t)(NB + kBTiles + 1) * kRowTile + (size_t)NB * kSinTile + 2 * kL * 4 + 16 + 64 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(ssd_chunk_scan_tc_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        configured = true;
    }
    ssd_chunk_scan_tc_kernel<NB><<<dim3(n_chunks, a.nh * (a.P / kP)), kThreads, smem, s>>>(map_conv, map_sin, a);
    return launch_status();
}
}  // namespace

// Does the tensor-core chunk scan take these sizes?  (Else kernel 3 of lb_ssd_prefill.)
extern "C" int lb_ssd_chunk_scan_tc_ok(int P, int N, int L) {
    return P >= kP && P % kP == 0 && P <= 256 && L == kL && N >= 64 && N <= 256 && N % 64 == 0 ? 1 : 0;
}

// The third step of lb_ssd_prefill (which is then called with run_scan = 0) for chunks of 128 tokens: conv
// [tokens, C] contiguous bfloat16 (x | B | C), s_in [n_chunks, nh, 64, N] bfloat16 as lb_ssd_prefill left it, y
// [tokens, nh * 64] contiguous.  `gate` (may be null): rows `gate_stride` elements apart (16-byte loads where they
// start on such boundaries).  `error`: a device int that is 0 before the call; non-zero afterwards: a wait inside the kernel
// gave up.
extern "C" int lb_ssd_chunk_scan_tc(const void* conv, long tokens, int C, const void* dt, long dt_stride,
                                    const float* A_log, const float* dt_bias, const float* D, void* y,
                                    const int* cu_seqlens, const int* chunks, int n_chunks, const void* s_in, int nh,
                                    int P, int N, int G, int L, float dt_scale, const void* gate, long gate_stride,
                                    float gate_scale, int* error, void* stream) {
    if (n_chunks <= 0) return kOk;
    if (!lb_ssd_chunk_scan_tc_ok(P, N, L) || nh <= 0 || G <= 0 || nh % G || C != nh * P + 2 * G * N) return kBadSize;
    if ((long)nh * (P / kP) > 65535 || (long)n_chunks * nh * P > 0x7fffffffL) return kTooLarge;
    if (((uintptr_t)conv | (uintptr_t)s_in | (uintptr_t)y) & 15) return kBadSize;
    CUtensorMap map_conv, map_sin;
    int rc = make_tile_map(&map_conv, conv, tokens, C, C, kL);
    if (rc == 0) rc = make_tile_map(&map_sin, s_in, (long)n_chunks * nh * P, N, N, kP);
    if (rc != 0) return rc;
    ScanArgs a{(const bf16*)dt, dt_stride, A_log, dt_bias, D, (bf16*)y, cu_seqlens, chunks, nh, P, N, G, dt_scale,
               (const bf16*)gate, gate_stride, gate_scale,
               (((uintptr_t)gate & 15) == 0 && gate_stride % 8 == 0) ? 1 : 0, error};
    cudaStream_t s = (cudaStream_t)stream;
    switch (N / 64) {
        case 1: return launch<1>(map_conv, map_sin, a, n_chunks, s);
        case 2: return launch<2>(map_conv, map_sin, a, n_chunks, s);
        case 3: return launch<3>(map_conv, map_sin, a, n_chunks, s);
        default: return launch<4>(map_conv, map_sin, a, n_chunks, s);
    }
}
