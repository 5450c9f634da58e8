// Chunked selective state-space scan (Mamba2 "SSD" form) for prompt portions, on tensor cores (bfloat16).
//
// The recurrence  S <- e^{dA_t} S + B_t (x) u_t ,  y_t = C_t . S + D x_t   (u_t = x_t dt_t; ssm.cu has the
// token-by-token kernel) is cut into chunks of L tokens.  With a_t the running sum of dA inside a chunk:
//
//   chunk state   dS   = sum_s e^{a_L - a_s} B_s (x) u_s                       [P x N]   (kernel 1, one CTA per chunk and head)
//   state pass    S_in(c+1) = e^{a_L(c)} S_in(c) + dS(c), from the request's saved state (zeros at
//                 position 0); the state after the last chunk goes back to the slot     (kernel 2, float32)
//   chunk scan    y_t  = e^{a_t} C_t . S_in + sum_{s<=t} [(C_t . B_s) e^{a_t - a_s} dt_s] x_s + D x_t      (kernel 3)
//
// (python/logssms/kernel/linear_attention/mamba2.py:148-194 and vendor/fla/chunk_o.py:79-136 of the
// reference, which fixes L = 64; here L is the configuration's chunk size.)  All three products of
// kernels 1 and 3 run on mma.sync m16n8k16 with bfloat16 operands and float32 accumulators; dt,
// softplus, the running sums and every decay factor are float32 (all exponents are <= 0); the state
// between chunks and in the slot is float32, and is rounded to bfloat16 only as the operand of
// C . S_in.  Portions have any length (the last chunk is masked) and resume from the saved state.
// Sizes: head_dim and state_dim multiples of 8, head_dim <= 128, state_dim <= 256, L <= 256; what
// does not fit is refused and the caller falls back to the token-by-token kernel.
#include "lb200/common.cuh"
using namespace lb200;

namespace {
typedef __nv_bfloat16 bf16;

struct SsdArgs {
    const bf16* conv; int C;                     // [tokens, C]: x | B | C after the conv
    const bf16* dt; long dt_stride;              // [tokens, nh] view
    const float* A_log; const float* dt_bias; const float* D;
    void* state;                                 // [slots, nh, P, N]: float32, or bfloat16 with `state_bf16`
    bf16* y;                                     // [tokens, nh * P]
    const int* cu_seqlens; const int* start_pos; const int* slots;
    const int* chunks;                           // [n_chunks][2]: request index, first token of the chunk in its portion
    const int* req_chunks;                       // [n_long][3]: request index, first chunk, number of chunks
    float* scratch;                              // [n_chunks, nh, P, N]: dS of every chunk
    bf16* s_in;                                  // [n_chunks, nh, P, N]: the state every chunk starts from, rounded
    float* chunk_a;                              // [n_chunks, nh]: a_L of the chunk
    int nh, P, N, G, L;
    float dt_scale;
    const bf16* gate; long gate_stride; float gate_scale;
    int state_bf16;
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;           // 0 bytes read: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;");
    asm volatile("cp.async.wait_group 0;");
}
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 p = __bfloat1622float2(h[i]); f[2 * i] = p.x; f[2 * i + 1] = p.y; }
}
__host__ __device__ constexpr int round_up(int v, int m) { return (v + m - 1) / m * m; }

// dt_s and the inclusive running sum a_s of dA over the chunk, for s < Lpad (s >= Lc: dt = 0, a = a_{Lc-1}).
// Every thread of the block must call it.  `tot` holds one float per warp.
__device__ void chunk_decay(const SsdArgs& a, int tok0, int Lc, int Lpad, int h, float* dt_s, float* a_s, float* tot) {
    const int s = threadIdx.x, lane = s & 31, warp = s >> 5;
    float dtv = 0.f, dA = 0.f;
    if (s < Lc) {
        dtv = round_to<bf16>(__bfloat162float(a.dt[(size_t)(tok0 + s) * a.dt_stride + h]) * a.dt_scale) + a.dt_bias[h];
        dtv = dtv > 20.f ? dtv : log1pf(expf(dtv));
        dA = -expf(a.A_log[h]) * dtv;
    }
    float run = dA;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, run, o);
        if (lane >= o) run += up;
    }
    if (lane == 31) tot[warp] = run;
    __syncthreads();
    float before = 0.f;
    for (int w = 0; w < warp; ++w) before += tot[w];
    if (s < Lpad) { dt_s[s] = dtv; a_s[s] = run + before; }
    __syncthreads();
}

// ---------------------------------------------------------------------------------------------- kernel 1
constexpr int kStateThreads = 256;

__global__ void __launch_bounds__(kStateThreads) ssd_chunk_state_kernel(SsdArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int chunk = blockIdx.x, h = blockIdx.y;
    const int b = a.chunks[2 * chunk], t0 = a.chunks[2 * chunk + 1];
    if (b < 0) return;                                  // a list entry without work: the lists of a step that was filled up to fixed sizes end in such entries
    const int begin = a.cu_seqlens[b], len = a.cu_seqlens[b + 1] - begin;
    const int Lc = min(a.L, len - t0), Lpad = round_up(a.L, 16);
    const int tok0 = begin + t0;
    const int P = a.P, N = a.N, Ppad = round_up(P, 16), Npad = round_up(N, 16);
    const int ldx = Ppad + 8, ldb = Npad + 8;
    float* dt_s = reinterpret_cast<float*>(smem_raw);           // [Lpad]
    float* a_s = dt_s + Lpad;                                   // [Lpad]
    float* tot = a_s + Lpad;                                    // [32]
    bf16* x_s = reinterpret_cast<bf16*>(tot + 32);              // [Lpad][ldx]  u_s * e^{a_L - a_s}
    bf16* b_s = x_s + Lpad * ldx;                               // [Lpad][ldb]
    // Everything the CTA reads is asked for before anything is waited for: B goes straight to shared memory
    // (cp.async, rows beyond the chunk and columns beyond N as zeros), the thread's pieces of x wait in registers
    // for the decay factors, which come from dt last.  One after the other these three were the kernel's time.
    const int g = h / (a.nh / a.G), inner = a.nh * P;
    const int npieces = Npad / 8;
    for (int i = threadIdx.x; i < Lpad * npieces; i += kStateThreads) {
        const int s = i / npieces, c = i % npieces;
        const bool valid = s < Lc && c * 8 < N;
        cp_async16(b_s + s * ldb + c * 8, a.conv + (size_t)(tok0 + (valid ? s : 0)) * a.C + inner + g * N + (valid ? c * 8 : 0), valid);
    }
    asm volatile("cp.async.commit_group;");
    const int ppieces = Ppad / 8;
    constexpr int kXAhead = 4;                                  // pieces of x a thread holds while the decay is computed
    uint4 xv[kXAhead];
#pragma unroll
    for (int u = 0; u < kXAhead; ++u) {
        const int i = threadIdx.x + u * kStateThreads, s = i / ppieces, p = (i % ppieces) * 8;
        xv[u] = make_uint4(0u, 0u, 0u, 0u);
        if (i < Lpad * ppieces && s < Lc && p < P)
            xv[u] = *reinterpret_cast<const uint4*>(a.conv + (size_t)(tok0 + s) * a.C + h * P + p);
    }
    chunk_decay(a, tok0, Lc, Lpad, h, dt_s, a_s, tot);
    const float aL = a_s[Lc - 1];
    for (int i0 = 0; i0 < Lpad * ppieces; i0 += kXAhead * kStateThreads) {
#pragma unroll
        for (int u = 0; u < kXAhead; ++u) {
            const int i = i0 + threadIdx.x + u * kStateThreads;
            if (i >= Lpad * ppieces) break;
            const int s = i / ppieces, p = (i % ppieces) * 8;
            uint4 raw = make_uint4(0u, 0u, 0u, 0u);
            const bool live = s < Lc && p < P;
            if (i0 == 0) raw = xv[u];
            else if (live) raw = *reinterpret_cast<const uint4*>(a.conv + (size_t)(tok0 + s) * a.C + h * P + p);
            uint4 packed = make_uint4(0u, 0u, 0u, 0u);
            if (live) {
                float f[8];
                unpack8(raw, f);
                const float dts = dt_s[s], wgt = expf(aL - a_s[s]);
                unsigned* o = reinterpret_cast<unsigned*>(&packed);
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    o[e] = pack_bf16(round_to<bf16>(f[2 * e] * dts) * wgt, round_to<bf16>(f[2 * e + 1] * dts) * wgt);
            }
            *reinterpret_cast<uint4*>(x_s + s * ldx + p) = packed;
        }
    }
    asm volatile("cp.async.wait_group 0;");
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, lg = lane >> 2, lt = lane & 3, mi = lane >> 3;
    const int ptiles = Ppad / 16, nchunks = (Npad + 63) / 64;
    float* out = a.scratch + ((size_t)chunk * a.nh + h) * P * N;
    for (int item = warp; item < ptiles * nchunks; item += kStateThreads / 32) {
        const int pt = item % ptiles, nc = item / ptiles;
        float acc[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
        for (int kk = 0; kk < Lpad / 16; ++kk) {
            unsigned xa[4];
            ldsm_x4_t(xa, x_s + (kk * 16 + (mi >> 1) * 8 + (lane & 7)) * ldx + pt * 16 + (mi & 1) * 8);
#pragma unroll
            for (int n2 = 0; n2 < 4; ++n2) {
                if (nc * 64 + n2 * 16 < Npad) {
                    unsigned bf[4];
                    ldsm_x4_t(bf, b_s + (kk * 16 + (mi & 1) * 8 + (lane & 7)) * ldb + nc * 64 + n2 * 16 + (mi >> 1) * 8);
                    mma_bf16(acc[2 * n2], xa, bf[0], bf[1]);
                    mma_bf16(acc[2 * n2 + 1], xa, bf[2], bf[3]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int n = nc * 64 + j * 8 + 2 * lt;
            if (n < N) {
                const int p0 = pt * 16 + lg, p1 = p0 + 8;
                if (p0 < P) *reinterpret_cast<float2*>(out + (size_t)p0 * N + n) = make_float2(acc[j][0], acc[j][1]);
                if (p1 < P) *reinterpret_cast<float2*>(out + (size_t)p1 * N + n) = make_float2(acc[j][2], acc[j][3]);
            }
        }
    }
    if (threadIdx.x == 0) a.chunk_a[(size_t)chunk * a.nh + h] = aL;
}

// ---------------------------------------------------------------------------------------------- kernel 2
// grid (long requests, heads, pieces of P*N/4); a thread owns four consecutive state values.
__global__ void __launch_bounds__(256) ssd_state_pass_kernel(SsdArgs a) {
    const int r = blockIdx.x, h = blockIdx.y;
    const int b = a.req_chunks[3 * r], c0 = a.req_chunks[3 * r + 1], nc = a.req_chunks[3 * r + 2];
    if (b < 0) return;                                  // a list entry without work: the lists of a step that was filled up to fixed sizes end in such entries
    const size_t per_head = (size_t)a.P * a.N;
    const size_t i = ((size_t)blockIdx.z * blockDim.x + threadIdx.x) * 4;
    if (i >= per_head) return;
    const size_t at = ((size_t)a.slots[b] * a.nh + h) * per_head + i;
    float* sp = (float*)a.state + at;
    bf16* sph = (bf16*)a.state + at;                    // the state as bfloat16 (state_bf16): four values are 8 bytes
    float4 S = make_float4(0.f, 0.f, 0.f, 0.f);
    if (a.start_pos[b] > 0) {
        if (a.state_bf16) {
            const uint2 v = *reinterpret_cast<const uint2*>(sph);
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
            S = make_float4(lo.x, lo.y, hi.x, hi.y);
        } else {
            S = *reinterpret_cast<const float4*>(sp);
        }
    }
    constexpr int kAhead = 4;                                    // chunks whose dS and decay are fetched together
    for (int c = c0; c < c0 + nc; c += kAhead) {
        float4 d[kAhead];
        float decay[kAhead];
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            if (c + u < c0 + nc) {
                d[u] = *reinterpret_cast<const float4*>(a.scratch + ((size_t)(c + u) * a.nh + h) * per_head + i);
                decay[u] = a.chunk_a[(size_t)(c + u) * a.nh + h];
            }
        }
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            if (c + u < c0 + nc) {
                // what the chunk starts from, as the bfloat16 operand of C . S_in
                *reinterpret_cast<uint2*>(a.s_in + ((size_t)(c + u) * a.nh + h) * per_head + i) =
                    make_uint2(pack_bf16(S.x, S.y), pack_bf16(S.z, S.w));
                const float e = expf(decay[u]);
                S.x = S.x * e + d[u].x; S.y = S.y * e + d[u].y; S.z = S.z * e + d[u].z; S.w = S.w * e + d[u].w;
            }
        }
    }
    if (a.state_bf16) *reinterpret_cast<uint2*>(sph) = make_uint2(pack_bf16(S.x, S.y), pack_bf16(S.z, S.w));
    else *reinterpret_cast<float4*>(sp) = S;
}

// ---------------------------------------------------------------------------------------------- kernel 3
// NKT: state_dim / 16 rounded up to the instantiated size; PT: head_dim / 8 likewise.  One warp per 16 tokens.
template <int NKT, int PT, int MAXT>
__global__ void __launch_bounds__(MAXT) ssd_chunk_scan_kernel(SsdArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int chunk = blockIdx.x, h = blockIdx.y;
    const int b = a.chunks[2 * chunk], t0 = a.chunks[2 * chunk + 1];
    if (b < 0) return;                                  // a list entry without work: the lists of a step that was filled up to fixed sizes end in such entries
    const int begin = a.cu_seqlens[b], len = a.cu_seqlens[b + 1] - begin;
    const int Lc = min(a.L, len - t0), Lpad = round_up(a.L, 16);
    const int tok0 = begin + t0;
    const int P = a.P, N = a.N, Ppad = round_up(P, 16), Npad = round_up(N, 16);
    const int ldn = Npad + 8, ldp = Ppad + 8;
    float* dt_s = reinterpret_cast<float*>(smem_raw);           // [Lpad]
    float* a_s = dt_s + Lpad;                                   // [Lpad]
    float* tot = a_s + Lpad;                                    // [32]
    bf16* c_s = reinterpret_cast<bf16*>(tot + 32);              // [Lpad][ldn]
    bf16* b_s = c_s + Lpad * ldn;                               // [Lpad][ldn]
    bf16* u_s = b_s + Lpad * ldn;                               // [Lpad][ldp]   x (dt rides in the masked scores)
    bf16* s_s = u_s + Lpad * ldp;                               // [Ppad][ldn]   S_in
    bf16* z_s = s_s + Ppad * ldn;                               // [Lpad][ldp]   the gate's rows (when there is one)
    const int g = h / (a.nh / a.G), inner = a.nh * P;
    const int threads = blockDim.x;
    // all four tiles come in 16-byte cp.async pieces (zeros outside the chunk and the real sizes)
    const int npieces = Npad / 8, ppieces = Ppad / 8;
    for (int i = threadIdx.x; i < Lpad * npieces; i += threads) {
        const int s = i / npieces, c = i % npieces;
        const bool ok = s < Lc && c * 8 < N;
        const bf16* row = a.conv + (size_t)(tok0 + (ok ? s : 0)) * a.C + inner + g * N + (ok ? c * 8 : 0);
        cp_async16(b_s + s * ldn + c * 8, row, ok);
        cp_async16(c_s + s * ldn + c * 8, row + a.G * N, ok);
    }
    for (int i = threadIdx.x; i < Lpad * ppieces; i += threads) {
        const int s = i / ppieces, p = (i % ppieces) * 8;
        const bool ok = s < Lc && p < P;
        cp_async16(u_s + s * ldp + p, a.conv + (size_t)(tok0 + (ok ? s : 0)) * a.C + h * P + (ok ? p : 0), ok);
    }
    const bf16* sin = a.s_in + ((size_t)chunk * a.nh + h) * P * N;
    for (int i = threadIdx.x; i < Ppad * npieces; i += threads) {
        const int p = i / npieces, n = (i % npieces) * 8;
        const bool ok = p < P && n < N;
        cp_async16(s_s + p * ldn + n, sin + (ok ? (size_t)p * N + n : 0), ok);
    }
    if (a.gate != nullptr) {
        // the gate is a view of a wider projection: 16-byte copies where its rows start on such boundaries
        const bool gate16 = ((uintptr_t)a.gate & 15) == 0 && a.gate_stride % 8 == 0;
        for (int i = threadIdx.x; i < Lpad * ppieces; i += threads) {
            const int s = i / ppieces, p = (i % ppieces) * 8;
            const bool ok = s < Lc && p < P;
            const bf16* src = a.gate + (size_t)(tok0 + (ok ? s : 0)) * a.gate_stride + h * P + (ok ? p : 0);
            if (gate16) {
                cp_async16(z_s + s * ldp + p, src, ok);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) z_s[s * ldp + p + e] = ok ? src[e] : __float2bfloat16_rn(0.f);
            }
        }
    }
    // the tiles are on their way while the decay factors are computed (that is a chain of its own: dt from
    // global memory, softplus, a prefix sum over the chunk)
    chunk_decay(a, tok0, Lc, Lpad, h, dt_s, a_s, tot);
    cp_async_wait_all();
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, lg = lane >> 2, lt = lane & 3, mi = lane >> 3;
    const int r0 = warp * 16;
    if (r0 >= Lc) return;
    // this warp's 16 rows of C as the left operand of both products
    unsigned cf[NKT][4];
#pragma unroll
    for (int kk = 0; kk < NKT; ++kk)
        if (kk * 16 < Npad) ldsm_x4(cf[kk], c_s + (r0 + (lane & 15)) * ldn + kk * 16 + (lane >> 4) * 8);
    float acc[PT][4];
#pragma unroll
    for (int j = 0; j < PT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    // e^{a_t} C_t . S_in
#pragma unroll
    for (int kk = 0; kk < NKT; ++kk) {
        if (kk * 16 < Npad) {
#pragma unroll
            for (int p2 = 0; p2 < PT / 2; ++p2) {
                if (p2 * 16 < Ppad) {
                    unsigned sf[4];
                    ldsm_x4(sf, s_s + (p2 * 16 + (mi >> 1) * 8 + (lane & 7)) * ldn + kk * 16 + (mi & 1) * 8);
                    mma_bf16(acc[2 * p2], cf[kk], sf[0], sf[1]);
                    mma_bf16(acc[2 * p2 + 1], cf[kk], sf[2], sf[3]);
                }
            }
        }
    }
    const float at0 = a_s[r0 + lg], at1 = a_s[r0 + lg + 8];
    const float e0 = expf(at0), e1 = expf(at1);
#pragma unroll
    for (int j = 0; j < PT; ++j) { acc[j][0] *= e0; acc[j][1] *= e0; acc[j][2] *= e1; acc[j][3] *= e1; }
    // sum over s <= t inside the chunk, 16 tokens s at a time
    for (int sb = 0; sb <= warp; ++sb) {
        float gs[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) gs[j][0] = gs[j][1] = gs[j][2] = gs[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < NKT; ++kk) {
            if (kk * 16 < Npad) {
                unsigned bf[4];
                ldsm_x4(bf, b_s + (sb * 16 + (mi >> 1) * 8 + (lane & 7)) * ldn + kk * 16 + (mi & 1) * 8);
                mma_bf16(gs[0], cf[kk], bf[0], bf[1]);
                mma_bf16(gs[1], cf[kk], bf[2], bf[3]);
            }
        }
        unsigned pa[4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float m[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int trow = r0 + lg + 8 * (e >> 1);
                const int s = sb * 16 + j * 8 + 2 * lt + (e & 1);
                const float at = (e >> 1) ? at1 : at0;
                m[e] = (s <= trow && s < Lc) ? gs[j][e] * expf(at - a_s[s]) * dt_s[s] : 0.f;
            }
            pa[2 * j] = pack_bf16(m[0], m[1]);
            pa[2 * j + 1] = pack_bf16(m[2], m[3]);
        }
#pragma unroll
        for (int p2 = 0; p2 < PT / 2; ++p2) {
            if (p2 * 16 < Ppad) {
                unsigned uf[4];
                ldsm_x4_t(uf, u_s + (sb * 16 + (mi & 1) * 8 + (lane & 7)) * ldp + p2 * 16 + (mi >> 1) * 8);
                mma_bf16(acc[2 * p2], pa, uf[0], uf[1]);
                mma_bf16(acc[2 * p2 + 1], pa, uf[2], uf[3]);
            }
        }
    }
    // + D x, optional gate, store
    const float Dh = a.D[h];
#pragma unroll
    for (int j = 0; j < PT; ++j) {
        const int p = j * 8 + 2 * lt;
        if (p < P) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int trow = r0 + lg + 8 * half;
                if (trow < Lc) {
                    const size_t tok = (size_t)(tok0 + trow);
                    const __nv_bfloat162 xv = *reinterpret_cast<const __nv_bfloat162*>(u_s + trow * ldp + p);
                    float y0 = acc[j][2 * half] + Dh * __bfloat162float(xv.x);
                    float y1 = acc[j][2 * half + 1] + Dh * __bfloat162float(xv.y);
                    if (a.gate != nullptr) {
                        const __nv_bfloat162 zv = *reinterpret_cast<const __nv_bfloat162*>(z_s + trow * ldp + p);
                        const float z0 = round_to<bf16>(__bfloat162float(zv.x) * a.gate_scale);
                        const float z1 = round_to<bf16>(__bfloat162float(zv.y) * a.gate_scale);
                        y0 = round_to<bf16>(y0) * round_to<bf16>(silu_f(z0));
                        y1 = round_to<bf16>(y1) * round_to<bf16>(silu_f(z1));
                    }
                    *reinterpret_cast<unsigned*>(a.y + tok * inner + h * P + p) = pack_bf16(y0, y1);
                }
            }
        }
    }
}

size_t state_smem(int L, int P, int N) {
    const int Lpad = round_up(L, 16), Ppad = round_up(P, 16), Npad = round_up(N, 16);
    return (size_t)(2 * Lpad + 32) * 4 + (size_t)Lpad * (Ppad + 8 + Npad + 8) * 2;
}
size_t scan_smem(int L, int P, int N) {
    const int Lpad = round_up(L, 16), Ppad = round_up(P, 16), Npad = round_up(N, 16);
    return (size_t)(2 * Lpad + 32) * 4 + ((size_t)2 * Lpad * (Npad + 8) + (size_t)2 * Lpad * (Ppad + 8) + (size_t)Ppad * (Npad + 8)) * 2;
}
constexpr size_t kSmemLimit = 200 * 1024;

template <int NKT, int PT, int MAXT>
int launch_scan(const SsdArgs& a, int n_chunks, cudaStream_t s) {
    const size_t smem = scan_smem(a.L, a.P, a.N);
    if (round_up(a.L, 16) * 2 > MAXT) return kTooLarge;
    static size_t have = 0;
    ensure_dynamic_smem(ssd_chunk_scan_kernel<NKT, PT, MAXT>, smem, have);
    ssd_chunk_scan_kernel<NKT, PT, MAXT><<<dim3(n_chunks, a.nh), round_up(a.L, 16) * 2, smem, s>>>(a);
    return launch_status();
}
// wide heads or states keep more of a row in registers: at most 8 warps (128 tokens) per chunk then
inline bool wide(int P, int N) { return N > 128 || P > 64; }
}  // namespace

// Chunk length the kernels use for a configured chunk size: at most `chunk`, at most kPreferredChunk (the work
// inside a chunk grows with its square, the work between chunks does not, and shorter chunks leave room for
// three CTAs per SM; the result does not depend on the cut beyond float32 rounding), halved until the
// shared-memory tiles fit; 0 when the sizes are not taken.
constexpr int kPreferredChunk = 64;
extern "C" int lb_ssd_chunk_len(int chunk, int P, int N) {
    if (P <= 0 || N <= 0 || P % 8 || N % 8 || P > 128 || N > 256 || chunk <= 0) return 0;
    int L = chunk > kPreferredChunk ? kPreferredChunk : chunk;
    if (wide(P, N) && L > 128) L = 128;
    while (L > 16 && (scan_smem(L, P, N) > kSmemLimit || state_smem(L, P, N) > kSmemLimit)) L = (L + 1) / 2;
    if (scan_smem(L, P, N) > kSmemLimit || state_smem(L, P, N) > kSmemLimit) return 0;
    return L;
}

extern "C" int lb_ssd_prefill(const void* conv, int C, const void* dt, long dt_stride, const float* A_log,
                              const float* dt_bias, const float* D, void* state, void* y, const int* cu_seqlens,
                              const int* start_pos, const int* slots, const int* chunks, int n_chunks,
                              const int* req_chunks, int n_long, float* scratch, void* s_in, float* chunk_a, int nh, int P, int N,
                              int G, int L, float dt_scale, const void* gate, long gate_stride, float gate_scale,
                              int run_scan, int state_bf16, int dtype, void* stream) {
    if (n_chunks <= 0 || n_long <= 0) return kOk;
    if (dtype != kBF16) return kBadDType;
    if (nh <= 0 || G <= 0 || nh % G || P <= 0 || N <= 0 || P % 8 || N % 8 || L <= 0) return kBadSize;
    if (C != nh * P + 2 * G * N) return kBadSize;
    if (P > 128 || N > 256 || L > 256 || nh > 65535) return kTooLarge;
    if ((run_scan && scan_smem(L, P, N) > kSmemLimit) || state_smem(L, P, N) > kSmemLimit) return kTooLarge;
    SsdArgs a{(const bf16*)conv, C, (const bf16*)dt, dt_stride, A_log, dt_bias, D, state, (bf16*)y, cu_seqlens,
              start_pos, slots, chunks, req_chunks, scratch, (bf16*)s_in, chunk_a, nh, P, N, G, L, dt_scale,
              (const bf16*)gate, gate_stride, gate_scale, state_bf16};
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem1 = state_smem(L, P, N);
    static size_t have1 = 0;
    ensure_dynamic_smem(ssd_chunk_state_kernel, smem1, have1);
    ssd_chunk_state_kernel<<<dim3(n_chunks, nh), kStateThreads, smem1, s>>>(a);
    int rc = launch_status();
    if (rc != 0) return rc;
    const int pieces = (int)(((size_t)P * N / 4 + 255) / 256);
    ssd_state_pass_kernel<<<dim3(n_long, nh, pieces), 256, 0, s>>>(a);
    rc = launch_status();
    if (rc != 0 || !run_scan) return rc;                 // run_scan 0: the caller runs lb_ssd_chunk_scan_tc behind this
    if (!wide(P, N)) return launch_scan<8, 8, 512>(a, n_chunks, s);
    return launch_scan<16, 16, 256>(a, n_chunks, s);
}
