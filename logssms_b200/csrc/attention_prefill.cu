// Causal grouped-query attention for prompt portions over the paged cache, on tensor cores (bfloat16).
//
// One CTA per (tile of 64 query tokens of one request, query head).  A group of 4 warps holds the 64 query
// rows (16 each); a CTA has up to 4 such groups, which take the key tiles in turn (group g: tiles g, g + NG,
// ...) with buffers and barriers of their own and merge their partial results through shared memory at the
// end: a tile's walk over the keys is a chain of dependent steps, and the longest chain (the last tile of a
// long prompt) sets the kernel's time, so it is cut into NG chains that run side by side.  The
// keys a tile may see (everything the request has in the cache up to the tile's last token, which
// includes earlier portions and the keys this step stored) are walked in tiles of 64: K and V rows
// are gathered page by page into shared memory with 16-byte cp.async (double buffered), S = Q K^T and
// O += P V run on mma.sync m16n8k16 (bfloat16 in, float32 accumulate), the softmax is the online
// form with float32 maximum, sum and output, masked by absolute position (causal, optional sliding
// window).  P is rounded to bfloat16 for the second product, as every flash-attention kernel does.
// Head sizes: multiples of 16 up to 256; any page size; any head counts (a CTA reads its key/value
// head's rows again for each query head of the group; they come from L2).
//
// Formula: python/logssms/layers/attention_backend/fi.py:175-190 (causal, scale head_dim^-1/2);
// chunked prompts: the query at absolute position p sees keys 0..p.
#include "lb200/common.cuh"
using namespace lb200;

namespace {
constexpr int kQTile = 64, kKTile = 64, kWarps = 4, kGroupThreads = kWarps * 32;
typedef __nv_bfloat16 bf16;

struct PrefillArgs {
    const bf16* q; const bf16* k_cache; const bf16* v_cache; bf16* out;
    const int* block_table; int bt_stride;
    const int* cu_seqlens; const int* start_pos;
    const int* tiles;                      // [n_tiles][2]: request index in the batch, first token of the tile in its portion
    int Hq, Hkv, hd, page_size, window;
    float scale_log2;                      // softmax scale * log2(e)
    int n_items, per_wave;                 // tiles * query heads; CTAs that start together (one per SM)
    int page_shift;                        // log2(page_size), or -1 when it is no power of two
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;           // 0 bytes read: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
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

// HDT: head_dim / 16, rounded up to the instantiated size (4, 8 or 16); loops are cut at the real hd.
// A barrier of one group's 128 threads (ids 1..4; a run-time id would make the compiler reserve all sixteen).
__device__ __forceinline__ void group_barrier(int group) {
    switch (group) {
        case 0: asm volatile("bar.sync 1, %0;" ::"n"(kGroupThreads) : "memory"); break;
        case 1: asm volatile("bar.sync 2, %0;" ::"n"(kGroupThreads) : "memory"); break;
        case 2: asm volatile("bar.sync 3, %0;" ::"n"(kGroupThreads) : "memory"); break;
        default: asm volatile("bar.sync 4, %0;" ::"n"(kGroupThreads) : "memory"); break;
    }
}
// Elements of shared memory per group: its two key and two value buffers, and room for its partial result
// (HDT * 2 + 1 float4 per thread) where small heads make the buffers smaller than that.
__host__ __device__ inline size_t group_elems(int hd, int hdt) {
    const size_t buffers = (size_t)4 * kKTile * (hd + 8), partial = (size_t)(hdt * 2 + 1) * kGroupThreads * 8;
    return buffers > partial ? buffers : partial;
}

// NG: groups of 4 warps that share the keys of the tile among them.
template <int HDT, int NG>
__global__ void __launch_bounds__(kGroupThreads * NG) attn_prefill_kernel(PrefillArgs a) {
    constexpr int kThreads = kGroupThreads * NG;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int hd = a.hd;
    const int ld = hd + 8;                               // row stride in elements: an odd number of 16-byte pieces
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);       // [64][ld]
    const int grp = threadIdx.x / kGroupThreads, tid_g = threadIdx.x % kGroupThreads;
    bf16* k_s = q_s + kQTile * ld + (size_t)grp * group_elems(hd, HDT);   // this group's [2][64][ld]
    bf16* v_s = k_s + 2 * kKTile * ld;                               // and [2][64][ld]
    const int warp = tid_g >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // The host lists the tiles heaviest first.  CTAs are handed to the SMs in rounds of one per SM; every
    // second round takes its items in reverse, so that the SM that got the heaviest item of one round
    // gets the lightest of the next (causal tiles differ by up to the whole context in cost).
    const int wave = blockIdx.x / a.per_wave, wave_pos = blockIdx.x % a.per_wave, wave_begin = wave * a.per_wave;
    const int item = (wave & 1) ? wave_begin + (min(a.per_wave, a.n_items - wave_begin) - 1 - wave_pos) : (int)blockIdx.x;
    const int tile = item / a.Hq;
    const int b = a.tiles[2 * tile], q0 = a.tiles[2 * tile + 1];
    if (b < 0) return;                                  // a list entry without work: the lists of a step that was filled up to fixed sizes end in such entries
    const int h = item % a.Hq, kvh = h / (a.Hq / a.Hkv);
    const int begin = a.cu_seqlens[b], len = a.cu_seqlens[b + 1] - begin;
    const int rows = min(kQTile, len - q0);              // valid query rows of this tile
    const int pos0 = a.start_pos[b] + q0;                // absolute position of row 0
    const int last_pos = pos0 + rows - 1;
    const int lo = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    const int* bt = a.block_table + (size_t)b * a.bt_stride;
    const int pieces = hd / 8;

    // Q tile -> shared memory (rows beyond the portion: zeros)
    for (int i = threadIdx.x; i < kQTile * pieces; i += kThreads) {
        const int r = i / pieces, c = i % pieces;
        const bf16* src = a.q + ((size_t)(begin + q0 + min(r, rows - 1)) * a.Hq + h) * hd + c * 8;
        cp_async16(q_s + r * ld + c * 8, src, r < rows);
    }
    const int kt_begin = lo / kKTile, kt_end = last_pos / kKTile + 1;
    // two threads per key row: one page lookup per row and tile, then 16-byte pieces side by side
    const int ld_row = tid_g >> 1, ld_half = tid_g & 1;
    const int ld_c0 = ld_half * ((pieces + 1) / 2), ld_c1 = ld_half ? pieces : (pieces + 1) / 2;
    auto load_kv = [&](int kt, int buf) {
        const int j = kt * kKTile + ld_row;
        const bool valid = j >= lo && j <= last_pos;
        size_t off = 0;
        if (valid) {
            const int page = a.page_shift >= 0 ? (j >> a.page_shift) : j / a.page_size;
            const int in_page = j - page * a.page_size;
            off = (((size_t)bt[page] * a.page_size + in_page) * a.Hkv + kvh) * hd;
        }
        bf16* kd = k_s + (buf * kKTile + ld_row) * ld;
        bf16* vd = v_s + (buf * kKTile + ld_row) * ld;
        for (int c = ld_c0; c < ld_c1; ++c) {
            cp_async16(kd + c * 8, a.k_cache + off + c * 8, valid);
            cp_async16(vd + c * 8, a.v_cache + off + c * 8, valid);
        }
    };
    cp_async_commit();                                   // the queries
    if (kt_begin + grp < kt_end) load_kv(kt_begin + grp, 0);
    cp_async_commit();
    if (NG > 1) {                                        // the queries came through every group's threads
        cp_async_wait<1>();
        __syncthreads();
    }

    float o[HDT * 2][4];
#pragma unroll
    for (int i = 0; i < HDT * 2; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // rows g and g + 8 of this warp's 16
    const int row0 = warp * 16 + g, row1 = row0 + 8;
    const int p0 = pos0 + row0, p1 = pos0 + row1;                  // absolute positions (rows beyond `rows` are never stored)
    const int lo0 = a.window > 0 ? p0 - a.window + 1 : 0, lo1 = a.window > 0 ? p1 - a.window + 1 : 0;

    for (int kt = kt_begin + grp, buf = 0; kt < kt_end; kt += NG, buf ^= 1) {
        if (kt + NG < kt_end) load_kv(kt + NG, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        group_barrier(grp);
        const bf16* kb = k_s + buf * kKTile * ld;
        const bf16* vb = v_s + buf * kKTile * ld;
        if (warp * 16 < rows) {
            // S = Q K^T for this warp's 16 rows and the tile's 64 keys
            float s[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < HDT; ++kk) {
                if (kk * 16 < hd) {
                    unsigned qa[4];
                    ldsm_x4(qa, q_s + (warp * 16 + (lane & 15)) * ld + kk * 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int n2 = 0; n2 < 4; ++n2) {           // two key tiles of 8 per ldmatrix
                        unsigned kf[4];
                        const int mi = lane >> 3;
                        ldsm_x4(kf, kb + (n2 * 16 + (mi >> 1) * 8 + (lane & 7)) * ld + kk * 16 + (mi & 1) * 8);
                        mma_bf16(s[2 * n2], qa, kf[0], kf[1]);
                        mma_bf16(s[2 * n2 + 1], qa, kf[2], kf[3]);
                    }
                }
            }
            // mask by absolute position (only on tiles that some row does not see whole), running maximum
            const int j0 = kt * kKTile;
            const bool whole = j0 + kKTile - 1 <= pos0 && (a.window <= 0 || j0 >= pos0 + kQTile - a.window);
            float mx0 = -INFINITY, mx1 = -INFINITY;
            if (!whole) {
#pragma unroll
                for (int n = 0; n < 8; ++n) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = j0 + n * 8 + 2 * t + (e & 1);
                        const bool ok = e < 2 ? (j <= p0 && j >= lo0) : (j <= p1 && j >= lo1);
                        if (!ok) s[n][e] = -INFINITY;
                    }
                }
            }
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
                mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            // m0, m1: running maxima of the scaled scores (log2 units); a row that has seen no key keeps -inf,
            // and 0 then stands in as the reference so that exp2(-inf - 0) = 0
            mx0 = fmaxf(m0, mx0 * a.scale_log2);
            mx1 = fmaxf(m1, mx1 * a.scale_log2);
            const float ref0 = mx0 == -INFINITY ? 0.f : mx0, ref1 = mx1 == -INFINITY ? 0.f : mx1;
            const float alpha0 = exp2f(m0 - ref0), alpha1 = exp2f(m1 - ref1);
            m0 = mx0; m1 = mx1;
            float sum0 = 0.f, sum1 = 0.f;
            unsigned pa[4][4];                                  // P as the A operand: 4 k-steps of 16 keys
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const float e0 = exp2f(fmaf(s[n][0], a.scale_log2, -ref0)), e1 = exp2f(fmaf(s[n][1], a.scale_log2, -ref0));
                const float e2 = exp2f(fmaf(s[n][2], a.scale_log2, -ref1)), e3 = exp2f(fmaf(s[n][3], a.scale_log2, -ref1));
                sum0 += e0 + e1; sum1 += e2 + e3;
                pa[n >> 1][(n & 1) * 2] = pack_bf16(e0, e1);
                pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16(e2, e3);
            }
            l0 = l0 * alpha0 + sum0;
            l1 = l1 * alpha1 + sum1;
#pragma unroll
            for (int i = 0; i < HDT * 2; ++i) { o[i][0] *= alpha0; o[i][1] *= alpha0; o[i][2] *= alpha1; o[i][3] *= alpha1; }
            // O += P V
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                for (int d2 = 0; d2 < HDT; ++d2) {               // two output tiles of 8 columns per ldmatrix
                    if (d2 * 16 < hd) {
                        unsigned vf[4];
                        const int mi = lane >> 3;
                        ldsm_x4_t(vf, vb + (kk * 16 + (mi & 1) * 8 + (lane & 7)) * ld + d2 * 16 + (mi >> 1) * 8);
                        mma_bf16(o[2 * d2], pa[kk], vf[0], vf[1]);
                        mma_bf16(o[2 * d2 + 1], pa[kk], vf[2], vf[3]);
                    }
                }
            }
        }
        group_barrier(grp);
    }
    cp_async_wait<0>();
    if (NG > 1) {
        // groups 1.. leave their partial results (in the threads' own fragment order) in their key buffers;
        // group 0 folds them into its own
        float4* part = reinterpret_cast<float4*>(k_s);   // [HDT * 2 + 1][128] per group
        if (grp > 0) {
#pragma unroll
            for (int i = 0; i < HDT * 2; ++i) part[i * kGroupThreads + tid_g] = make_float4(o[i][0], o[i][1], o[i][2], o[i][3]);
            part[HDT * 2 * kGroupThreads + tid_g] = make_float4(m0, m1, l0, l1);
        }
        __syncthreads();
        if (grp > 0) return;
#pragma unroll
        for (int other = 1; other < NG; ++other) {
            const float4* theirs = reinterpret_cast<const float4*>(k_s + (size_t)other * group_elems(hd, HDT));
            const float4 ml = theirs[HDT * 2 * kGroupThreads + tid_g];
            const float n0 = fmaxf(m0, ml.x), n1 = fmaxf(m1, ml.y);
            const float r0 = n0 == -INFINITY ? 0.f : n0, r1 = n1 == -INFINITY ? 0.f : n1;
            const float fa0 = exp2f(m0 - r0), fb0 = exp2f(ml.x - r0), fa1 = exp2f(m1 - r1), fb1 = exp2f(ml.y - r1);
            m0 = n0; m1 = n1;
            l0 = l0 * fa0 + ml.z * fb0;
            l1 = l1 * fa1 + ml.w * fb1;
#pragma unroll
            for (int i = 0; i < HDT * 2; ++i) {
                const float4 v = theirs[i * kGroupThreads + tid_g];
                o[i][0] = o[i][0] * fa0 + v.x * fb0; o[i][1] = o[i][1] * fa0 + v.y * fb0;
                o[i][2] = o[i][2] * fa1 + v.z * fb1; o[i][3] = o[i][3] * fa1 + v.w * fb1;
            }
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = 1.f / l0, inv1 = 1.f / l1;
#pragma unroll
    for (int i = 0; i < HDT * 2; ++i) {
        const int d = i * 8 + 2 * t;
        if (d < hd) {
            if (row0 < rows)
                *reinterpret_cast<unsigned*>(a.out + ((size_t)(begin + q0 + row0) * a.Hq + h) * hd + d) =
                    pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
            if (row1 < rows)
                *reinterpret_cast<unsigned*>(a.out + ((size_t)(begin + q0 + row1) * a.Hq + h) * hd + d) =
                    pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
        }
    }
}

template <int HDT, int NG>
int launch_hdt(const PrefillArgs& a, int n_tiles, cudaStream_t s) {
    const size_t smem = ((size_t)kQTile * (a.hd + 8) + NG * group_elems(a.hd, HDT)) * sizeof(bf16);
    static size_t have = 0;
    ensure_dynamic_smem(attn_prefill_kernel<HDT, NG>, smem, have);
    attn_prefill_kernel<HDT, NG><<<dim3(a.n_items), kGroupThreads * NG, smem, s>>>(a);
    return launch_status();
}
}  // namespace

// q, out: [tokens, Hq, hd] bfloat16; caches [pages, page_size, Hkv, hd]; tiles: int32 [n_tiles, 2]
// (request index, first token of the tile within the request's portion; 64 tokens per tile).
extern "C" int lb_attention_prefill(const void* q, const void* k_cache, const void* v_cache, void* out,
                                    const int* block_table, int bt_stride, const int* cu_seqlens,
                                    const int* start_pos, const int* tiles, int n_tiles, int Hq, int Hkv, int hd,
                                    int page_size, float scale, int window, int dtype, void* stream) {
    if (n_tiles <= 0) return kOk;
    if (dtype != kBF16) return kBadDType;
    if (hd <= 0 || hd > 256 || hd % 16 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || page_size <= 0) return kBadSize;
    if ((long)n_tiles * Hq > 0x7fffffffL) return kTooLarge;
    static int num_sms = 0;
    if (num_sms == 0) {
        int device = 0, count = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) count = 148;
        num_sms = count;
    }
    PrefillArgs a{(const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, block_table, bt_stride,
                  cu_seqlens, start_pos, tiles, Hq, Hkv, hd, page_size, window, scale * 1.4426950408889634f,
                  n_tiles * Hq, num_sms, -1};
    for (int sh = 0; sh < 31; ++sh) if ((1 << sh) == page_size) a.page_shift = sh;
    // Groups per CTA.  Measured on a 2,048-token prompt of 8 heads of 64: 57 us with one group, 42 with two (two
    // CTAs per SM), 44 with four (one CTA per SM); 256-wide heads fill the shared memory with one group.
    if (hd <= 64) return launch_hdt<4, 2>(a, n_tiles, (cudaStream_t)stream);
    if (hd <= 128) return launch_hdt<8, 2>(a, n_tiles, (cudaStream_t)stream);
    return launch_hdt<16, 1>(a, n_tiles, (cudaStream_t)stream);
}
