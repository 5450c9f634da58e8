// One launch for the attention of a decode step: every token of the batch is the only new token of its
// request.  What otherwise takes three launches (rotate + store, split-KV attention, merge) is one:
//
//   * the CTA reads its query heads straight from the q|k|v projection and rotates them while loading;
//   * the CTA whose key range ends at the token's own position rotates the new key (after the key
//     multiplier), keeps it and the new value in shared memory for its own use, and (one CTA per
//     key/value head) stores both into the page cache;
//   * keys and values of a 32-key tile are all requested before any arithmetic starts (the kernel lives
//     on memory-level parallelism: a decode step is bound by reading the cache once);
//   * with several ranges per token, the CTA that finishes last (a counter per token and head group,
//     bumped after a fence) merges the ranges' partial results, so no second launch is needed.  The
//     counter returns to zero for the next call.  Nobody ever waits on anybody.
//
// Rotation: python/logssms/kernel/fused.py:161-256 (key scaled and rounded before the rotation,
// half-split pairing); attention: python/logssms/layers/attention_backend/fi.py:175-190.
// Softmax statistics and accumulators are float32, exp is expf.  Head sizes: multiples of 16 up to 256.
#include "lb200/common.cuh"
#include "lb200/tcgen05.cuh"
using namespace lb200;

namespace {
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;

struct FusedArgs {
    const void* qkv; long row_stride;              // [tokens, (Hq + 2 Hkv) * hd], columns q | k | v
    void* k_cache; void* v_cache; void* out;       // caches [pages, page_size, Hkv, hd]; out [tokens, Hq, hd]
    const int* block_table; int bt_stride;
    const int* token_req; const int* positions; const int* slot_mapping;
    const float* cos_sin; int table_rows; int rotary_dim;
    float* part_o; float* part_ml; int* counters;
    int Hq, Hkv, hd, page_size, window, splits, head_tiles, write_kv;
    float scale, key_scale;
    // the tensor-core form only: the step rows of the call's tokens (null: rows 0 .. tokens - 1), and whether the
    // queries still have to be rotated (0: `qkv` holds rotated queries, [rows, Hq * hd]; then write_kv is 0 as well)
    const int* token_list; int rotate;
    int* error;                                    // the tile-copy form only: where a wait that gave up records itself
};

// eight consecutive elements held raw in registers until they are needed
template <typename T> struct Raw8;
template <> struct Raw8<__nv_bfloat16> {
    uint4 v;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void zero() { v = make_uint4(0u, 0u, 0u, 0u); }
    __device__ __forceinline__ void get(float* f) const {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
    }
};
template <> struct Raw8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) {
        a = *reinterpret_cast<const float4*>(p); b = *reinterpret_cast<const float4*>(p + 4);
    }
    __device__ __forceinline__ void zero() { a = b = make_float4(0.f, 0.f, 0.f, 0.f); }
    __device__ __forceinline__ void get(float* f) const {
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
};

// rotated value of column c of a head row `src` (values already scaled/rounded by `pre`)
template <typename T>
__device__ __forceinline__ float rotated(const T* src, int c, int rotary_dim, const float* cs, float pre, bool round_pre) {
    float val = to_f32(src[c]) * pre;
    if (round_pre) val = round_to<T>(val);
    if (c < rotary_dim) {
        const int half = rotary_dim >> 1;
        const int f = c < half ? c : c - half;
        float partner = to_f32(src[c < half ? c + half : c - half]) * pre;
        if (round_pre) partner = round_to<T>(partner);
        val = val * cs[f] + (c < half ? -partner : partner) * cs[half + f];
    }
    return round_to<T>(val);
}

// GT: query heads per CTA.  CHP: 8-element pieces per head row, rounded up to a power of two (2..32).
template <typename T, int GT, int CHP>
__global__ void __launch_bounds__(kThreads) attn_decode_fused_kernel(FusedArgs a) {
    extern __shared__ float smem[];
    const int hd = a.hd;
    float* q_s = smem;                                   // [GT][hd]  rotated queries, pre-scaled
    float* kn_s = q_s + GT * hd;                         // [hd]      the token's own key (rotated)
    float* vn_s = kn_s + hd;                             // [hd]      the token's own value
    float* mrg = vn_s + hd;                              // [kWarps][GT][hd + 2]
    __shared__ int last_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t t = blockIdx.x;
    const int kvh = blockIdx.y / a.head_tiles, ht = blockIdx.y % a.head_tiles;
    const int G = a.Hq / a.Hkv;
    const int h0 = kvh * G + ht * GT;
    const int nheads = min(GT, G - ht * GT);
    const int split = blockIdx.z;
    const int pos = a.positions[t];
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int n = pos - lo + 1;
    // a range is never shorter than one tile per warp; ranges beyond the context have no CTA work at all
    const int chunk = (max((n + a.splits - 1) / a.splits, kWarps * 32) + 31) / 32 * 32;
    const int used = (n + chunk - 1) / chunk;            // ranges that hold keys
    if (split >= used) return;
    const int begin = lo + split * chunk;
    const int end = min(begin + chunk, pos + 1);
    const bool use_new = a.write_kv != 0;                // else the own position was stored by another layer
    const bool owns_new = use_new && begin <= pos && pos < end;     // this CTA's range holds the token's own key
    const int* bt = a.block_table + (size_t)a.token_req[t] * a.bt_stride;
    const T* row = (const T*)a.qkv + t * a.row_stride;
    const float* cs = a.cos_sin + (size_t)min(max(pos, 0), a.table_rows - 1) * a.rotary_dim;

    for (int i = threadIdx.x; i < GT * hd; i += kThreads) {
        const int g = i / hd, c = i % hd;
        q_s[i] = g < nheads ? rotated<T>(row + (size_t)(h0 + g) * hd, c, a.rotary_dim, cs, 1.f, false) * a.scale : 0.f;
    }
    if (owns_new) {
        const T* ksrc = row + (size_t)(a.Hq + kvh) * hd;
        const T* vsrc = row + (size_t)(a.Hq + a.Hkv + kvh) * hd;
        const long slot = a.slot_mapping[t];
        const bool store = ht == 0 && slot >= 0;
        for (int c = threadIdx.x; c < hd; c += kThreads) {
            const float kv = rotated<T>(ksrc, c, a.rotary_dim, cs, a.key_scale, true);
            const float vv = to_f32(vsrc[c]);
            kn_s[c] = kv; vn_s[c] = vv;
            if (store) {
                ((T*)a.k_cache)[((size_t)slot * a.Hkv + kvh) * hd + c] = from_f32<T>(kv);
                ((T*)a.v_cache)[((size_t)slot * a.Hkv + kvh) * hd + c] = vsrc[c];
            }
        }
    }
    __syncthreads();

    constexpr int KPI = 32 / CHP;                        // keys per value-load instruction
    constexpr int KB = CHP < 8 ? CHP : 8;                // pieces of a key row fetched together
    constexpr int VB = CHP < 8 ? CHP : 8;                // value-load instructions fetched together
    const int piece = lane % CHP, ksub = lane / CHP;
    const bool piece_ok = piece * 8 < hd;
    const int pieces = hd / 8;
    float acc[GT][8];
    float m[GT], l[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
    }
    const T* kc = (const T*)a.k_cache;
    const T* vc = (const T*)a.v_cache;

    for (int j0 = begin + warp * 32; j0 < end; j0 += kWarps * 32) {
        const int j = j0 + lane;
        const bool valid = j < end;
        const bool from_cache = valid && !(use_new && j == pos);       // the token's own key and value come from shared memory
        long krow = 0;
        if (from_cache) krow = (long)bt[j / a.page_size] * a.page_size + (j % a.page_size);
        const int count = min(32, end - j0);
        const int own_key = (use_new && pos >= j0 && pos < j0 + 32) ? pos - j0 : -1;   // lane of the own key in this tile

        float s[GT];
#pragma unroll
        for (int g = 0; g < GT; ++g) s[g] = 0.f;
        Raw8<T> vreg[VB];
#pragma unroll 1
        for (int kb = 0; kb < CHP; kb += KB) {
            // this batch of key pieces, and on the first pass the first batch of value pieces, all in flight together
            Raw8<T> kreg[KB];
#pragma unroll
            for (int c = 0; c < KB; ++c) {
                if (from_cache && kb + c < pieces) kreg[c].load(kc + ((size_t)krow * a.Hkv + kvh) * hd + (kb + c) * 8);
                else kreg[c].zero();
            }
            if (kb == 0) {
#pragma unroll
                for (int i = 0; i < VB; ++i) {
                    const int key = i * KPI + ksub;
                    const long rj = __shfl_sync(0xffffffffu, krow, key);
                    if (key < count && key != own_key && piece_ok) vreg[i].load(vc + ((size_t)rj * a.Hkv + kvh) * hd + piece * 8);
                    else vreg[i].zero();
                }
            }
#pragma unroll
            for (int c = 0; c < KB; ++c) {
                if (kb + c < pieces) {
                    float f[8];
                    kreg[c].get(f);
                    if (valid && !from_cache) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) f[e] = kn_s[(kb + c) * 8 + e];
                    }
#pragma unroll
                    for (int g = 0; g < GT; ++g) {
                        const float* qg = q_s + g * hd + (kb + c) * 8;
#pragma unroll
                        for (int e = 0; e < 8; ++e) s[g] = fmaf(qg[e], f[e], s[g]);
                    }
                }
            }
        }
        float p[GT];
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            const float m_new = fmaxf(m[g], warp_max(valid ? s[g] : -INFINITY));
            const float alpha = expf(m[g] - m_new);          // m = -inf at first: exp(-inf) = 0
            p[g] = valid ? expf(s[g] - m_new) : 0.f;
            l[g] = l[g] * alpha + p[g];
            m[g] = m_new;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] *= alpha;
        }
#pragma unroll 1
        for (int vb = 0; vb < CHP; vb += VB) {
            if (vb > 0) {
#pragma unroll
                for (int i = 0; i < VB; ++i) {
                    const int key = (vb + i) * KPI + ksub;
                    const long rj = __shfl_sync(0xffffffffu, krow, key);
                    if (key < count && key != own_key && piece_ok) vreg[i].load(vc + ((size_t)rj * a.Hkv + kvh) * hd + piece * 8);
                    else vreg[i].zero();
                }
            }
#pragma unroll
            for (int i = 0; i < VB; ++i) {
                const int key = (vb + i) * KPI + ksub;
                float pj[GT];
#pragma unroll
                for (int g = 0; g < GT; ++g) pj[g] = __shfl_sync(0xffffffffu, p[g], key);
                if (key < count && piece_ok) {
                    float f[8];
                    vreg[i].get(f);
                    if (key == own_key) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) f[e] = vn_s[piece * 8 + e];
                    }
#pragma unroll
                    for (int g = 0; g < GT; ++g)
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pj[g], f[e], acc[g][e]);
                }
            }
        }
    }
    // lanes that hold the same columns -> lane `piece`
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        l[g] = warp_sum(l[g]);
#pragma unroll
        for (int o = CHP; o < 32; o <<= 1)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], o);
    }
    const int stride = hd + 2;
    if (lane < CHP && piece_ok) {
#pragma unroll
        for (int g = 0; g < GT; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) mrg[(warp * GT + g) * stride + piece * 8 + e] = acc[g][e];
    }
    if (lane == 0) {
#pragma unroll
        for (int g = 0; g < GT; ++g) { mrg[(warp * GT + g) * stride + hd] = m[g]; mrg[(warp * GT + g) * stride + hd + 1] = l[g]; }
    }
    __syncthreads();
    const size_t group = t * (size_t)(a.Hkv * a.head_tiles) + blockIdx.y;      // (token, kv head, head tile)
    for (int i = threadIdx.x; i < nheads * hd; i += kThreads) {
        const int g = i / hd, d = i % hd;
        float mt = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mt = fmaxf(mt, mrg[(w * GT + g) * stride + hd]);
        float lt = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float mw = mrg[(w * GT + g) * stride + hd];
            const float f = mw == -INFINITY ? 0.f : expf(mw - mt);
            lt += mrg[(w * GT + g) * stride + hd + 1] * f;
            o += mrg[(w * GT + g) * stride + d] * f;
        }
        const int h = h0 + g;
        if (used == 1) {
            ((T*)a.out)[(t * a.Hq + h) * hd + d] = from_f32<T>(o / lt);
        } else {
            const size_t slot = ((size_t)t * a.Hq + h) * a.splits + split;
            a.part_o[slot * hd + d] = o;
            if (d == 0) { a.part_ml[slot * 2] = mt; a.part_ml[slot * 2 + 1] = lt; }
        }
    }
    if (used == 1) return;
    // the last CTA of this (token, head group) to get here merges all ranges
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int done = atomicAdd(a.counters + group, 1);
        last_flag = done == used - 1;
        if (last_flag) a.counters[group] = 0;              // ready for the next call
    }
    __syncthreads();
    if (!last_flag) return;
    __threadfence();
    for (int i = threadIdx.x; i < nheads * hd; i += kThreads) {
        const int g = i / hd, d = i % hd;
        const int h = h0 + g;
        const size_t base = ((size_t)t * a.Hq + h) * a.splits;
        float mt = -INFINITY;
        for (int s2 = 0; s2 < used; ++s2) mt = fmaxf(mt, __ldcg(a.part_ml + (base + s2) * 2));
        float lt = 0.f, o = 0.f;
        for (int s2 = 0; s2 < used; ++s2) {
            const float ms = __ldcg(a.part_ml + (base + s2) * 2);
            const float f = expf(ms - mt);
            lt += __ldcg(a.part_ml + (base + s2) * 2 + 1) * f;
            o += __ldcg(a.part_o + (base + s2) * hd + d) * f;
        }
        ((T*)a.out)[(t * a.Hq + h) * hd + d] = from_f32<T>(o / lt);
    }
}

template <typename T, int GT>
int launch_chp(const FusedArgs& a, int tokens, cudaStream_t s) {
    const int pieces = a.hd / 8;
    dim3 grid(tokens, a.Hkv * a.head_tiles, a.splits);
    const size_t smem = (size_t)(GT * a.hd + 2 * a.hd + kWarps * GT * (a.hd + 2)) * sizeof(float);
#define LB_CHP(N)                                                                                          \
    {                                                                                                      \
        if (smem > 48 * 1024)                                                                              \
            cudaFuncSetAttribute(attn_decode_fused_kernel<T, GT, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        attn_decode_fused_kernel<T, GT, N><<<grid, kThreads, smem, s>>>(a);                                \
    }
    if (pieces <= 2) LB_CHP(2)
    else if (pieces <= 4) LB_CHP(4)
    else if (pieces <= 8) LB_CHP(8)
    else if (pieces <= 16) LB_CHP(16)
    else LB_CHP(32)
#undef LB_CHP
    return launch_status();
}

// ------------------------------------------------------------------------------------------------
// The same step on tensor cores (bfloat16, head_dim <= 128, at most 16 query heads per key/value head).
// The query heads that share a key/value head are the 16 rows of an mma.sync m16n8k16 tile; every warp
// walks its own 32-key tiles of the CTA's range: K and V rows arrive by 16-byte cp.async into the warp's
// own ring of buffers (4 for head sizes up to 64, else 2) (the next tiles are in flight while this one is used), S = Q K^T and O += P V are
// tensor-core products, the softmax statistics stay float32.  Per 32 keys this costs ~200 instructions
// where the kernel above needs ~2000, and the copies keep the memory system busy with few warps.
typedef __nv_bfloat16 bf16;
constexpr int kKT = 32;                                  // keys per tile

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;                        // 0 bytes read: the 16 bytes are filled with zeros
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

// Distributed shared memory: the address of one's own shared variable in the CTA of rank `rank` of the cluster.
__device__ __forceinline__ unsigned cluster_map(const void* p, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ float ld_cluster(unsigned addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
// every thread of every CTA of the cluster (a hardware barrier: the CTAs of a cluster run together)
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// HDT: head_dim / 16 rounded up to the instantiated size (4 or 8).
// CL: the key ranges of a token and key/value head are the CTAs of one thread-block cluster (2 to 8 of them): their
// partial results meet through distributed shared memory and two cluster barriers instead of global memory, a
// fence, an atomic counter and the loads of the last CTA - about 2 us off a kernel of 13.
// TMA: a tile's keys and values come as boxes of 32 cache rows x 64 dims through the tensor maps (128-byte swizzle,
// one lane asks, an mbarrier per stage tells the warp that they landed) instead of 16 cp.async per lane with their
// address arithmetic: the loop of a 32-key tile was several hundred instructions, most of them not arithmetic, and
// with two warps per scheduler it was the issue rate, not the memory system, that bounded a batch of 64 at
// 4 TB/s.  Needs head_dim 64 or 128, pages of a multiple of the tile, no window.
// KT: keys per tile, 32, or 16 for heads of 128 by TMA: a stage is then 8 KB as for heads of 64, and two CTAs
// share an SM instead of one with its four warps.
template <int HDT, int NS, bool CL, bool TMA, int KT>
__global__ void __launch_bounds__(kThreads) attn_decode_mma_kernel(FusedArgs a, const __grid_constant__ CUtensorMap map_k,
                                                                   const __grid_constant__ CUtensorMap map_v) {
    extern __shared__ __align__(16) unsigned char smem_dyn[];
    // the tile-copy form wants its tiles on a 1024-byte boundary (the swizzle pattern repeats every 1024 bytes)
    unsigned char* smem_raw = TMA ? smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u) : smem_dyn;
    const int hd = a.hd, ld = hd + 8;                    // row stride of q (and of cp.async tiles): an odd number of 16-byte pieces
    constexpr int kTileElems = KT * HDT * 16;            // TMA: K (or V) of one tile: HDT / 4 blocks of KT rows x 64 values
    constexpr int kStageElems = 2 * kTileElems;          //      K and V of a stage
    bf16* tiles;                                         // cp.async: [kWarps][NS stages][K, V][KT][ld]; TMA: [kWarps][NS][K, V][blocks][KT][64]
    bf16* q_s;                                           // [16][ld]   rotated queries (rows beyond the group: zeros)
    if (TMA) {
        tiles = reinterpret_cast<bf16*>(smem_raw);
        q_s = tiles + (size_t)kWarps * NS * kStageElems;
    } else {
        q_s = reinterpret_cast<bf16*>(smem_raw);
        tiles = q_s + 18 * ld;
    }
    bf16* kn_s = q_s + 16 * ld;                          // [ld]       the token's own key (rotated)
    bf16* vn_s = kn_s + ld;                              // [ld]       the token's own value
    float* mrg = reinterpret_cast<float*>(tiles);        // [kWarps][16][hd + 2], over the tiles once the keys are done
    float* cta_part = mrg + kWarps * 16 * (hd + 2);      // [16][hd + 2]: the CTA's own partial result (cluster form)
    __shared__ __align__(8) uint64_t full[kWarps][NS];   // TMA: a stage's boxes have landed
    __shared__ int last_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, lg = lane >> 2, lt = lane & 3, mi = lane >> 3;
    // `ti`: which of the call's tokens; `t`: its row in the step (the same unless the call lists its tokens)
    const size_t ti = blockIdx.x, t = a.token_list != nullptr ? (size_t)a.token_list[ti] : ti;
    const int kvh = blockIdx.y;
    const int G = a.Hq / a.Hkv, h0 = kvh * G;
    const int split = blockIdx.z;
    const int pos = a.positions[t];
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int n = pos - lo + 1;
    // a range is at least two tiles per warp: shorter ranges only add partial results to merge
    const int chunk = (max((n + a.splits - 1) / a.splits, 2 * kWarps * KT) + KT - 1) / KT * KT;
    const int used = (n + chunk - 1) / chunk;
    const bool idle = split >= used;                     // a range without keys
    if (idle && (!CL || used == 1)) return;              // in a cluster it still meets the others at the barriers
    const int begin = idle ? pos + 1 : lo + split * chunk;
    const int end = idle ? pos + 1 : min(begin + chunk, pos + 1);
    const bool use_new = a.write_kv != 0;
    const bool owns_new = use_new && begin <= pos && pos < end;
    const int* bt = a.block_table + (size_t)a.token_req[t] * a.bt_stride;
    const bf16* row = (const bf16*)a.qkv + t * a.row_stride;
    const float* cs = a.cos_sin + (size_t)min(max(pos, 0), a.table_rows - 1) * a.rotary_dim;
    const int pieces = hd / 8;

    bf16* my_tiles = TMA ? tiles + (size_t)warp * NS * kStageElems : tiles + (size_t)warp * NS * 2 * KT * ld;
    const bf16* kc = (const bf16*)a.k_cache;
    const bf16* vc = (const bf16*)a.v_cache;
    // TMA: the cache row at which the tile of key j0 starts (tiles never cross a page: pages are multiples of 32 keys,
    // ranges start at multiples of 32), and the request for its boxes by one lane.
    auto tile_row = [&](int j0) -> int {
        if (j0 >= end) return 0;
        const int page = j0 / a.page_size;
        return __ldg(bt + page) * a.page_size + (j0 - page * a.page_size);
    };
    auto fetch_tma = [&](int cache_row, int stage) {
        if (lane == 0) {
            bf16* kd = my_tiles + (size_t)stage * kStageElems;           // K blocks, then V blocks
            tc::mbar_expect_tx(&full[warp][stage], kStageElems * (int)sizeof(bf16));
#pragma unroll
            for (int blk = 0; blk < HDT / 4; ++blk) {
                tc::tma_load_2d(kd + blk * (KT * 64), &map_k, &full[warp][stage], kvh * hd + blk * 64, cache_row);
                tc::tma_load_2d(kd + kTileElems + blk * (KT * 64), &map_v, &full[warp][stage], kvh * hd + blk * 64, cache_row);
            }
        }
    };
    // cp.async: lane l looks up the cache row of key j0 + l once; the copies then run with consecutive lanes on
    // consecutive 16-byte pieces of the same row, so that one instruction covers whole 128-byte lines.
    // The block-table entry of a tile is read one iteration before its copies are issued, so that the warp
    // never waits on that load with tensor-core work behind it.
    auto lookup = [&](int j0) -> long long {
        const int j = j0 + lane;
        if (j >= end || (use_new && j == pos)) return -1;
        const int page = j / a.page_size;
        return (((long long)__ldg(bt + page) * a.page_size + (j - page * a.page_size)) * a.Hkv + kvh) * hd;
    };
    auto fetch = [&](long long off, int stage) {
        bf16* kd = my_tiles + (size_t)(stage * 2) * KT * ld;
        bf16* vd = kd + KT * ld;
        if (hd == HDT * 16) {                             // the usual case: shifts for the divisions, copies unrolled
            constexpr int kPieces = HDT * 2;
#pragma unroll
            for (int it = 0; it < KT * kPieces / 32; ++it) {
                const int i = it * 32 + lane, r = i / kPieces, c = i % kPieces;
                const long long roff = __shfl_sync(0xffffffffu, off, r);
                const bool valid = roff >= 0;
                cp_async16(kd + r * ld + c * 8, kc + (valid ? roff : 0) + c * 8, valid);
                cp_async16(vd + r * ld + c * 8, vc + (valid ? roff : 0) + c * 8, valid);
            }
        } else {
            for (int i = lane; i < KT * pieces; i += 32) {
                const int r = i / pieces, c = i - r * pieces;
                const long long roff = __shfl_sync(0xffffffffu, off, r);
                const bool valid = roff >= 0;
                cp_async16(kd + r * ld + c * 8, kc + (valid ? roff : 0) + c * 8, valid);
                cp_async16(vd + r * ld + c * 8, vc + (valid ? roff : 0) + c * 8, valid);
            }
        }
    };
    float o[HDT * 2][4];
#pragma unroll
    for (int i = 0; i < HDT * 2; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;     // rows lg and lg + 8 (query heads)
    const float scale_log2 = a.scale * 1.4426950408889634f;
    // NS - 1 tiles are on their way before the first one is used (and while the queries are prepared): a warp's
    // share of the memory system is what it keeps in flight, and a tile takes well over a microsecond to arrive
    const int first = begin + warp * KT;
    constexpr int kStride = kWarps * KT;
    long long off_next = -1;
    int row_next = 0;
    if (TMA) {
        if (lane == 0) {
#pragma unroll
            for (int p = 0; p < NS; ++p) tc::mbar_init(&full[warp][p], 1);
            tc::mbar_fence_init();
        }
        __syncwarp();
#pragma unroll
        for (int p = 0; p < NS - 1; ++p)
            if (first + p * kStride < end) fetch_tma(tile_row(first + p * kStride), p);
        row_next = tile_row(first + (NS - 1) * kStride);
    } else {
#pragma unroll
        for (int p = 0; p < NS - 1; ++p) {
            if (first + p * kStride < end) fetch(lookup(first + p * kStride), p);
            cp_async_commit();
        }
        off_next = lookup(first + (NS - 1) * kStride);
    }
    // Up to here only step tables and keys and values of earlier tokens were read: that may run under the tail of
    // the q|k|v projection before this kernel.  Its output is read from here on.
    pdl_wait();
    const int rotary = a.rotate ? a.rotary_dim : 0;      // queries that come rotated already are only copied
    const int half = a.rotary_dim >> 1;
    if ((half & 7) == 0 && (a.row_stride & 7) == 0 && ((uintptr_t)a.qkv & 15) == 0) {
        // eight columns per thread: the piece, its partner half a rotation away, cos and sin come as 16-byte loads
        // that are all in flight together (element by element this was a chain of 2- and 4-byte loads per column)
        for (int i = threadIdx.x; i < 16 * pieces; i += kThreads) {
            const int g = i / pieces, c0 = (i - g * pieces) * 8;
            uint4 packed = make_uint4(0u, 0u, 0u, 0u);
            if (g < G) {
                const bf16* src = row + (size_t)(h0 + g) * hd;
                packed = *reinterpret_cast<const uint4*>(src + c0);
                if (c0 < rotary) {
                    const bool low = c0 < half;
                    const int f0 = low ? c0 : c0 - half;
                    const uint4 other = *reinterpret_cast<const uint4*>(src + (low ? c0 + half : c0 - half));
                    const float4 cA = *reinterpret_cast<const float4*>(cs + f0), cB = *reinterpret_cast<const float4*>(cs + f0 + 4);
                    const float4 sA = *reinterpret_cast<const float4*>(cs + half + f0), sB = *reinterpret_cast<const float4*>(cs + half + f0 + 4);
                    const float cosv[8] = {cA.x, cA.y, cA.z, cA.w, cB.x, cB.y, cB.z, cB.w};
                    const float sinv[8] = {sA.x, sA.y, sA.z, sA.w, sB.x, sB.y, sB.z, sB.w};
                    const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&packed);
                    const __nv_bfloat162* yh = reinterpret_cast<const __nv_bfloat162*>(&other);
                    uint4 res;
                    unsigned* rw = reinterpret_cast<unsigned*>(&res);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 x = __bfloat1622float2(xh[e]), y = __bfloat1622float2(yh[e]);
                        const float v0 = x.x * cosv[2 * e] + (low ? -y.x : y.x) * sinv[2 * e];
                        const float v1 = x.y * cosv[2 * e + 1] + (low ? -y.y : y.y) * sinv[2 * e + 1];
                        rw[e] = pack_bf16(v0, v1);
                    }
                    packed = res;
                }
            }
            *reinterpret_cast<uint4*>(q_s + g * ld + c0) = packed;
        }
    } else {
        for (int i = threadIdx.x; i < 16 * hd; i += kThreads) {
            const int g = i / hd, c = i % hd;
            q_s[g * ld + c] = __float2bfloat16_rn(g < G ? rotated<bf16>(row + (size_t)(h0 + g) * hd, c, rotary, cs, 1.f, false) : 0.f);
        }
    }
    if (owns_new) {
        const bf16* ksrc = row + (size_t)(a.Hq + kvh) * hd;
        const bf16* vsrc = row + (size_t)(a.Hq + a.Hkv + kvh) * hd;
        const long slot = a.slot_mapping[t];
        for (int c = threadIdx.x; c < hd; c += kThreads) {
            const bf16 kv = __float2bfloat16_rn(rotated<bf16>(ksrc, c, a.rotary_dim, cs, a.key_scale, true));
            kn_s[c] = kv; vn_s[c] = vsrc[c];
            if (slot >= 0) {
                ((bf16*)a.k_cache)[((size_t)slot * a.Hkv + kvh) * hd + c] = kv;
                ((bf16*)a.v_cache)[((size_t)slot * a.Hkv + kvh) * hd + c] = vsrc[c];
            }
        }
    }
    __syncthreads();

    unsigned qa[HDT][4];                                 // the queries' fragments stay in registers
#pragma unroll
    for (int kk = 0; kk < HDT; ++kk)
        if (kk * 16 < hd) ldsm_x4(qa[kk], q_s + (lane & 15) * ld + kk * 16 + (lane >> 4) * 8);
    int stage = 0;
    unsigned phase = 0;                                  // TMA: parity of the stage ring's current round
    // swizzled tiles: 16-byte piece c of row r lies at piece c ^ (r & 7); the rows a lane addresses have r & 7 == lane & 7
    const int sw = lane & 7;
    for (int j0 = first; j0 < end; j0 += kStride) {
        const int ahead = j0 + (NS - 1) * kStride;
        bf16 *kb, *vb;
        if (TMA) {
            if (ahead < end) fetch_tma(row_next, (stage + NS - 1) % NS);       // into the stage that was used last iteration
            row_next = tile_row(ahead + kStride);
            const bool landed = tc::mbar_wait(&full[warp][stage], phase);
            if (!__all_sync(0xffffffffu, landed)) {       // the copy engine never answered: give up, the step is invalid
                if (lane == 0 && a.error != nullptr)
                    atomicCAS(a.error, 0, 0x31000000 | ((blockIdx.x & 0xFFF) << 12) | ((blockIdx.y & 0x3F) << 6) | (blockIdx.z & 0x3F));
                break;
            }
            kb = my_tiles + (size_t)stage * kStageElems;
            vb = kb + kTileElems;
            if (use_new && pos >= j0 && pos < j0 + KT) { // the token's own key and value take their row of the tile
                const int r = pos - j0;
                for (int c = lane; c < hd; c += 32) {
                    const int at = (c >> 6) * (KT * 64) + r * 64 + ((((c & 63) >> 3) ^ (r & 7)) << 3) + (c & 7);
                    kb[at] = kn_s[c]; vb[at] = vn_s[c];
                }
                __syncwarp();
            }
            if (j0 + KT > end) {                         // rows of the page beyond the last key hold anything: their values
                const int r0 = end - j0;                  // must not meet the zero weights as NaN or infinity
                for (int i = lane; i < (KT - r0) * (HDT * 2); i += 32) {
                    const int r = r0 + i / (HDT * 2), c = i % (HDT * 2);
                    *reinterpret_cast<uint4*>(vb + (c >> 3) * (KT * 64) + r * 64 + (c & 7) * 8) = make_uint4(0u, 0u, 0u, 0u);
                }
                __syncwarp();
            }
        } else {
            if (ahead < end) fetch(off_next, (stage + NS - 1) % NS);       // into the stage that was used last iteration
            cp_async_commit();
            off_next = lookup(ahead + kStride);
            cp_async_wait<NS - 1>();
            __syncwarp();
            kb = my_tiles + (size_t)(stage * 2) * KT * ld;
            vb = kb + KT * ld;
            if (use_new && pos >= j0 && pos < j0 + KT) { // the token's own key and value take their row of the tile
                for (int c = lane; c < hd; c += 32) { kb[(pos - j0) * ld + c] = kn_s[c]; vb[(pos - j0) * ld + c] = vn_s[c]; }
                __syncwarp();
            }
        }
        float s[KT / 8][4];
#pragma unroll
        for (int i = 0; i < KT / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HDT; ++kk) {
            if (kk * 16 < hd) {
#pragma unroll
                for (int n2 = 0; n2 < KT / 16; ++n2) {
                    unsigned kf[4];
                    if (TMA)
                        ldsm_x4(kf, kb + (kk >> 2) * (KT * 64) + (n2 * 16 + (mi >> 1) * 8 + (lane & 7)) * 64
                                        + ((((kk & 3) * 2 + (mi & 1)) ^ sw) << 3));
                    else
                        ldsm_x4(kf, kb + (n2 * 16 + (mi >> 1) * 8 + (lane & 7)) * ld + kk * 16 + (mi & 1) * 8);
                    mma_bf16(s[2 * n2], qa[kk], kf[0], kf[1]);
                    mma_bf16(s[2 * n2 + 1], qa[kk], kf[2], kf[3]);
                }
            }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
        if (j0 + KT > end) {                            // only a range's last tile has keys beyond its end
#pragma unroll
            for (int nn = 0; nn < KT / 8; ++nn)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (j0 + nn * 8 + 2 * lt + (e & 1) >= end) s[nn][e] = -INFINITY;
        }
#pragma unroll
        for (int nn = 0; nn < KT / 8; ++nn) {
            mx0 = fmaxf(mx0, fmaxf(s[nn][0], s[nn][1]));
            mx1 = fmaxf(mx1, fmaxf(s[nn][2], s[nn][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        mx0 = fmaxf(m0, mx0 * scale_log2);               // every tile of a warp holds at least one key: finite
        mx1 = fmaxf(m1, mx1 * scale_log2);
        // a row's sums are rescaled only when some row of the warp met a larger score (the weights lie in [0, 1]
        // and become bfloat16 operands next: the one-instruction 2^x is exact enough)
        const bool grew = __any_sync(0xffffffffu, mx0 > m0 || mx1 > m1);
        float sum0 = 0.f, sum1 = 0.f;
        unsigned pa[KT / 16][4];
#pragma unroll
        for (int nn = 0; nn < KT / 8; ++nn) {
            const float e0 = tc::ex2_approx(fmaf(s[nn][0], scale_log2, -mx0)), e1 = tc::ex2_approx(fmaf(s[nn][1], scale_log2, -mx0));
            const float e2 = tc::ex2_approx(fmaf(s[nn][2], scale_log2, -mx1)), e3 = tc::ex2_approx(fmaf(s[nn][3], scale_log2, -mx1));
            sum0 += e0 + e1; sum1 += e2 + e3;
            pa[nn >> 1][(nn & 1) * 2] = pack_bf16(e0, e1);
            pa[nn >> 1][(nn & 1) * 2 + 1] = pack_bf16(e2, e3);
        }
        if (grew) {
            const float alpha0 = tc::ex2_approx(m0 - mx0), alpha1 = tc::ex2_approx(m1 - mx1);
            m0 = mx0; m1 = mx1;
            l0 *= alpha0; l1 *= alpha1;
#pragma unroll
            for (int i = 0; i < HDT * 2; ++i) { o[i][0] *= alpha0; o[i][1] *= alpha0; o[i][2] *= alpha1; o[i][3] *= alpha1; }
        }
        l0 += sum0;
        l1 += sum1;
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
#pragma unroll
            for (int d2 = 0; d2 < HDT; ++d2) {
                if (d2 * 16 < hd) {
                    unsigned vf[4];
                    if (TMA)
                        ldsm_x4_t(vf, vb + (d2 >> 2) * (KT * 64) + (kk * 16 + (mi & 1) * 8 + (lane & 7)) * 64
                                          + ((((d2 & 3) * 2 + (mi >> 1)) ^ sw) << 3));
                    else
                        ldsm_x4_t(vf, vb + (kk * 16 + (mi & 1) * 8 + (lane & 7)) * ld + d2 * 16 + (mi >> 1) * 8);
                    mma_bf16(o[2 * d2], pa[kk], vf[0], vf[1]);
                    mma_bf16(o[2 * d2 + 1], pa[kk], vf[2], vf[3]);
                }
            }
        }
        __syncwarp();
        if (++stage == NS) { stage = 0; phase ^= 1u; }
    }
    pdl_trigger();                                       // the output projection may fetch its weights under the merge
    cp_async_wait<0>();
    __syncthreads();                                     // every warp is done with its tiles: the partial results go there
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    // per warp: rows (query heads) x columns -> shared memory, in natural-exponent units for the merge
    const int stride = hd + 2;
    const float ln2 = 0.6931471805599453f;
#pragma unroll
    for (int i = 0; i < HDT * 2; ++i) {
        const int d = i * 8 + 2 * lt;
        if (d < hd) {
            mrg[(warp * 16 + lg) * stride + d] = o[i][0]; mrg[(warp * 16 + lg) * stride + d + 1] = o[i][1];
            mrg[(warp * 16 + lg + 8) * stride + d] = o[i][2]; mrg[(warp * 16 + lg + 8) * stride + d + 1] = o[i][3];
        }
    }
    if (lt == 0) {
        mrg[(warp * 16 + lg) * stride + hd] = m0 * ln2; mrg[(warp * 16 + lg) * stride + hd + 1] = l0;
        mrg[(warp * 16 + lg + 8) * stride + hd] = m1 * ln2; mrg[(warp * 16 + lg + 8) * stride + hd + 1] = l1;
    }
    __syncthreads();
    const size_t group = ti * (size_t)a.Hkv + kvh;
    for (int i = threadIdx.x; i < G * hd; i += kThreads) {
        const int g = i / hd, d = i % hd;
        float mt = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mt = fmaxf(mt, mrg[(w * 16 + g) * stride + hd]);
        float lsum = 0.f, osum = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float mw = mrg[(w * 16 + g) * stride + hd];
            const float f = mw == -INFINITY ? 0.f : expf(mw - mt);
            lsum += mrg[(w * 16 + g) * stride + hd + 1] * f;
            osum += mrg[(w * 16 + g) * stride + d] * f;
        }
        const int h = h0 + g;
        if (used == 1) {
            ((bf16*)a.out)[(t * a.Hq + h) * hd + d] = __float2bfloat16_rn(osum / lsum);
        } else if (CL) {
            cta_part[g * stride + d] = osum;
            if (d == 0) { cta_part[g * stride + hd] = mt; cta_part[g * stride + hd + 1] = lsum; }
        } else {
            const size_t slot = ((size_t)ti * a.Hq + h) * a.splits + split;
            a.part_o[slot * hd + d] = osum;
            if (d == 0) { a.part_ml[slot * 2] = mt; a.part_ml[slot * 2 + 1] = lsum; }
        }
    }
    if (used == 1) return;
    if (CL) {
        cluster_barrier();                                // every range's partial result stands in its CTA's shared memory
        // Every CTA of the cluster merges a contiguous share of the G * hd outputs, one output per thread, and
        // asks for all ranges' values at once: the loads from the other CTAs' shared memory take hundreds of
        // cycles each, so one CTA walking the ranges one after the other was a quarter of the kernel's time.
        {
            const int n_out = G * hd, per = (n_out + a.splits - 1) / a.splits;
            for (int i = split * per + threadIdx.x; i < min(n_out, (split + 1) * per); i += kThreads) {
                const int g = i / hd, d = i % hd;
                float mv[8], lv[8], ov[8];
#pragma unroll
                for (int s2 = 0; s2 < 8; ++s2) {
                    const bool on = s2 < used;
                    mv[s2] = on ? ld_cluster(cluster_map(cta_part + g * stride + hd, s2)) : -INFINITY;
                    lv[s2] = on ? ld_cluster(cluster_map(cta_part + g * stride + hd + 1, s2)) : 0.f;
                    ov[s2] = on ? ld_cluster(cluster_map(cta_part + g * stride + d, s2)) : 0.f;
                }
                float mt = -INFINITY;
#pragma unroll
                for (int s2 = 0; s2 < 8; ++s2) mt = fmaxf(mt, mv[s2]);
                float lsum = 0.f, osum = 0.f;
#pragma unroll
                for (int s2 = 0; s2 < 8; ++s2) {
                    const float f = s2 < used ? expf(mv[s2] - mt) : 0.f;
                    lsum += lv[s2] * f;
                    osum += ov[s2] * f;
                }
                ((bf16*)a.out)[(t * a.Hq + h0 + g) * hd + d] = __float2bfloat16_rn(osum / lsum);
            }
        }
        cluster_barrier();                                // nobody leaves while its shared memory may still be read
        return;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int done = atomicAdd(a.counters + group, 1);
        last_flag = done == used - 1;
        if (last_flag) a.counters[group] = 0;
    }
    __syncthreads();
    if (!last_flag) return;
    __threadfence();
    for (int i = threadIdx.x; i < G * hd; i += kThreads) {
        const int g = i / hd, d = i % hd;
        const size_t base = ((size_t)ti * a.Hq + h0 + g) * a.splits;
        float mt = -INFINITY;
        for (int s2 = 0; s2 < used; ++s2) mt = fmaxf(mt, __ldcg(a.part_ml + (base + s2) * 2));
        float lsum = 0.f, osum = 0.f;
        for (int s2 = 0; s2 < used; ++s2) {
            const float f = expf(__ldcg(a.part_ml + (base + s2) * 2) - mt);
            lsum += __ldcg(a.part_ml + (base + s2) * 2 + 1) * f;
            osum += __ldcg(a.part_o + (base + s2) * hd + d) * f;
        }
        ((bf16*)a.out)[(t * a.Hq + h0 + g) * hd + d] = __float2bfloat16_rn(osum / lsum);
    }
}

template <int HDT, int NS, bool TMA, int KT>
int launch_mma_form(const FusedArgs& a, int tokens, cudaStream_t s, const CUtensorMap& map_k, const CUtensorMap& map_v) {
    const int ld = a.hd + 8;
    // the per-warp partial results (kWarps * 16 * (hd + 2) floats) lie over the tiles, which are larger
    const size_t smem = TMA ? 1024 + (size_t)kWarps * NS * 2 * KT * HDT * 16 * sizeof(bf16) + (size_t)18 * ld * sizeof(bf16)
                            : (size_t)(16 + 2 + kWarps * NS * 2 * kKT) * ld * sizeof(bf16);
    if (a.splits >= 2 && a.splits <= 8) {
        // the ranges of one (token, head) as one cluster along z
        static size_t have = 0;
        ensure_dynamic_smem(attn_decode_mma_kernel<HDT, NS, true, TMA, KT>, smem, have);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(tokens, a.Hkv, a.splits); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = smem; cfg.stream = s;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = (unsigned)a.splits;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = tokens <= kPdlMaxRows ? 2 : 1;
        return (int)cudaLaunchKernelEx(&cfg, attn_decode_mma_kernel<HDT, NS, true, TMA, KT>, a, map_k, map_v);
    }
    static size_t have_plain = 0;
    ensure_dynamic_smem(attn_decode_mma_kernel<HDT, NS, false, TMA, KT>, smem, have_plain);
    return launch_pdl_if(tokens <= kPdlMaxRows, attn_decode_mma_kernel<HDT, NS, false, TMA, KT>, dim3(tokens, a.Hkv, a.splits),
                         dim3(kThreads), smem, s, a, map_k, map_v);
}

// The tile-copy form where the sizes allow it (head_dim 64 or 128, pages of a multiple of 32 tokens, no window, caches
// on 16-byte boundaries), else the cp.async form.  `pages`: pages of the caches (the tensor maps' extent).
template <int HDT, int NS, int KT>
int launch_mma_tiles(const FusedArgs& a, int tokens, long pages, cudaStream_t s) {
    CUtensorMap map_k = {}, map_v = {};
    const bool tma = a.hd == HDT * 16 && (a.hd == 64 || a.hd == 128) && a.page_size % KT == 0 && a.window <= 0 && pages > 0 &&
                     ((((uintptr_t)a.k_cache) | ((uintptr_t)a.v_cache)) & 15) == 0;
    if (tma) {
        int rc = tc::make_tile_map(&map_k, a.k_cache, pages * a.page_size, (long)a.Hkv * a.hd, (long)a.Hkv * a.hd, KT);
        if (rc == 0) rc = tc::make_tile_map(&map_v, a.v_cache, pages * a.page_size, (long)a.Hkv * a.hd, (long)a.Hkv * a.hd, KT);
        if (rc != 0) return rc;
        return launch_mma_form<HDT, NS, true, KT>(a, tokens, s, map_k, map_v);
    }
    return launch_mma_form<HDT, NS, false, kKT>(a, tokens, s, map_k, map_v);
}

// The tile-copy form where the sizes allow it (head_dim 64 or 128, pages of a multiple of the tile, no window, caches
// on 16-byte boundaries), else the cp.async form.  `pages`: pages of the caches (the tensor maps' extent).
// Heads of 128 take 16-key tiles up to 32 tokens, where the kernel is bound by the chains of its few warps and two
// CTAs per SM help (24 tokens of 2,048 keys: 27 -> 17 us); with more tokens it runs beside the state update and is
// bound by the memory both share, and the 32-key form leaves that kernel more room (a 7B-size step of 64 tokens:
// 2.08 against 2.17 ms).
template <int HDT, int NS>
int launch_mma(const FusedArgs& a, int tokens, long pages, cudaStream_t s) {
    if (HDT == 8 && tokens <= 32) return launch_mma_tiles<HDT, NS, 16>(a, tokens, pages, s);
    return launch_mma_tiles<HDT, NS, kKT>(a, tokens, pages, s);
}

template <typename T>
int launch(FusedArgs a, int tokens, cudaStream_t s) {
    const int G = a.Hq / a.Hkv;
    const int gt = G >= 8 ? 8 : (G > 2 ? 4 : (G == 2 ? 2 : 1));
    a.head_tiles = (G + gt - 1) / gt;
    switch (gt) {
        case 1: return launch_chp<T, 1>(a, tokens, s);
        case 2: return launch_chp<T, 2>(a, tokens, s);
        case 4: return launch_chp<T, 4>(a, tokens, s);
        default: return launch_chp<T, 8>(a, tokens, s);
    }
}
}  // namespace

// Number of counters the call needs: tokens * Hkv * head tiles (head tiles = ceil((Hq / Hkv) / heads per CTA)).
extern "C" int lb_attention_decode_fused_counters(int tokens, int Hq, int Hkv) {
    if (tokens <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return 0;
    const int G = Hq / Hkv;
    const int gt = G >= 8 ? 8 : (G > 2 ? 4 : (G == 2 ? 2 : 1));
    return tokens * Hkv * ((G + gt - 1) / gt);
}

// qkv: [tokens, (Hq + 2 Hkv) * hd] rows (row stride in elements); every token is the only new token of its
// request; `counters`: zero-initialised int32, at least lb_attention_decode_fused_counters(...) entries, left
// at zero by the call; part_o / part_ml as for lb_attention_decode (may be null when splits == 1).
extern "C" int lb_attention_decode_fused(const void* qkv, long row_stride, void* k_cache, void* v_cache, void* out,
                                         const int* block_table, int bt_stride, const int* token_req,
                                         const int* positions, const int* slot_mapping, const float* cos_sin,
                                         int table_rows, int rotary_dim, int tokens, int Hq, int Hkv, int hd,
                                         int page_size, float scale, float key_scale, int window, int write_kv,
                                         int splits, float* part_o, float* part_ml, int* counters, long pages,
                                         int* error, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (hd <= 0 || hd > 256 || hd % 16 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || page_size <= 0 || splits < 1) return kBadSize;
    if (rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1)) return kBadSize;
    if (splits > 1 && (part_o == nullptr || part_ml == nullptr || counters == nullptr)) return kBadSize;
    if (splits > 65535 || (long)Hkv * ((Hq / Hkv + 7) / 8 + 1) > 65535) return kTooLarge;
    FusedArgs a{qkv, row_stride, k_cache, v_cache, out, block_table, bt_stride, token_req, positions, slot_mapping,
                cos_sin, table_rows, rotary_dim, part_o, part_ml, counters, Hq, Hkv, hd, page_size, window, splits, 1,
                write_kv, scale, key_scale, nullptr, 1, error};
    if (dtype == kBF16 && hd <= 128 && Hq / Hkv <= 16)
    {
        // Stages of a warp's tile ring: 3 for a grid of up to 96 CTAs (two tiles on their way before the first is used:
        // a lone request), 2 beyond, which keeps three CTAs per SM instead of two.  Measured on 36-layer decode steps
        // with the tile-copy form at batch 8 / 64: 1.262 / 2.552 ms with 2 stages, 1.283 / 2.606 ms with 3 (batch 1,
        // 64 CTAs: no difference).
        const bool small = (long)tokens * Hkv * splits <= 96;
        cudaStream_t st = (cudaStream_t)stream;
        if (hd <= 64) return small ? launch_mma<4, 3>(a, tokens, pages, st) : launch_mma<4, 2>(a, tokens, pages, st);
        return small ? launch_mma<8, 3>(a, tokens, pages, st) : launch_mma<8, 2>(a, tokens, pages, st);
    }
    LB_DISPATCH_DTYPE(dtype, return launch<T>(a, tokens, (cudaStream_t)stream));
    return kOk;
}

// Does lb_attention_decode_listed take these sizes (the tensor-core form of the kernel above)?
extern "C" int lb_attention_decode_listed_ok(int Hq, int Hkv, int hd, int dtype) {
    return dtype == kBF16 && hd > 0 && hd <= 128 && hd % 16 == 0 && Hkv > 0 && Hq % Hkv == 0 && Hq / Hkv <= 16 ? 1 : 0;
}

// The same attention for some tokens of a step that holds prompt portions as well: `token_list` names the `count` step
// rows to run (each the newest token of its request: single decoded tokens, or the tokens of a short portion one by
// one), `q` [rows, Hq, hd] holds the queries already rotated, and every key and value, the tokens' own included, is
// already in the cache (the rotate-and-store kernel ran before).  Rows of `out` [rows, Hq, hd] that are not listed
// are left as they are.  bfloat16, hd <= 128, group <= 16 (lb_attention_decode_listed_ok).
extern "C" int lb_attention_decode_listed(const void* q, void* k_cache, void* v_cache, void* out, const int* block_table,
                                          int bt_stride, const int* token_req, const int* positions, const int* token_list,
                                          int count, int Hq, int Hkv, int hd, int page_size, float scale, int window,
                                          int splits, float* part_o, float* part_ml, int* counters, long pages,
                                          int* error, void* stream) {
    if (count <= 0) return kOk;
    if (!lb_attention_decode_listed_ok(Hq, Hkv, hd, kBF16) || page_size <= 0 || splits < 1 || token_list == nullptr) return kBadSize;
    if (splits > 1 && (part_o == nullptr || part_ml == nullptr || counters == nullptr)) return kBadSize;
    if (splits > 65535 || Hkv > 65535) return kTooLarge;
    FusedArgs a{q, (long)Hq * hd, k_cache, v_cache, out, block_table, bt_stride, token_req, positions, nullptr,
                nullptr, 1, 0, part_o, part_ml, counters, Hq, Hkv, hd, page_size, window, splits, 1,
                0, scale, 1.f, token_list, 0, error};
    const bool small = (long)count * Hkv * splits <= 96;
    cudaStream_t st = (cudaStream_t)stream;
    if (hd <= 64) return small ? launch_mma<4, 3>(a, count, pages, st) : launch_mma<4, 2>(a, count, pages, st);
    return small ? launch_mma<8, 3>(a, count, pages, st) : launch_mma<8, 2>(a, count, pages, st);
}
