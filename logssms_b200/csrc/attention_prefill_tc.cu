// Causal grouped-query attention for prompt portions over the paged cache on the 5th-generation tensor cores
// (tcgen05, accumulators in tensor memory, operands brought by TMA).  bfloat16, head size 64 or 128, pages of a
// multiple of 64 tokens; every other shape stays on the mma.sync kernel (attention_prefill.cu).  The description
// below gives the numbers for heads of 64; with heads of 128 a tile is two blocks of 64 dims side by side, S takes
// 8 products, PV 4 per block of output dims, O has 128 columns and the ring 6 stages.
//
// One CTA per (128 query tokens of one request's portion, query head), 11 warps:
//   warp 0     one thread: TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of the Q tile once, then of the
//              K and V tiles (64 keys each: one box per tile, since a tile never crosses a page) into a ring of 8
//              stages, each with a "full" and an "empty" mbarrier; the page of a tile comes from the block table
//   warp 1     allocates the tensor memory; one thread issues the first softmax group's products,
//   warp 2     one thread those of the second group:
//                  S  = Q K^T    (M 128 queries, N 64 keys, K 64 dims: 4 x tcgen05.mma, both operands K-major), into
//                                one of the group's two S buffers in turn
//                  O += P V      (M 128, N 64 dims, K 64 keys: 4 x tcgen05.mma, P from tensor memory, V as an MN-major operand: the rows of
//                                the cache are keys, which is the K dimension of this product); O stays in tensor
//                                memory for the whole CTA
//              S of a group's first two tiles is issued up front, S of tile t + 2 right behind PV of tile t, so a
//              row never waits for its next S
//   warps 3-10 two groups of 128 threads, one thread per query row in each; group g owns the key tiles g, g + 2, ...
//              with its own S / P buffers, O and running (maximum, sum), so that one group's chain of
//              product -> softmax -> product runs while the other's is in another phase; the two partial results
//              meet in shared memory at the end.  A thread: read the row of S from tensor memory (tcgen05.ld), mask
//              by absolute position (causal, optional window; tiles that need no mask take a loop without it),
//              softmax weights in float32 relative to a maximum that follows the row's true maximum lazily (O is
//              fetched, scaled and put back only when the maximum has grown by more than 2^8; exact, since O and
//              the row sum carry the same factor), P rounded to bfloat16 and stored into tensor memory over the S
//              it was made from (tcgen05.st): PV takes it from there as its A operand, without a round trip through
//              shared memory
// Keys of the last tile beyond the newest token are rows of the page that nobody has written for this request:
// their scores are masked by selection, and their V rows are overwritten with zeros in shared memory before PV
// (0 x stale-NaN would poison the row).
//
// Every wait on an mbarrier is bounded: after about a second of polling the thread records where it gave up in
// `error`, all roles stop, tensor memory is freed and the kernel returns.
//
// Formula: python/logssms/layers/attention_backend/fi.py:175-190 (causal, scale head_dim^-1/2); chunked prompts:
// the query at absolute position p sees keys 0..p.
#include "lb200/common.cuh"
#include "lb200/tcgen05.cuh"
using namespace lb200;
using namespace lb200::tc;

namespace {
typedef __nv_bfloat16 bf16;
constexpr int kQ = 128, kKV = 64;                         // queries per CTA, keys per tile
constexpr int kGroups = 2;                                // softmax groups of 128 threads
constexpr int kFirstSoftmaxWarp = 1 + kGroups;            // warp 0: TMA; warps 1..kGroups: one issuing thread per group
constexpr int kThreads = 32 * (kFirstSoftmaxWarp + 4 * kGroups);
constexpr uint32_t kTmemCols = 512;
constexpr float kTau = 8.f;                               // log2 of the growth of a row's maximum that O is rescaled for
// Per head size (64 or 128).  A tile of shared memory is made of blocks of 64 dims (rows of 128 bytes, the width
// of the 128-byte swizzle): one block for heads of 64, two side by side for heads of 128.
template <int HD> struct Shape {
    static constexpr int kBlocks = HD / 64;
    // K|V tiles in shared memory: each group has three in use, the rest are on their way (6 x 32 KB + Q fill the SM at 128)
    static constexpr int kStages = HD == 64 ? 8 : 6;
    static constexpr uint32_t kQBlock = kQ * 128, kKVBlock = kKV * 128;          // bytes of one block of Q, of K or V
    static constexpr uint32_t kQBytes = kQBlock * kBlocks, kTileBytes = kKVBlock * kBlocks;
    static constexpr uint32_t kGroupCols = 128 + HD;      // per group: S (then P) of even tiles 0..63, of odd tiles 64..127, O from 128
    static constexpr uint32_t kMergeBytes = (64 + 2) * kQ * 4;   // a group's partial result for 64 dims, [column][row] float32
    static_assert(kGroups * kGroupCols <= kTmemCols, "tensor memory");
    static_assert((kGroups - 1) * kMergeBytes <= kStages * 2 * kTileBytes, "the partial results lie over the K|V ring");
};

struct TcArgs {
    bf16* out;                                            // [tokens, Hq, 64]
    const int* block_table; int bt_stride;
    const int* cu_seqlens; const int* start_pos;
    const int* tiles;                                     // [n_tiles][2]: request index, first token of the tile in its portion
    int Hq, Hkv, page_size, window;
    float scale_log2;
    int n_items;                                          // tiles * query heads
    int* error;
    // With `splits` > 1 the keys of a tile are cut into that many ranges, each a CTA of its own (a step of few
    // query tiles over a long context would otherwise leave most SMs idle): a CTA then leaves its rows unnormalised
    // in `part_o` [item][split][128][hd] with (maximum in log2 units, sum) in `part_ml` [item][split][128][2], and
    // attn_prefill_merge_kernel puts the ranges together.
    int splits; float* part_o; float* part_ml;
};

__device__ __forceinline__ void report(int* error, int role, int tile) {
    if (error != nullptr) atomicCAS(error, 0, (role << 24) | ((blockIdx.x & 0xFFF) << 12) | (tile & 0xFFF) | 0x40000000);
}

template <int HD>
__global__ void __launch_bounds__(kThreads)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, TcArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    typedef Shape<HD> Sh;
    constexpr int kHD = HD, kStages = Sh::kStages, kBlocks = Sh::kBlocks;
    constexpr uint32_t kQBytes = Sh::kQBytes, kTileBytes = Sh::kTileBytes, kGroupCols = Sh::kGroupCols;
    uint8_t* q_s = base;                                  // blocks of [128][128 B]
    uint8_t* kv_s = q_s + kQBytes;                        // stages of K (blocks of [64][128 B]) | V (the same)
    float* merge = reinterpret_cast<float*>(kv_s);        // at the end, over the ring: per group beyond the first [66][128]
    uint64_t* kv_full = reinterpret_cast<uint64_t*>(kv_s + kStages * 2 * kTileBytes);
    uint64_t* kv_empty = kv_full + kStages;
    uint64_t* q_full = kv_empty + kStages;
    uint64_t* s_ready = q_full + 1;                       // per group and tile parity: S of the tile is in tensor memory
    // per group and tile parity: P of the tile is in tensor memory (128 arrivals).  Two barriers per group, because a
    // warp may be a tile ahead of its neighbours (S of the next tile is ready early, and only some warps take the
    // detour that rescales O): with one barrier its arrival for tile t + 1 would count towards tile t, and the
    // product would start before a slower warp had stored its rows of P.  Nobody can be two tiles ahead: S of tile
    // t + 2 is issued behind the product of tile t.
    uint64_t* p_ready = s_ready + 2 * kGroups;
    uint64_t* o_ready = p_ready + 2 * kGroups;            // per group and tile parity: PV of the tile is added to O
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_ready + 2 * kGroups);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // heaviest tiles first (the host lists them so); the query heads of a tile follow one another
    const int item = blockIdx.x / a.splits, split = blockIdx.x % a.splits;
    const int tile = item / a.Hq, h = item % a.Hq, kvh = h / (a.Hq / a.Hkv);
    const int b = a.tiles[2 * tile], q0 = a.tiles[2 * tile + 1];
    if (b < 0) return;                                  // a list entry without work: the lists of a step that was filled up to fixed sizes end in such entries
    const int begin = a.cu_seqlens[b], len = a.cu_seqlens[b + 1] - begin;
    const int rows = min(kQ, len - q0);
    const int pos0 = a.start_pos[b] + q0, last_pos = pos0 + rows - 1;
    const int lo = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    int kt_begin = lo / kKV, kt_end = last_pos / kKV + 1;
    if (a.splits > 1) {                                   // this CTA's share of the key tiles
        const int per = (kt_end - kt_begin + a.splits - 1) / a.splits;
        kt_begin += split * per;
        kt_end = min(kt_end, kt_begin + per);
        if (kt_begin >= kt_end) {                         // a range without keys: the merge skips it
            if (threadIdx.x < kQ) {
                float* ml = a.part_ml + (((size_t)item * a.splits + split) * kQ + threadIdx.x) * 2;
                ml[0] = -INFINITY; ml[1] = 0.f;
            }
            return;
        }
    }
    const int n_kt = kt_end - kt_begin;
    const int* bt = a.block_table + (size_t)b * a.bt_stride;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(kv_full + s, 1); mbar_init(kv_empty + s, 1); }
        mbar_init(q_full, 1);
        for (int g = 0; g < kGroups; ++g) {
            mbar_init(s_ready + 2 * g, 1); mbar_init(s_ready + 2 * g + 1, 1);
            mbar_init(o_ready + 2 * g, 1); mbar_init(o_ready + 2 * g + 1, 1);
            mbar_init(p_ready + 2 * g, 128); mbar_init(p_ready + 2 * g + 1, 128);
        }
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
            mbar_expect_tx(q_full, kQBytes);
#pragma unroll
            for (int blk = 0; blk < kBlocks; ++blk) tma_load_2d(q_s + blk * Sh::kQBlock, &map_q, q_full, h * kHD + blk * 64, begin + q0);
            int issued = 0;
            for (int i = 0; i < n_kt && !*failed; ++i, ++issued) {
                const int s = i % kStages;
                if (i >= kStages && !mbar_wait(kv_empty + s, ((i / kStages) - 1) & 1)) { report(a.error, 1, i); *failed = 1; break; }
                const int j0 = (kt_begin + i) * kKV;
                const int page = j0 / a.page_size;
                const int row = bt[page] * a.page_size + (j0 - page * a.page_size);
                uint8_t* k_tile = kv_s + (size_t)s * 2 * kTileBytes;
                mbar_expect_tx(kv_full + s, 2 * kTileBytes);
#pragma unroll
                for (int blk = 0; blk < kBlocks; ++blk) {
                    tma_load_2d(k_tile + blk * Sh::kKVBlock, &map_k, kv_full + s, kvh * kHD + blk * 64, row);
                    tma_load_2d(k_tile + kTileBytes + blk * Sh::kKVBlock, &map_v, kv_full + s, kvh * kHD + blk * 64, row);
                }
            }
            if (*failed) {                                 // let the copies already under way land before the CTA leaves
                mbar_wait(q_full, 0);
                for (int i = max(0, issued - kStages); i < issued; ++i) mbar_wait(kv_full + i % kStages, (i / kStages) & 1);
            }
        }
    } else if (warp < kFirstSoftmaxWarp) {
        if (lane == 0) {
            // One issuing thread per softmax group (its tiles g, g + kGroups, ...): a thread that served all of them
            // would wait for one group's P while another's is ready.
            const int g = warp - 1;
            // float32 accumulator, bfloat16 operands, N 64, M 128; the B operand of PV is MN-major (V)
            const uint32_t idesc_s = umma_idesc(kQ, kKV);
            const uint32_t idesc_o = idesc_s | kBMnMajor;
            uint64_t qdesc[kBlocks];
#pragma unroll
            for (int blk = 0; blk < kBlocks; ++blk) qdesc[blk] = umma_desc(q_s + blk * Sh::kQBlock);
            bool ok = mbar_wait(q_full, 0);
            if (!ok) { report(a.error, 2, 0xFFF); *failed = 1; }
            auto issue_s = [&](int i, int t) -> bool {     // S of tile i, the group's tile number t, into its S buffer t & 1
                const int s = i % kStages;
                if (!mbar_wait(kv_full + s, (i / kStages) & 1)) { report(a.error, 2, i); *failed = 1; return false; }
                fence_after_sync();
#pragma unroll
                for (int blk = 0; blk < kBlocks; ++blk) {
                    const uint64_t kdesc = umma_desc(kv_s + (size_t)s * 2 * kTileBytes + blk * Sh::kKVBlock);
#pragma unroll
                    for (int k = 0; k < 4; ++k)            // 16 dims per product, 64 per block
                        umma_bf16(tmem + g * kGroupCols + (t & 1) * 64, qdesc[blk] + 2 * k, kdesc + 2 * k, idesc_s, (blk | k) != 0);
                }
                umma_commit(s_ready + 2 * g + (t & 1));
                return true;
            };
            // S of the group's first two tiles is on its way before any softmax starts; from then on S of tile t + 2
            // follows PV of tile t (whose P the rows wrote after they had read S of tile t out of that buffer), so a
            // row never waits for the tensor core to start on its next S
            if (ok && g < n_kt) ok = issue_s(g, 0);
            if (ok && g + kGroups < n_kt) ok = issue_s(g + kGroups, 1);
            for (int i = g, t = 0; i < n_kt && ok && !*failed; i += kGroups, ++t) {
                const int s = i % kStages;
                // P of tile i is written (and O rescaled where a row's maximum grew): O += P V
                if (!mbar_wait(p_ready + 2 * g + (t & 1), (t >> 1) & 1)) { report(a.error, 3, i); *failed = 1; break; }
                fence_after_sync();
                const uint32_t p_tmem = tmem + g * kGroupCols + (t & 1) * 64;     // P lies over the S it was made from
#pragma unroll
                for (int blk = 0; blk < kBlocks; ++blk) {  // 64 dims of O per block of V
                    const uint64_t vdesc = umma_desc(kv_s + (size_t)s * 2 * kTileBytes + kTileBytes + blk * Sh::kKVBlock);
#pragma unroll
                    for (int k = 0; k < kKV / 16; ++k)     // 16 keys: 8 columns of P (two bfloat16 each), two 8-row groups of V = 2048 bytes
                        umma_bf16_tmem_a(tmem + g * kGroupCols + 128 + blk * 64, p_tmem + 8 * k, vdesc + (uint64_t)(2048 >> 4) * k, idesc_o,
                                         (t > 0 || k != 0) ? 1u : 0u);
                }
                umma_commit(o_ready + 2 * g + (t & 1));
                umma_commit(kv_empty + s);                 // both products have read the stage
                if (i + 2 * kGroups < n_kt) ok = issue_s(i + 2 * kGroups, t + 2);
            }
        }
    } else {
        const int grp = (warp - kFirstSoftmaxWarp) / 4;    // which tiles: grp, grp + kGroups, ...
        const int r = (warp & 3) * 32 + lane;              // the row of the tile this thread owns (its lane of tensor memory)
        const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + grp * kGroupCols;
        const int p = pos0 + r;                            // absolute position of the row's query
        const int lo_r = a.window > 0 ? p - a.window + 1 : 0;
        // The output row O stays in tensor memory, where the PV products add to it.  It and the row sum l are kept
        // relative to m_used, a maximum that follows the true one lazily: only when the row's maximum has grown by
        // more than 2^kTau does the thread fetch O, scale it and put it back (with random scores after a handful of
        // tiles never again); until then P = 2^(s - m_used) may exceed 1, by at most 2^kTau.  The result is the same:
        // O and l carry the same factor, and it cancels in O / l.
        float m_used = -INFINITY, l = 0.f;
        uint64_t* o_bar = o_ready + 2 * grp;
        bool ok = true;
        int done = 0;                                      // tiles of this group whose P has been handed over
        auto wait_pv = [&](int t_of, int code, int tile) -> bool {      // PV of the group's tile number t_of is in O
            bool good = mbar_wait(o_bar + (t_of & 1), (t_of >> 1) & 1);
            if (!good && lane == 0) { report(a.error, code, tile); *failed = 1; }
            return __all_sync(0xffffffffu, good && !*failed);
        };
        for (int i = grp, t = 0; i < n_kt; i += kGroups, ++t) {
            const int j0 = (kt_begin + i) * kKV;
            ok = mbar_wait(s_ready + 2 * grp + (t & 1), (t >> 1) & 1);
            if (!ok && lane == 0) { report(a.error, 5, i); *failed = 1; }
            if (!__all_sync(0xffffffffu, ok && !*failed)) { ok = false; break; }
            fence_after_sync();
            // keys of this tile beyond the newest token: zero their V rows (the rows share the work)
            if (j0 + kKV - 1 > last_pos) {
                uint8_t* v_tile = kv_s + (size_t)(i % kStages) * 2 * kTileBytes + kTileBytes;
                const int first_bad = last_pos + 1 - j0;   // >= 1: the tile holds at least one key
                for (int x = r; x < (kKV - first_bad) * 8 * kBlocks; x += 128) {
                    const int blk = x / ((kKV - first_bad) * 8), y = x - blk * (kKV - first_bad) * 8;
                    *reinterpret_cast<uint4*>(v_tile + blk * Sh::kKVBlock + (size_t)(first_bad + y / 8) * 128 + (y % 8) * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            const bool whole = j0 + kKV - 1 <= pos0 && (a.window <= 0 || j0 >= pos0 + kQ - a.window);
            uint32_t pk[32];                               // the row of P, two bfloat16 per word
            {
                uint32_t s0[32], s1[32];
                tmem_ld32(lane_addr + (t & 1) * 64, s0);
                tmem_ld32(lane_addr + (t & 1) * 64 + 32, s1);
                float mx = -INFINITY;
                if (whole) {                               // no key of the tile is masked for any row: the common case
#pragma unroll
                    for (int c = 0; c < 32; ++c) mx = fmaxf(mx, fmaxf(__uint_as_float(s0[c]), __uint_as_float(s1[c])));
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        float v0 = __uint_as_float(s0[c]), v1 = __uint_as_float(s1[c]);
                        const int ka = j0 + c, kb = j0 + 32 + c;
                        if (ka > p || ka < lo_r) v0 = -INFINITY;
                        if (kb > p || kb < lo_r) v1 = -INFINITY;
                        s0[c] = __float_as_uint(v0); s1[c] = __float_as_uint(v1);
                        mx = fmaxf(mx, fmaxf(v0, v1));
                    }
                }
                mx *= a.scale_log2;
                const bool grow = mx > m_used + kTau;      // also the first key a row sees (m_used = -inf)
                float factor = 1.f;
                if (grow) { factor = exp2f(m_used - mx); m_used = mx; l *= factor; }
                if (t > 0 && __any_sync(0xffffffffu, grow)) {
                    // O <- O * factor for the rows of this warp whose maximum grew (factor 1 for the others); the
                    // product of the tile before must have landed in O first
                    if (!wait_pv(t - 1, 6, i)) { ok = false; break; }
                    fence_after_sync();
#pragma unroll
                    for (int piece = 0; piece < kHD / 32; ++piece) {
                        uint32_t ov[32];
                        tmem_ld32(lane_addr + 128 + piece * 32, ov);
#pragma unroll
                        for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * factor);
                        tmem_st32(lane_addr + 128 + piece * 32, ov);
                    }
                    tmem_st_wait();
                }
                const float ref = m_used == -INFINITY ? 0.f : m_used;  // a row that has seen no key yet
                float sum = 0.f;
#pragma unroll
                for (int c = 0; c < 64; c += 2) {
                    const float x0 = __uint_as_float(c < 32 ? s0[c] : s1[c - 32]);
                    const float x1 = __uint_as_float(c + 1 < 32 ? s0[c + 1] : s1[c + 1 - 32]);
                    const float e0 = ex2_approx(fmaf(x0, a.scale_log2, -ref)), e1 = ex2_approx(fmaf(x1, a.scale_log2, -ref));
                    __nv_bfloat162 pr = __floats2bfloat162_rn(e0, e1);
                    pk[c >> 1] = *reinterpret_cast<uint32_t*>(&pr);
                    // the row sum takes the weights as the product will see them (rounded): relative to a lazy maximum
                    // the largest weight is no power of two, and its rounding would otherwise show in O / l undiminished
                    const float2 seen = __bfloat1622float2(pr);
                    sum += seen.x + seen.y;
                }
                l += sum;
            }
            // P goes into tensor memory, over the S it was made from (this thread has that row of S in registers; S of
            // the group's tile after the next goes there only behind the product that reads this P)
            tmem_st32(lane_addr + (t & 1) * 64, pk);
            tmem_st_wait();
            if (j0 + kKV - 1 > last_pos) fence_async_smem();               // the zeroed V rows are for the tensor core's reads
            fence_before_sync();
            mbar_arrive(p_ready + 2 * grp + (t & 1));
            done = t + 1;
        }
        // The rows of O once the group's last product has landed, 64 dims at a time.  The groups' partial results meet
        // in shared memory ([column][row]: a warp's rows lie side by side), over the K|V ring: every group's products
        // have read it by now (each group waits for its own last one first).
        if (ok && done > 0) ok = wait_pv(done - 1, 8, grp + (done - 1) * kGroups);
        if (ok && done > 0) fence_after_sync();
        float* theirs0 = merge;                            // per group beyond the first: [66][128] floats
        float f0 = 1.f, l_all = l, m_all = m_used;
        float fg[kGroups] = {};
#pragma unroll 1
        for (int piece = 0; piece < kHD / 64; ++piece) {
            float o[64];
#pragma unroll
            for (int d = 0; d < 64; ++d) o[d] = 0.f;
            if (ok && done > 0) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t ov[32];
                    tmem_ld32(lane_addr + 128 + piece * 64 + half * 32, ov);
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[half * 32 + c] = __uint_as_float(ov[c]);
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kGroups * 128) : "memory");       // the ring (or the piece before) is done with
            if (grp > 0) {
                float* mine = theirs0 + (size_t)(grp - 1) * (64 + 2) * kQ;
#pragma unroll
                for (int d = 0; d < 64; ++d) mine[d * kQ + r] = o[d];
                mine[64 * kQ + r] = m_used;
                mine[(64 + 1) * kQ + r] = l;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kGroups * 128) : "memory");
            if (grp == 0) {
                if (piece == 0) {
                    float mt = m_used;
#pragma unroll
                    for (int g = 1; g < kGroups; ++g) mt = fmaxf(mt, theirs0[(size_t)(g - 1) * (64 + 2) * kQ + 64 * kQ + r]);
                    const float ref = mt == -INFINITY ? 0.f : mt;
                    m_all = mt;
                    f0 = exp2f(m_used - ref);
                    l_all = l * f0;
#pragma unroll
                    for (int g = 1; g < kGroups; ++g) {
                        const float* theirs = theirs0 + (size_t)(g - 1) * (64 + 2) * kQ;
                        fg[g] = exp2f(theirs[64 * kQ + r] - ref);
                        l_all += theirs[(64 + 1) * kQ + r] * fg[g];
                    }
                }
#pragma unroll
                for (int d = 0; d < 64; ++d) o[d] *= f0;
#pragma unroll
                for (int g = 1; g < kGroups; ++g) {
                    const float* theirs = theirs0 + (size_t)(g - 1) * (64 + 2) * kQ;
#pragma unroll
                    for (int d = 0; d < 64; ++d) o[d] += theirs[d * kQ + r] * fg[g];
                }
                if (a.splits > 1) {
                    // unnormalised, relative to the maximum that the groups agreed on; the merge kernel does the rest
                    const size_t at = ((size_t)item * a.splits + split) * kQ + r;
                    float4* po = reinterpret_cast<float4*>(a.part_o + at * kHD + piece * 64);
#pragma unroll
                    for (int c4 = 0; c4 < 16; ++c4) po[c4] = make_float4(o[4 * c4], o[4 * c4 + 1], o[4 * c4 + 2], o[4 * c4 + 3]);
                    if (piece == 0) { a.part_ml[at * 2] = ok ? m_all : -INFINITY; a.part_ml[at * 2 + 1] = ok ? l_all : 0.f; }
                } else if (ok && r < rows) {
                    const float inv = 1.f / l_all;
                    bf16* dst = a.out + ((size_t)(begin + q0 + r) * a.Hq + h) * kHD + piece * 64;
#pragma unroll
                    for (int c8 = 0; c8 < 8; ++c8) {
                        uint4 pc;
                        uint32_t* pw = reinterpret_cast<uint32_t*>(&pc);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 pr = __floats2bfloat162_rn(o[c8 * 8 + 2 * e] * inv, o[c8 * 8 + 2 * e + 1] * inv);
                            pw[e] = *reinterpret_cast<uint32_t*>(&pr);
                        }
                        *reinterpret_cast<uint4*>(dst + c8 * 8) = pc;
                    }
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    __syncwarp();
    if (warp == 1) tmem_free<kTmemCols>(tmem);
}
}  // namespace

namespace {
// Puts the key ranges of every (tile, head) together: one thread per query row and 16 dims.
__global__ void __launch_bounds__(kQ) attn_prefill_merge_kernel(TcArgs a, int hd) {
    const int item = blockIdx.x, r = threadIdx.x, d0 = blockIdx.y * 16;
    const int tile = item / a.Hq, h = item % a.Hq;
    const int b = a.tiles[2 * tile], q0 = a.tiles[2 * tile + 1];
    if (b < 0) return;
    const int begin = a.cu_seqlens[b], len = a.cu_seqlens[b + 1] - begin;
    if (r >= min(kQ, len - q0)) return;
    float mt = -INFINITY;
    for (int s = 0; s < a.splits; ++s) mt = fmaxf(mt, a.part_ml[(((size_t)item * a.splits + s) * kQ + r) * 2]);
    float acc[16], lsum = 0.f;
#pragma unroll
    for (int d = 0; d < 16; ++d) acc[d] = 0.f;
    for (int s = 0; s < a.splits; ++s) {
        const size_t at = ((size_t)item * a.splits + s) * kQ + r;
        const float ms = a.part_ml[at * 2];
        if (ms == -INFINITY) continue;                    // a range without keys left nothing to read
        const float f = exp2f(ms - mt);
        lsum += a.part_ml[at * 2 + 1] * f;
        const float4* po = reinterpret_cast<const float4*>(a.part_o + at * hd + d0);
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
            const float4 v = po[c4];
            acc[4 * c4] += v.x * f; acc[4 * c4 + 1] += v.y * f; acc[4 * c4 + 2] += v.z * f; acc[4 * c4 + 3] += v.w * f;
        }
    }
    const float inv = 1.f / lsum;
    bf16* dst = a.out + ((size_t)(begin + q0 + r) * a.Hq + h) * hd + d0;
#pragma unroll
    for (int c8 = 0; c8 < 2; ++c8) {
        uint4 pc;
        uint32_t* pw = reinterpret_cast<uint32_t*>(&pc);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 pr = __floats2bfloat162_rn(acc[c8 * 8 + 2 * e] * inv, acc[c8 * 8 + 2 * e + 1] * inv);
            pw[e] = *reinterpret_cast<uint32_t*>(&pr);
        }
        *reinterpret_cast<uint4*>(dst + c8 * 8) = pc;
    }
}
}  // namespace

// Does the tensor-core kernel take these sizes?  (Else: lb_attention_prefill.)
extern "C" int lb_attention_prefill_tc_ok(int Hq, int Hkv, int hd, int page_size) {
    return (hd == 64 || hd == 128) && page_size > 0 && page_size % kKV == 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 ? 1 : 0;
}

namespace {
template <int HD>
int launch_tc(const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v, const TcArgs& a, cudaStream_t stream) {
    typedef Shape<HD> Sh;
    const size_t smem = Sh::kQBytes + (size_t)Sh::kStages * 2 * Sh::kTileBytes + 256 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        configured = true;
    }
    attn_prefill_tc_kernel<HD><<<(unsigned)a.n_items * a.splits, kThreads, smem, stream>>>(map_q, map_k, map_v, a);
    if (a.splits > 1) attn_prefill_merge_kernel<<<dim3((unsigned)a.n_items, HD / 16), kQ, 0, stream>>>(a, HD);
    return launch_status();
}
}  // namespace

// q, out: [tokens, Hq, hd] bfloat16 contiguous, hd 64 or 128; caches [pages, page_size, Hkv, hd] contiguous; tiles: int32
// [n_tiles, 2] (request index, first token of the tile within the request's portion; 128 tokens per tile).
// `error`: a device int that is 0 before the call; non-zero afterwards: a wait inside the kernel gave up.
// `splits` > 1: key ranges per tile, with float32 scratch part_o [n_tiles * Hq * splits * 128 * hd] and
// part_ml [n_tiles * Hq * splits * 128 * 2] (see TcArgs).
extern "C" int lb_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out, long tokens,
                                       long pages, const int* block_table, int bt_stride, const int* cu_seqlens,
                                       const int* start_pos, const int* tiles, int n_tiles, int Hq, int Hkv, int hd,
                                       int page_size, float scale, int window, int* error, int splits, float* part_o,
                                       float* part_ml, void* stream) {
    if (n_tiles <= 0) return kOk;
    if (!lb_attention_prefill_tc_ok(Hq, Hkv, hd, page_size)) return kBadSize;
    if (splits < 1 || splits > 64 || (splits > 1 && (part_o == nullptr || part_ml == nullptr))) return kBadSize;
    if ((long)n_tiles * Hq * splits > 0x7fffffffL) return kTooLarge;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15) return kBadSize;
    CUtensorMap map_q, map_k, map_v;
    int rc = make_tile_map(&map_q, q, tokens, (long)Hq * hd, (long)Hq * hd, kQ);
    if (rc == 0) rc = make_tile_map(&map_k, k_cache, pages * page_size, (long)Hkv * hd, (long)Hkv * hd, kKV);
    if (rc == 0) rc = make_tile_map(&map_v, v_cache, pages * page_size, (long)Hkv * hd, (long)Hkv * hd, kKV);
    if (rc != 0) return rc;
    TcArgs a{(bf16*)out, block_table, bt_stride, cu_seqlens, start_pos, tiles, Hq, Hkv, page_size, window,
             scale * 1.4426950408889634f, n_tiles * Hq, error, splits, part_o, part_ml};
    return hd == 64 ? launch_tc<64>(map_q, map_k, map_v, a, (cudaStream_t)stream)
                    : launch_tc<128>(map_q, map_k, map_v, a, (cudaStream_t)stream);
}
