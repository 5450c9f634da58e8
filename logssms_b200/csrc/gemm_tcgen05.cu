// Projections of prompt portions on the 5th-generation tensor cores:  C[M, N] = A[M, K] W[N, K]^T, bfloat16
// operands, float32 accumulation in tensor memory, with the epilogues the layers need fused in.
//
//   tile      128 (M) x 128 (N) per CTA, K in blocks of 64 (one 128-byte swizzle row of bfloat16)
//   warp 0    one thread issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle, zero fill outside the
//             matrices) of the A block and the two 64-row halves of the W block into a 3-stage ring of
//             shared memory; each stage has a "full" mbarrier (armed with the stage's byte count) and an
//             "empty" one
//   warp 1    allocates 128 columns of tensor memory; one thread issues tcgen05.mma (cta_group::1, kind::f16,
//             M 128, N 128, K 16: four per block, the shared-memory descriptors advanced by 32 bytes) and
//             tcgen05.commit onto the stage's "empty" barrier, at the end onto the "accumulator ready" barrier
//   warps 2-5 read the accumulator with tcgen05.ld (32 lanes x 32 columns at a time; warp w may touch lanes
//             32 (w mod 4) .. +31, i.e. rows of the tile), apply the epilogue and store
//   Two CTAs fit on an SM (97 KB shared memory, 128 of 512 tensor-memory columns each), so one CTA's epilogue
//   overlaps the other's main loop.  A product with so few 128-wide tiles that SMs would stay idle runs with
//   64-wide tiles (one W box per stage, 4 stages) instead.
//
// Epilogues, rounding where the unfused chain rounds (python/logssms/layers/linear.py:26,
// python/logssms/kernel/fused.py:32-50):
//   plain  : out = round(round(acc + bias) * out_scale)                              bfloat16
//   f32    : out = float(round(acc + bias)) * out_scale                              float32
//   swiglu : W = [gate rows; up rows]; the W block holds 64 gate rows and the 64 up rows of the same
//            features, so accumulator columns j and j + 64 pair up:
//            out = round(round(silu(round(round(acc_gate) * act_scale))) * round(acc_up))     bfloat16
//
// Every wait on an mbarrier is bounded: after about a second of polling the thread records (role, block,
// k-block) in `error`, the roles stop, tensor memory is freed and the kernel returns.
#include <cuda.h>

#include "lb200/common.cuh"
using namespace lb200;

namespace {
constexpr int BM = 128, BK = 64;                          // the N extent of a tile is a template parameter: 128 or 64
constexpr int kThreads = 192;
constexpr uint32_t kABytes = BM * BK * 2, kBHalfBytes = 64 * BK * 2;     // W arrives in boxes of 64 rows
constexpr uint32_t stage_bytes(int bn) { return kABytes + (bn / 64) * kBHalfBytes; }
constexpr uint32_t kSpinLimit = 1u << 22;                 // polls of try_wait before a wait gives up

struct GemmArgs {
    void* out; long ldo;
    const __nv_bfloat16* bias;
    int M, N, K;                                          // N: output features (for swiglu: of the product, = I)
    float out_scale, act_scale;
    int epilogue;                                         // 0 plain, 1 float32 out, 2 swiglu
    int* error;
};
enum : int { kPlain = 0, kOutF32 = 1, kSwiglu = 2 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// true when the phase with this parity has completed; gives up after kSpinLimit polls
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// K-major operand tile in shared memory, rows of 128 bytes, 128-byte swizzle: 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(const void* tile) {
    uint64_t d = (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;                               // leading byte offset (unused with a swizzle): 16 bytes
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                               // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                               // 128-byte swizzle
    return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void report(int* error, int role, int kb) {
    if (error != nullptr) atomicCAS(error, 0, (role << 24) | ((blockIdx.x & 0xFFF) << 12) | (kb & 0xFFF) | 0x40000000);
}

template <int kStages, int BN>
__global__ void __launch_bounds__(kThreads)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmArgs g) {
    constexpr uint32_t kStageBytes = stage_bytes(BN);
    constexpr uint32_t kTmemCols = BN;                    // accumulator columns (a power of two >= 32)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzle atoms: 1024-byte aligned
    uint64_t* full = reinterpret_cast<uint64_t*>(base + kStages * kStageBytes);
    uint64_t* empty = full + kStages;
    uint64_t* acc_ready = empty + kStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (g.N + (g.epilogue == kSwiglu ? BN / 2 : BN) - 1) / (g.epilogue == kSwiglu ? BN / 2 : BN);
    const int tile_m = blockIdx.x / tiles_n, tile_n = blockIdx.x % tiles_n;
    const int m0 = tile_m * BM;
    // rows of W for the two halves of the block: consecutive features, or gate and up rows of the same features
    const int w_row0 = g.epilogue == kSwiglu ? tile_n * (BN / 2) : tile_n * BN;
    const int w_row1 = g.epilogue == kSwiglu ? g.N + tile_n * (BN / 2) : tile_n * BN + BN / 2;
    const int num_kb = (g.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        mbar_init(acc_ready, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < num_kb && !*failed; ++kb, ++issued) {
                const int s = kb % kStages;
                if (kb >= kStages && !mbar_wait(empty + s, ((kb / kStages) - 1) & 1)) { report(g.error, 1, kb); *failed = 1; break; }
                uint8_t* a_tile = base + s * kStageBytes;
                mbar_expect_tx(full + s, kStageBytes);
                tma_load_2d(a_tile, &map_a, full + s, kb * BK, m0);
                tma_load_2d(a_tile + kABytes, &map_b, full + s, kb * BK, w_row0);
                if (BN == 128) tma_load_2d(a_tile + kABytes + kBHalfBytes, &map_b, full + s, kb * BK, w_row1);
            }
            if (*failed) {                                 // let the copies already under way land before the CTA leaves
                for (int kb = max(0, issued - kStages); kb < issued; ++kb) mbar_wait(full + kb % kStages, (kb / kStages) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, N >> 3, M >> 4
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            for (int kb = 0; kb < num_kb && !*failed; ++kb) {
                const int s = kb % kStages;
                if (!mbar_wait(full + s, (kb / kStages) & 1)) { report(g.error, 2, kb); *failed = 1; break; }
                tc_fence_after();
                const uint64_t adesc = umma_desc(base + s * kStageBytes);
                const uint64_t bdesc = umma_desc(base + s * kStageBytes + kABytes);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)          // 16 bfloat16 = 32 bytes along K: + 2 in the 16-byte address field
                    umma_bf16(tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
                umma_commit(empty + s);                    // arrives when these products have read the stage
            }
            umma_commit(acc_ready);
        }
    } else {
        const bool ok = mbar_wait(acc_ready, 0);
        if (!ok && lane == 0) { report(g.error, 3, 0); *failed = 1; }
        tc_fence_after();
        if (__all_sync(0xffffffffu, ok && !*failed)) {     // tcgen05.ld wants the whole warp: decide together
            const int quarter = warp & 3;                  // the lanes of tensor memory this warp may read
            const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
            // The stage ring is idle now (every product has been committed): this warp's 32 rows pass through
            // its own slice of it, so that the stores to global memory are whole 16-byte pieces of a row.
            const int out_cols = g.epilogue == kSwiglu ? BN / 2 : BN;          // columns of the output tile
            const int col0 = tile_n * out_cols;
            const int esz = g.epilogue == kOutF32 ? 4 : 2;
            const int row_bytes = out_cols * esz + 16;                          // padded: rows land in different banks
            uint8_t* stage_rows = base + (size_t)quarter * 32 * (BN * 4 + 16);
            uint8_t* my_row = stage_rows + (size_t)lane * row_bytes;
#pragma unroll 1
            for (int c = 0; c < out_cols; c += 32) {
                uint32_t acc[32];
                tmem_ld32(lane_addr + c, acc);
                if (g.epilogue == kSwiglu) {
                    uint32_t up[32];
                    tmem_ld32(lane_addr + BN / 2 + c, up);
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        float o2[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const float gv = round_to<__nv_bfloat16>(round_to<__nv_bfloat16>(__uint_as_float(acc[j + e])) * g.act_scale);
                            const float act = round_to<__nv_bfloat16>(silu_f(gv));
                            o2[e] = act * round_to<__nv_bfloat16>(__uint_as_float(up[j + e]));
                        }
                        *reinterpret_cast<__nv_bfloat162*>(my_row + (c + j) * 2) = __floats2bfloat162_rn(o2[0], o2[1]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        float v2[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            float v = __uint_as_float(acc[j + e]);
                            if (g.bias != nullptr && col0 + c + j + e < g.N) v += __bfloat162float(g.bias[col0 + c + j + e]);
                            v2[e] = round_to<__nv_bfloat16>(v) * g.out_scale;
                        }
                        if (g.epilogue == kOutF32) *reinterpret_cast<float2*>(my_row + (c + j) * 4) = make_float2(v2[0], v2[1]);
                        else *reinterpret_cast<__nv_bfloat162*>(my_row + (c + j) * 2) = __floats2bfloat162_rn(v2[0], v2[1]);
                    }
                }
            }
            __syncwarp();
            // rows of the warp, 16 bytes per lane; whole pieces when the row start and N allow it, else element by element
            const int pieces = out_cols * esz / 16;
            const bool vec_ok = ((g.ldo * esz) % 16 == 0) && (((uintptr_t)g.out) % 16 == 0) && ((col0 * esz) % 16 == 0);
            for (int i = lane; i < 32 * pieces; i += 32) {
                const int r = i / pieces, pc = i % pieces;
                const int grow = m0 + quarter * 32 + r;
                if (grow >= g.M) continue;
                const int first_col = col0 + pc * (16 / esz);
                const uint8_t* src = stage_rows + (size_t)r * row_bytes + pc * 16;
                uint8_t* dst = (uint8_t*)g.out + ((size_t)grow * g.ldo + first_col) * esz;
                if (vec_ok && first_col + 16 / esz <= g.N) {
                    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
                } else {
                    for (int e = 0; e < 16 / esz && first_col + e < g.N; ++e) {
                        if (esz == 4) reinterpret_cast<float*>(dst)[e] = reinterpret_cast<const float*>(src)[e];
                        else reinterpret_cast<__nv_bfloat16*>(dst)[e] = reinterpret_cast<const __nv_bfloat16*>(src)[e];
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encoder() {
    static EncodeTiled fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    }
    return fn;
}

// rows x K bfloat16 matrix with a row stride (elements); box = box_rows x 64 elements, 128-byte swizzle, zero fill
int make_map(CUtensorMap* map, const void* ptr, long rows, long K, long row_stride, int box_rows) {
    EncodeTiled enc = encoder();
    if (enc == nullptr) return (int)cudaErrorNotSupported;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}
}  // namespace

// a: [M, K] bfloat16 rows (row stride lda elements, a multiple of 8; 16-byte aligned); w: [N, K] contiguous
// ([2N, K] for swiglu: gate rows, then up rows); K a multiple of 8.  `error`: a device int that is 0 before
// the call; a non-zero value afterwards means a wait inside the kernel gave up (role, block, k-block).
extern "C" int lb_gemm_tcgen05(const void* a, long lda, const void* w, const void* bias, void* out, long ldo, int M,
                               int N, int K, float out_scale, float act_scale, int epilogue, int* error, void* stream) {
    if (M <= 0 || N <= 0) return kOk;
    if (K <= 0 || K % 8 || lda % 8 || epilogue < 0 || epilogue > 2) return kBadSize;
    if (((uintptr_t)a | (uintptr_t)w) & 15) return kBadSize;
    CUtensorMap map_a, map_b;
    int rc = make_map(&map_a, a, M, K, lda, BM);
    if (rc != 0) return rc;
    rc = make_map(&map_b, w, epilogue == kSwiglu ? 2L * N : N, K, K, 64);
    if (rc != 0) return rc;
    GemmArgs g{out, ldo, (const __nv_bfloat16*)bias, M, N, K, out_scale, act_scale, epilogue, error};
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const long tiles_m = (M + BM - 1) / BM;
    // 128-wide tiles unless they would not even give every SM one CTA; then 64-wide ones (twice as many).
    // SwiGLU always takes 64 gate + 64 up rows of W per tile.
    const bool narrow = epilogue != kSwiglu && tiles_m * ((N + 127) / 128) <= sms;
    const int per_tile_n = (epilogue == kSwiglu || narrow) ? 64 : 128;
    const long tiles = tiles_m * ((N + per_tile_n - 1) / per_tile_n);
    if (tiles > 0x7fffffffL) return kTooLarge;
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(gemm_tcgen05_kernel<3, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * (int)stage_bytes(128) + 1280);
        cudaFuncSetAttribute(gemm_tcgen05_kernel<4, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * (int)stage_bytes(64) + 1280);
        configured = true;
    }
    if (narrow) {
        const size_t smem = 4 * (size_t)stage_bytes(64) + 1280;         // 4 x 24 KB: two CTAs per SM
        gemm_tcgen05_kernel<4, 64><<<(unsigned)tiles, kThreads, smem, (cudaStream_t)stream>>>(map_a, map_b, g);
    } else {
        const size_t smem = 3 * (size_t)stage_bytes(128) + 1280;        // 3 x 32 KB: two CTAs per SM
        gemm_tcgen05_kernel<3, 128><<<(unsigned)tiles, kThreads, smem, (cudaStream_t)stream>>>(map_a, map_b, g);
    }
    return launch_status();
}
