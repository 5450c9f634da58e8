// Inline-PTX pieces shared by the kernels that run on the 5th-generation tensor cores: mbarriers with bounded
// waits, TMA tile loads, shared-memory operand descriptors, tcgen05.mma / commit / ld and the fences around them.
//
// Operand tiles in shared memory are rows of 128 bytes (64 bfloat16) with the 128-byte swizzle, 8-row groups 1024
// bytes apart, on a 1024-byte boundary: what a TMA box of 64 x rows elements with CU_TENSOR_MAP_SWIZZLE_128B
// leaves, and what a thread writes as 16-byte piece `c ^ (row & 7)` of its row.  The same tile is read K-major
// (its rows are M or N, a row holds 64 values of k; 16 values of k further on = descriptor + 2) or MN-major (its
// rows are k, a row holds 64 values of m or n; 16 values of k further on = descriptor + 2048 / 16): the
// instruction descriptor says which.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lb200 {
namespace tc {

constexpr uint32_t kSpinLimit = 1u << 22;                  // polls of an mbarrier before a wait gives up (about a second)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// false: the phase did not complete within kSpinLimit polls
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
// x: element index along the rows (x * element size must be a multiple of 16 bytes), y: row
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ uint64_t umma_desc(const void* tile) {
    uint64_t d = (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;                               // leading byte offset: unused (one 64-wide block)
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                               // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                               // 128-byte swizzle
    return d;
}
// float32 accumulator, bfloat16 operands, both K-major; `kBMnMajor` added: the B operand is MN-major
__host__ __device__ constexpr uint32_t umma_idesc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
constexpr uint32_t kBMnMajor = 1u << 16;
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with the A operand in tensor memory (M rows = lanes, two 16-bit values of k per column)
__device__ __forceinline__ void umma_bf16_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// the barrier gets one arrival when every product issued by this thread so far has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 consecutive float32 columns of this thread's lane of tensor memory
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
// the way back: 32 consecutive float32 columns of this thread's lane; tmem_st_wait() before anybody else reads them
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
template <uint32_t kCols>
__device__ __forceinline__ void tmem_alloc(uint32_t* slot) {     // one whole warp; the address lands in *slot
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "n"(kCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <uint32_t kCols>
__device__ __forceinline__ void tmem_free(uint32_t addr) {       // the same warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "n"(kCols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// writes of this thread to shared memory become visible to the tensor core's and TMA's reads
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 2^x in one special-function instruction (relative error 2^-22, results below 2^-126 flushed to zero): for softmax
// weights and decay factors, which lie in [0, 1] and are rounded to bfloat16 operands next
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiled tensor_map_encoder() {
    static EncodeTiled fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    }
    return fn;
}
// A rows x width bfloat16 matrix whose rows lie `row_stride` elements apart (a multiple of 8; base on a 16-byte
// boundary); box = box_rows x 64 elements, 128-byte swizzle, zeros outside.  0 or a cudaError.
inline int make_tile_map(CUtensorMap* map, const void* ptr, long rows, long width, long row_stride, int box_rows) {
    // The same few tensors come back step after step (caches; activations that the allocator hands out at the same
    // address): the last maps are kept, an encoding costs the host a few microseconds.
    struct Entry { const void* ptr; long rows, width, stride; int box_rows; CUtensorMap map; };
    constexpr int kEntries = 256;                         // two caches per layer of a deep model and a few activations
    thread_local Entry cache[kEntries] = {};
    thread_local int next = 0;
    for (int i = 0; i < kEntries; ++i) {
        const Entry& e = cache[i];
        if (e.ptr == ptr && e.rows == rows && e.width == width && e.stride == row_stride && e.box_rows == box_rows) {
            *map = e.map;
            return 0;
        }
    }
    EncodeTiled enc = tensor_map_encoder();
    if (enc == nullptr) return (int)cudaErrorNotSupported;
    const cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    cache[next] = Entry{ptr, rows, width, row_stride, box_rows, *map};
    next = (next + 1) % kEntries;
    return 0;
}

}  // namespace tc
}  // namespace lb200
