// tcgen05 / TMA / mbarrier wrappers, guarded waits and tensor-map helpers shared by the GEMM
// kernels (bf16 operands, fp32 accumulators in tensor memory, 128-byte swizzle).  The tile
// shape of the single-CTA kernels is in gb_tc_tile.cuh; the CTA-pair kernel has its own.
// Include from one translation unit per kernel file; everything has internal linkage.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                 :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// What a role needs to give up cleanly: the kernel's error word, the team's abort word (set by
// any bounded wait of the team that ran out, in this or an earlier kernel) and the deadline of
// one wait.  Error codes: 1 operand stage never freed, 2 shard flag never raised, 3 accumulator
// never drained, 4 operand stage never filled, 5 accumulator never completed.
struct TcGuard {
    unsigned int* error;
    const unsigned int* abort;
    unsigned long long limit_ns;
};
__device__ __forceinline__ unsigned long long tc_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool tc_dead(const TcGuard& g) {
    return *reinterpret_cast<volatile const unsigned int*>(g.error) != 0u ||
           *reinterpret_cast<volatile const unsigned int*>(g.abort) != 0u;
}
// Wait until the barrier's phase `parity` has completed.  Gives up - and returns false - when
// the deadline passes (the error word then gets `code`) or when some other wait of the kernel or
// the team has already given up.  After a false return the caller leaves its tile loop: a role
// that kept going would run every later wait to its deadline too.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const TcGuard& g,
                                          unsigned code) {
    unsigned long long t0 = 0;
    for (unsigned spins = 0; spins < 0x40000000u; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 31u) == 31u) {
            if (tc_dead(g)) return false;
            const unsigned long long now = tc_now();
            if (t0 == 0) t0 = now;
            else if (now - t0 > g.limit_ns) break;
            __nanosleep(64);
        }
    }
    atomicCAS(g.error, 0u, code);
    return false;
}
// The same wait by a whole warp whose next instruction is warp-wide (tcgen05.ld): either every
// lane goes on or none does.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, const TcGuard& g,
                                               unsigned code) {
    const bool ok = mbar_wait(bar, parity, g, code);
    return __all_sync(0xffffffffu, ok) != 0;
}
// Poll a flag in global memory (written with release semantics by another block of this GPU)
// until it reaches `want`; same giving-up rules as mbar_wait.
__device__ __forceinline__ bool tc_wait_flag(const unsigned int* flag, unsigned want,
                                             const TcGuard& g, unsigned code) {
    unsigned long long t0 = 0;
    for (unsigned spins = 0; spins < 0x40000000u; ++spins) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if ((int)(v - want) >= 0) return true;
        __nanosleep(100);
        if ((spins & 31u) == 31u) {
            if (tc_dead(g)) return false;
            const unsigned long long now = tc_now();
            if (t0 == 0) t0 = now;
            else if (now - t0 > g.limit_ns) break;
        }
    }
    atomicCAS(g.error, 0u, code);
    return false;
}
// After a producer gave up: the loads it already issued still write into this block's shared
// memory, so the block may not exit before they have landed.  `issued` loads went out in ring
// order; wait - briefly, bounded - for the last `stages` of them.
__device__ __forceinline__ void tc_drain_loads(uint64_t* full, uint32_t issued, int stages) {
    const uint32_t first = issued > (uint32_t)stages ? issued - (uint32_t)stages : 0u;
    for (uint32_t i = first; i < issued; ++i) {
        uint64_t* bar = full + (i % (uint32_t)stages);
        const uint32_t parity = (i / (uint32_t)stages) & 1u;
        const unsigned long long t0 = tc_now();
        for (unsigned spins = 0; spins < (1u << 20); ++spins) {
            if (mbar_try_wait(bar, parity)) break;
            if ((spins & 31u) == 31u && tc_now() - t0 > 2000000ull) break;      // 2 ms
        }
    }
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y,
                                            uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%2, %3}], [%4];"
                 :: "r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(smem_u32(smem_result)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(addr), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 :: "r"(smem_u32(bar)) : "memory");
}
// After the issuer gave up: its earlier tcgen05.mma instructions may still be reading shared
// memory and writing tensor memory.  Commit once more to a spare barrier and wait - briefly,
// bounded - for that, so that nothing is in flight when the block frees its tensor memory.
__device__ __forceinline__ void tc_drain_mma(uint64_t* spare) {
    tc_commit(spare);
    const unsigned long long t0 = tc_now();
    for (unsigned spins = 0; spins < (1u << 20); ++spins) {
        if (mbar_try_wait(spare, 0u)) break;
        if ((spins & 31u) == 31u && tc_now() - t0 > 2000000ull) break;          // 2 ms
    }
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// 32 consecutive fp32 columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and 128-byte swizzle:
// start address / 16, leading byte offset 1 (unused for swizzled K-major), stride byte offset
// 1024 / 16 (eight rows), version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc(const void* tile) {
    const uint64_t addr = (uint64_t)(smem_u32(tile) >> 4) & 0x3FFFu;
    return addr | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: D = F32, A = B = BF16, both K-major, N and M of the instruction.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encoder() {
    static EncodeTiled fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) ==
                cudaSuccess && status == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(ptr);
    }
    return fn;
}

// A [rows, K] row-major bf16 matrix, read in boxes of box_rows x 64 with 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    constexpr int BOX_K = 64;                        // 128 bytes: one swizzle row
    EncodeTiled encode = encoder();
    if (encode == nullptr) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BOX_K, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
           CUDA_SUCCESS;
}

}  // namespace
