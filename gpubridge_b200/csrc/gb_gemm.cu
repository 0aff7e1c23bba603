// All-gather fused into a tcgen05 GEMM:  Y[M, N] = X[M, K] * W[N, K]^T  (bf16 in, fp32
// accumulate in tensor memory, bf16 out), where W is sharded by rows over the team the way
// FSDP2 shards a Linear weight.  This replaces "all_gather_into_tensor(weight shards), then
// F.linear" (reference: src/gpubridge/torch_backend.py:271-285 plus the model's nn.Linear).
//
// One persistent kernel, three kinds of blocks:
//   * communication blocks stage this rank's shard in its symmetric workspace, meet the peers
//     (team barrier), load every peer's shard over NVLink into the local gathered weight and
//     raise one ready flag per shard;
//   * GEMM blocks walk the output tiles shard by shard, starting with the own shard (which
//     needs no transfer), and only wait for a shard's flag right before the first TMA load
//     that touches it - so the tensor cores work on shard s while shard s+1 is in flight;
//   * inside a GEMM block: warp 0 issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle, one
//     destination block per load: every block reads this GPU's own memory) into a 4-stage shared-memory ring,
//     warp 1 issues tcgen05.mma (128 x 256 x 16, cta_group::1) from shared-memory descriptors
//     into one of two 256-column accumulators in tensor memory, warps 2-5 drain the other
//     accumulator with tcgen05.ld, convert to bf16 and store.
// Every mbarrier and flag wait is bounded; on expiry an error word is set, the wait falls
// through, and the block still frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gb_common.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;                 // 16 KiB
constexpr int B_BYTES = BN * BK * 2;                 // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;                    // TMA warp, MMA warp, four epilogue warps
constexpr int TMEM_COLS = 512;                       // two accumulators of 256 columns
constexpr unsigned WAIT_LIMIT = 1u << 27;

struct GemmArgs {
    __nv_bfloat16* y;
    const __nv_bfloat16* shard;      // this rank's rows of W: [shard_rows, K]
    __nv_bfloat16* gathered;         // the whole W, local: [N, K]
    unsigned int* flags;             // one per shard: the epoch for which it is complete
    unsigned int* error;             // set to 1 when a wait ran out
    unsigned int epoch;
    int M, N, K;
    int shard_rows;                  // N / world
    int gemm_blocks;                 // blocks [0, gemm_blocks) compute, the rest communicate
    size_t ws_off;                   // staging area for shards inside the workspaces
};

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
// Bounded wait: returns false (and records it) when the barrier never flipped.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned int* error) {
    for (unsigned spins = 0; spins < WAIT_LIMIT; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if (spins > 1024) __nanosleep(64);
    }
    atomicExch(error, 1u);
    return false;
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

// Output tile t of the schedule: shards in the order own, own+1, ...; inside a shard the
// n-tiles, inside an n-tile the m-tiles (so a weight tile is reused from L2 across m).
struct Tile { int m0, n0, shard; };
__device__ __forceinline__ Tile tile_at(const GemmArgs& a, const GbTeam& tm, long t) {
    const int m_tiles = (a.M + BM - 1) / BM;
    const int n_per_shard = (a.shard_rows + BN - 1) / BN;
    const long per_shard = (long)m_tiles * n_per_shard;
    const int step = (int)(t / per_shard);
    const long rest = t % per_shard;
    Tile tile;
    tile.shard = (tm.rank + step) % tm.world;
    tile.n0 = tile.shard * a.shard_rows + (int)(rest / m_tiles) * BN;
    tile.m0 = (int)(rest % m_tiles) * BM;
    return tile;
}

__global__ void __launch_bounds__(GEMM_THREADS)
allgather_gemm_kernel(const __grid_constant__ CUtensorMap map_x,
                      const __grid_constant__ CUtensorMap map_w, GbTeam tm, GemmArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // ---- communication blocks -------------------------------------------------------------
    if ((int)blockIdx.x >= a.gemm_blocks) {
        const int comm_blocks = (int)gridDim.x - a.gemm_blocks;
        const GbLane L = gb_lane_blocks(a.gemm_blocks, comm_blocks, tm.ld_mode);
        const size_t shard_bytes = (size_t)a.shard_rows * a.K * 2;
        char* mine = reinterpret_cast<char*>(a.gathered) + (size_t)tm.rank * shard_bytes;
        // the own shard goes straight into the gathered weight and into the workspace
        gb_copy_bytes(L, mine, a.shard, shard_bytes, false);
        if (tm.world > 1) gb_copy_bytes(L, tm.ws[tm.rank] + a.ws_off, a.shard, shard_bytes, false);
        if (!gb_sync(tm, 0, (unsigned)comm_blocks, 0, true, true)) return;
        if (L.tid == 0) gb_st_release_gpu(a.flags + tm.rank, a.epoch);
        for (int d = 1; d < tm.world; ++d) {
            const int peer = (tm.rank + d) % tm.world;
            gb_copy_bytes(L, reinterpret_cast<char*>(a.gathered) + (size_t)peer * shard_bytes,
                          tm.ws[peer] + a.ws_off, shard_bytes, true);
            // every block's stores, then one flag
            if (!gb_sync(tm, 0, (unsigned)comm_blocks, 1, false, false)) return;
            if (L.tid == 0) gb_st_release_gpu(a.flags + peer, a.epoch);
        }
        // peers may still be loading from this rank's workspace: leave together
        gb_sync(tm, 0, (unsigned)comm_blocks, 2, false, true);
        return;
    }
    // ---- GEMM blocks ------------------------------------------------------------------------
    // 128-byte swizzled tiles must start on a 1024-byte boundary
    unsigned char* tiles = reinterpret_cast<unsigned char*>(
        ((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;          // [2]
    uint64_t* acc_empty = acc_full + 2;           // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int m_tiles = (a.M + BM - 1) / BM;
    const int n_per_shard = (a.shard_rows + BN - 1) / BN;
    const long total = (long)m_tiles * n_per_shard * tm.world;
    const int k_blocks = (a.K + BK - 1) / BK;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        uint32_t stage = 0, phase = 0;
        int ready_shard = -1;
        for (long t = blockIdx.x; t < total; t += a.gemm_blocks) {
            const Tile tile = tile_at(a, tm, t);
            if (tile.shard != ready_shard) {
                // the shard's rows must have landed in the gathered weight
                bool ok = false;
                for (unsigned spins = 0; spins < WAIT_LIMIT; ++spins) {
                    if ((int)(gb_ld_acquire_gpu(a.flags + tile.shard) - a.epoch) >= 0) { ok = true; break; }
                    __nanosleep(100);
                }
                if (!ok) atomicExch(a.error, 2u);
                asm volatile("fence.proxy.async.global;" ::: "memory");
                ready_shard = tile.shard;
            }
            for (int kb = 0; kb < k_blocks; ++kb) {
                mbar_wait(empty + stage, phase ^ 1u, a.error);
                unsigned char* sa = tiles + stage * STAGE_BYTES;
                mbar_expect_tx(full + stage, STAGE_BYTES);
                tma_load_2d(sa, &map_x, kb * BK, tile.m0, full + stage);
                tma_load_2d(sa + A_BYTES, &map_w, kb * BK, tile.n0, full + stage);
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        constexpr uint32_t idesc = instr_desc(BM, BN);
        uint32_t stage = 0, phase = 0, local = 0;
        for (long t = blockIdx.x; t < total; t += a.gemm_blocks, ++local) {
            const uint32_t buf = local & 1u, use = local >> 1;
            mbar_wait(acc_empty + buf, (use & 1u) ^ 1u, a.error);   // the epilogue drained it
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + buf * BN;
            for (int kb = 0; kb < k_blocks; ++kb) {
                mbar_wait(full + stage, phase, a.error);
                tc_fence_after();
                const unsigned char* sa = tiles + stage * STAGE_BYTES;
                const uint64_t da = smem_desc(sa), db = smem_desc(sa + A_BYTES);
                #pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk)           // 32 bytes along K per step
                    tc_mma(tmem_d, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
                tc_commit(empty + stage);                      // frees the stage when they finish
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            tc_commit(acc_full + buf);
        }
    } else if (warp >= 2) {
        // ---- epilogue: tensor memory -> registers -> bf16 -> global ----
        const int quarter = warp & 3;                          // the lanes this warp may read
        uint32_t local = 0;
        for (long t = blockIdx.x; t < total; t += a.gemm_blocks, ++local) {
            const Tile tile = tile_at(a, tm, t);
            const uint32_t buf = local & 1u, use = local >> 1;
            mbar_wait(acc_full + buf, use & 1u, a.error);
            tc_fence_after();
            const int row = tile.m0 + quarter * 32 + lane;
            const int shard_end = (tile.shard + 1) * a.shard_rows;
            #pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + c, r);
                const int col = tile.n0 + c;
                if (row < a.M && col < shard_end && col < a.N) {
                    __nv_bfloat16* dst = a.y + (size_t)row * a.N + col;
                    if (col + 32 <= shard_end && col + 32 <= a.N &&
                        ((((size_t)row * a.N + col) & 7) == 0)) {
                        #pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            uint4 out;
                            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
                            #pragma unroll
                            for (int j = 0; j < 4; ++j)
                                h[j] = __floats2bfloat162_rn(__uint_as_float(r[8 * g + 2 * j]),
                                                             __uint_as_float(r[8 * g + 2 * j + 1]));
                            *reinterpret_cast<uint4*>(dst + 8 * g) = out;
                        }
                    } else {
                        for (int j = 0; j < 32 && col + j < shard_end && col + j < a.N; ++j)
                            dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + buf);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_free(tmem_base, TMEM_COLS);
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
    EncodeTiled encode = encoder();
    if (encode == nullptr) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
           CUDA_SUCCESS;
}

}  // namespace

// Y = X * gather(W shards)^T.  x: [M, K], shard: [N / world, K], gathered: [N, K] (scratch that
// ends up holding the whole weight), y: [M, N]; all bf16, 16-byte aligned, K a multiple of 8.
// flags: world zero-initialised words that persist across calls; error: one word; epoch:
// increases by one per call.  grid = gemm_blocks + comm_blocks (comm_blocks >= 1).
// Returns a cudaError_t, or -3 when the tensor maps could not be built.
extern "C" int gb_allgather_gemm(const GbTeam* team, void* y, const void* x, const void* shard,
                                 void* gathered, unsigned int* flags, unsigned int* error,
                                 unsigned int epoch, int M, int N, int K, size_t ws_off,
                                 int gemm_blocks, int comm_blocks, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0 || (K & 7) || N % team->world || gemm_blocks < 1 ||
        comm_blocks < 1)
        return (int)cudaErrorInvalidValue;
    CUtensorMap map_x, map_w;
    if (!make_map(&map_x, x, M, K, BM) || !make_map(&map_w, gathered, N, K, BN)) return -3;
    GemmArgs a;
    a.y = static_cast<__nv_bfloat16*>(y);
    a.shard = static_cast<const __nv_bfloat16*>(shard);
    a.gathered = static_cast<__nv_bfloat16*>(gathered);
    a.flags = flags; a.error = error; a.epoch = epoch;
    a.M = M; a.N = N; a.K = K;
    a.shard_rows = N / team->world;
    a.gemm_blocks = gemm_blocks;
    a.ws_off = ws_off;
    const size_t smem = STAGES * STAGE_BYTES + 256 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(allgather_gemm_kernel,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
        configured = true;
    }
    allgather_gemm_kernel<<<gemm_blocks + comm_blocks, GEMM_THREADS, smem, stream>>>(map_x, map_w,
                                                                                   *team, a);
    return (int)cudaGetLastError();
}
