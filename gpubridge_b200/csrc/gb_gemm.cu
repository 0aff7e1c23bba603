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
// Every mbarrier and flag wait has a deadline (the team's wait limit) and also ends as soon as
// the error word or the team's abort word is set; a role whose wait gave up leaves its tile
// loop, the producer waits briefly for the loads it has in flight, the issuer for its last
// instructions, and the block still meets at its barrier, frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gb_common.cuh"
#include "gb_tc_tile.cuh"

namespace {

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
    size_t ws_off;                   // staging area for shards inside the workspaces ...
    size_t ws_half;                  // ... two halves this far apart, one per parity
};

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
        // The staging region has two halves selected by the parity of the team's collective
        // counter, like every region that is written before a kernel's first barrier: the
        // collective before this one (an all-gather that leaves without a closing barrier, say)
        // used the other half, so a slow peer may still be reading it.  Read before the barrier
        // below advances the counter.
        const size_t stage_off = a.ws_off + (size_t)(gb_ld_volatile(&tm.ctrl->epoch) & 1u) * a.ws_half;
        // the own shard goes straight into the gathered weight and into the workspace
        gb_copy_bytes(L, mine, a.shard, shard_bytes, false);
        if (tm.world > 1) gb_copy_bytes(L, tm.ws[tm.rank] + stage_off, a.shard, shard_bytes, false);
        if (!gb_sync(tm, 0, (unsigned)comm_blocks, 0, true, true)) return;
        if (L.tid == 0) gb_st_release_gpu(a.flags + tm.rank, a.epoch);
        for (int d = 1; d < tm.world; ++d) {
            const int peer = (tm.rank + d) % tm.world;
            gb_copy_bytes(L, reinterpret_cast<char*>(a.gathered) + (size_t)peer * shard_bytes,
                          tm.ws[peer] + stage_off, shard_bytes, true);
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
    uint64_t* drained = acc_empty + 2;            // the issuer's last instructions after a failure
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drained + 1);
    const TcGuard guard = {a.error, &tm.ctrl->abort, tm.timeout_ns};
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 4); }
        mbar_init(drained, 1);
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
        uint32_t stage = 0, phase = 0, issued = 0;
        int ready_shard = -1;
        bool alive = true;
        for (long t = blockIdx.x; alive && t < total; t += a.gemm_blocks) {
            const Tile tile = tile_at(a, tm, t);
            if (tile.shard != ready_shard) {
                // the shard's rows must have landed in the gathered weight
                if (!tc_wait_flag(a.flags + tile.shard, a.epoch, guard, 2u)) { alive = false; break; }
                asm volatile("fence.proxy.async.global;" ::: "memory");
                ready_shard = tile.shard;
            }
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(empty + stage, phase ^ 1u, guard, 1u)) { alive = false; break; }
                unsigned char* sa = tiles + stage * STAGE_BYTES;
                mbar_expect_tx(full + stage, STAGE_BYTES);
                tma_load_2d(sa, &map_x, kb * BK, tile.m0, full + stage);
                tma_load_2d(sa + A_BYTES, &map_w, kb * BK, tile.n0, full + stage);
                ++issued;
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        if (!alive) tc_drain_loads(full, issued, STAGES);
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        constexpr uint32_t idesc = instr_desc(BM, BN);
        uint32_t stage = 0, phase = 0, local = 0;
        bool alive = true;
        for (long t = blockIdx.x; alive && t < total; t += a.gemm_blocks, ++local) {
            const uint32_t buf = local & 1u, use = local >> 1;
            // the epilogue drained it
            if (!mbar_wait(acc_empty + buf, (use & 1u) ^ 1u, guard, 3u)) { alive = false; break; }
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + buf * BN;
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(full + stage, phase, guard, 4u)) { alive = false; break; }
                tc_fence_after();
                const unsigned char* sa = tiles + stage * STAGE_BYTES;
                const uint64_t da = smem_desc(sa), db = smem_desc(sa + A_BYTES);
                #pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk)           // 32 bytes along K per step
                    tc_mma(tmem_d, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
                tc_commit(empty + stage);                      // frees the stage when they finish
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (alive) tc_commit(acc_full + buf);
        }
        if (!alive) tc_drain_mma(drained);
    } else if (warp >= 2) {
        // ---- epilogue: tensor memory -> registers -> bf16 -> global ----
        const int quarter = warp & 3;                          // the lanes this warp may read
        uint32_t local = 0;
        for (long t = blockIdx.x; t < total; t += a.gemm_blocks, ++local) {
            const Tile tile = tile_at(a, tm, t);
            const uint32_t buf = local & 1u, use = local >> 1;
            if (!mbar_wait_warp(acc_full + buf, use & 1u, guard, 5u)) break;
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

}  // namespace

// Y = X * gather(W shards)^T.  x: [M, K], shard: [N / world, K], gathered: [N, K] (scratch that
// ends up holding the whole weight), y: [M, N]; all bf16, 16-byte aligned, K a multiple of 8.
// flags: world zero-initialised words that persist across calls; error: one word; epoch:
// increases by one per call.  [ws_off, ws_off + 2 * ws_half) of every workspace is the staging
// region (two halves of ws_half bytes, each at least one shard).  grid = gemm_blocks +
// comm_blocks (comm_blocks >= 1).
// Returns a cudaError_t, or -3 when the tensor maps could not be built.
extern "C" int gb_allgather_gemm(const GbTeam* team, void* y, const void* x, const void* shard,
                                 void* gathered, unsigned int* flags, unsigned int* error,
                                 unsigned int epoch, int M, int N, int K, size_t ws_off,
                                 size_t ws_half, int gemm_blocks, int comm_blocks, cudaStream_t stream) {
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
    a.ws_half = ws_half;
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

GB_BOUNDS_HOST(gemm)
