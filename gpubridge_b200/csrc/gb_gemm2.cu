// The all-gather GEMM of gb_gemm.cu on CTA pairs (tcgen05 cta_group::2).
//
// Measured on B200, the single-CTA kernel runs at the rate one SM can pull operands from L2:
// a 128 x 256 x 64 step needs 48 KB for 4.19 MFLOP.  Here two CTAs of a cluster work on one
// 256 x 256 output tile: each loads its own 128 rows of X and only its half (128 rows) of the
// W tile, the tensor cores of both SMs read the two halves of W from both shared memories, and
// each CTA accumulates its 128 x 256 half in its own tensor memory.  Per SM that is 32 KB per
// step for the same math (131 FLOP/B instead of 87), and six pipeline stages fit instead of
// four.
//
// Roles per CTA: warp 0 issues the TMA loads of its halves (completion counted on the pair
// leader's barrier), warp 1 of the leader issues tcgen05.mma for the pair and commits to the
// barriers of both CTAs, warps 2-5 of each CTA drain their CTA's accumulator.  No load
// fans out to several CTAs: every CTA reads this GPU's own memory with plain tile loads.
// Every wait has a deadline (the team's wait limit) and ends early once the error word or the
// team's abort word is set; a role whose wait gave up leaves its tile loop, and the CTAs still
// meet at the cluster barrier, free their tensor memory and return.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "gb_common.cuh"
#include "gb_tc.cuh"

namespace {

constexpr int BM = 256, BK = 64;               // per pair
constexpr int HALF = 128;                      // rows of X and rows of W per CTA and MMA
constexpr int A_BYTES = HALF * BK * 2;         // 16 KiB
constexpr int B_BYTES = HALF * BK * 2;         // 16 KiB per 256-column half of the output tile
constexpr int THREADS2 = 192;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_TILES = 192 << 10;          // operand ring of either shape

// The output tile of a pair is 256 x (256 * NH).  NH = 1: two 256-column accumulators, so the
// epilogue of one tile runs under the main loop of the next; 32 KB of operands per CTA and
// step, six stages.  NH = 2: one 512-column accumulator (all of tensor memory) fed by two MMAs
// per step that share the X tile; 48 KB per CTA and step for twice the math - a quarter less
// operand traffic per FLOP, which is what bounds this kernel (measured: loading the operands
// alone takes longer than cuBLAS's whole GEMM) - at the price of an epilogue that the next
// tile's main loop has to wait for; four stages.
template <int NH> struct Shape {
    static constexpr int BN = 256 * NH;
    static constexpr int STAGE_BYTES = A_BYTES + NH * B_BYTES;
    static constexpr int STAGES = SMEM_TILES / STAGE_BYTES;
    static constexpr int ACCS = NH == 1 ? 2 : 1;
};
constexpr int MAX_STAGES = 6;

struct Gemm2Args {
    __nv_bfloat16* y;
    const __nv_bfloat16* shard;
    __nv_bfloat16* gathered;
    unsigned int* flags;
    unsigned int* error;
    unsigned int epoch;
    int M, N, K;
    int shard_rows;
    int gemm_blocks;                 // even; the CTAs after the communication CTAs compute in pairs
    int comm_blocks;                 // even; CTAs [0, comm_blocks) communicate (scheduled first)
    size_t ws_off;                   // staging region inside the workspaces: two halves ...
    size_t ws_half;                  // ... this far apart, selected by the collective counter's parity
    int group;                       // > 1: walk a shard's tiles in bands of this many n-tiles
    int probe;                       // 1: load operands but issue no MMA (measures the ingest rate alone)
};

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of `local` in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t in_cta(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void pair_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\t"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(s32(bar)), "r"(count));
}
__device__ __forceinline__ void bar_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                 :: "r"(s32(bar)), "r"(bytes) : "memory");
}
// One arrival on a barrier given by its address in the cluster window (own or peer CTA).
__device__ __forceinline__ void bar_arrive_cluster(uint32_t addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(addr) : "memory");
}
// Tile load of the pair: the data lands in this CTA, the bytes are counted on `bar` (an
// address in the cluster window: the leader's barrier).
__device__ __forceinline__ void load_tile(void* dst, const CUtensorMap* map, int x, int y,
                                          uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile"
                 ".mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(s32(dst)), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void pair_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 :: "r"(bar) : "memory");
}
__device__ __forceinline__ void pair_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void ld32(uint32_t addr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major tile, 128-byte rows, 128-byte swizzle (see gb_gemm.cu).
__device__ __forceinline__ uint64_t tile_desc(const void* tile) {
    const uint64_t addr = (uint64_t)(s32(tile) >> 4) & 0x3FFFu;
    return addr | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__host__ __device__ constexpr uint32_t pair_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct Tile2 { int m0, n0, shard; };
__device__ __forceinline__ Tile2 tile_of(const Gemm2Args& a, const GbTeam& tm, long t, int BN) {
    const int m_tiles = (a.M + BM - 1) / BM;
    const int n_per_shard = (a.shard_rows + BN - 1) / BN;
    const long per_shard = (long)m_tiles * n_per_shard;
    const int step = (int)(t / per_shard);
    const long rest = t % per_shard;
    Tile2 tile;
    tile.shard = (tm.rank + step) % tm.world;
    if (a.group > 1) {
        // Bands of `group` n-tiles, inside a band m outer and n inner: the pairs that run at the
        // same time then share about sqrt(pairs) tiles of X and of W each instead of reading one
        // tile of W and every tile of X, which keeps both operands in L2.
        const long band_tiles = (long)a.group * m_tiles;
        const int band = (int)(rest / band_tiles);
        const int width = n_per_shard - band * a.group < a.group ? n_per_shard - band * a.group : a.group;
        const long r = rest - (long)band * band_tiles;
        tile.n0 = tile.shard * a.shard_rows + (band * a.group + (int)(r % width)) * BN;
        tile.m0 = (int)(r / width) * BM;
        return tile;
    }
    tile.n0 = tile.shard * a.shard_rows + (int)(rest / m_tiles) * BN;
    tile.m0 = (int)(rest % m_tiles) * BM;
    return tile;
}

template <int NH>
__global__ void __launch_bounds__(THREADS2)
allgather_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x,
                           const __grid_constant__ CUtensorMap map_w, GbTeam tm, Gemm2Args a) {
    constexpr int BN = Shape<NH>::BN, STAGES = Shape<NH>::STAGES, STAGE_BYTES = Shape<NH>::STAGE_BYTES;
    constexpr int ACCS = Shape<NH>::ACCS;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    if ((int)blockIdx.x < a.comm_blocks) {
        // ---- communication CTAs: as in the single-CTA kernel; the lowest indices, so they are
        // resident before the pairs that wait for their flags ---------------------------------
        const int comm_blocks = a.comm_blocks;
        const GbLane L = gb_lane_blocks(0, comm_blocks, tm.ld_mode);
        const size_t shard_bytes = (size_t)a.shard_rows * a.K * 2;
        char* mine = reinterpret_cast<char*>(a.gathered) + (size_t)tm.rank * shard_bytes;
        // the half of the staging region the collective before this one did not use (read
        // before the barrier below advances the counter)
        const size_t stage_off = a.ws_off + (size_t)(gb_ld_volatile(&tm.ctrl->epoch) & 1u) * a.ws_half;
        gb_copy_bytes(L, mine, a.shard, shard_bytes, false);
        if (tm.world > 1) gb_copy_bytes(L, tm.ws[tm.rank] + stage_off, a.shard, shard_bytes, false);
        if (!gb_sync(tm, 0, (unsigned)comm_blocks, 0, true, true)) return;
        if (L.tid == 0) gb_st_release_gpu(a.flags + tm.rank, a.epoch);
        for (int d = 1; d < tm.world; ++d) {
            const int peer = (tm.rank + d) % tm.world;
            gb_copy_bytes(L, reinterpret_cast<char*>(a.gathered) + (size_t)peer * shard_bytes,
                          tm.ws[peer] + stage_off, shard_bytes, true);
            if (!gb_sync(tm, 0, (unsigned)comm_blocks, 1, false, false)) return;
            if (L.tid == 0) gb_st_release_gpu(a.flags + peer, a.epoch);
        }
        gb_sync(tm, 0, (unsigned)comm_blocks, 2, false, true);
        return;
    }
    // ---- GEMM CTA pairs ---------------------------------------------------------------------
    unsigned char* tiles = reinterpret_cast<unsigned char*>(
        ((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + SMEM_TILES);
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* acc_full = empty + MAX_STAGES;      // [2]
    uint64_t* acc_empty = acc_full + 2;           // [2], used on the leader
    uint64_t* drained = acc_empty + 2;            // the issuer's last instructions after a failure
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drained + 1);
    const TcGuard guard = {a.error, &tm.ctrl->abort, tm.timeout_ns};
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cta_rank();             // 0: the pair's leader
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { bar_init(full + s, 1); bar_init(empty + s, 1); }
        for (int b = 0; b < 2; ++b) { bar_init(acc_full + b, 1); bar_init(acc_empty + b, 8); }
        bar_init(drained, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(s32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    pair_sync();                                   // both CTAs' barriers and tensor memory exist
    fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int m_tiles = (a.M + BM - 1) / BM;
    const int n_per_shard = (a.shard_rows + BN - 1) / BN;
    const long total = (long)m_tiles * n_per_shard * tm.world;
    const int k_blocks = (a.K + BK - 1) / BK;
    const long pair = ((int)blockIdx.x - a.comm_blocks) >> 1, pairs = a.gemm_blocks >> 1;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer of this CTA's halves ----
        uint32_t stage = 0, phase = 0;
        int ready_shard = -1;
        bool alive = true;
        for (long t = pair; alive && t < total; t += pairs) {
            const Tile2 tile = tile_of(a, tm, t, BN);
            if (tile.shard != ready_shard) {
                if (!tc_wait_flag(a.flags + tile.shard, a.epoch, guard, 2u)) { alive = false; break; }
                asm volatile("fence.proxy.async.global;" ::: "memory");
                ready_shard = tile.shard;
            }
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(empty + stage, phase ^ 1u, guard, 1u)) { alive = false; break; }
                unsigned char* sa = tiles + stage * STAGE_BYTES;
                const uint32_t leader_full = in_cta(s32(full + stage), 0);
                if (leader) bar_expect(full + stage, 2 * STAGE_BYTES);   // both CTAs' bytes
                load_tile(sa, &map_x, kb * BK, tile.m0 + (int)rank * HALF, leader_full);
                #pragma unroll
                for (int h = 0; h < NH; ++h)                     // this CTA's 128 rows of every half
                    load_tile(sa + A_BYTES + h * B_BYTES, &map_w, kb * BK,
                              tile.n0 + h * 256 + (int)rank * HALF, leader_full);
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        // Loads still in flight after a failure land in this CTA's shared memory and count on
        // the leader's barriers; both CTAs stay until the cluster barrier at the end, which the
        // leader reaches only after its issuer has waited (bounded) for the tensor pipe.
    } else if (warp == 1 && lane == 0 && leader) {
        // ---- MMA issuer of the pair ----
        constexpr uint32_t idesc = pair_idesc(BM, 256);
        uint32_t stage = 0, phase = 0, local = 0;
        bool alive = true;
        for (long t = pair; alive && t < total; t += pairs, ++local) {
            const uint32_t buf = ACCS == 2 ? (local & 1u) : 0u, use = ACCS == 2 ? (local >> 1) : local;
            // both epilogues drained it
            if (!mbar_wait(acc_empty + buf, (use & 1u) ^ 1u, guard, 3u)) { alive = false; break; }
            fence_after();
            const uint32_t tmem_d = tmem_base + buf * 256;
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(full + stage, phase, guard, 4u)) { alive = false; break; }
                fence_after();
                const unsigned char* sa = tiles + stage * STAGE_BYTES;
                const uint64_t da = tile_desc(sa);
                if (!a.probe) {
                    #pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        const uint64_t db = tile_desc(sa + A_BYTES + h * B_BYTES);
                        #pragma unroll
                        for (int kk = 0; kk < BK / 16; ++kk)
                            pair_mma(tmem_d + h * 256, da + 2 * kk, db + 2 * kk, idesc,
                                     (kb | kk) != 0 ? 1u : 0u);
                    }
                }
                pair_commit(s32(empty + stage));                       // frees the stage here ...
                pair_commit(in_cta(s32(empty + stage), 1));            // ... and in the peer
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (alive) {
                pair_commit(s32(acc_full + buf));
                pair_commit(in_cta(s32(acc_full + buf), 1));
            }
        }
        if (!alive) {
            // nothing of the pair's earlier instructions may be in flight when tensor memory goes
            pair_commit(s32(drained));
            const unsigned long long t0 = tc_now();
            for (unsigned spins = 0; spins < (1u << 20); ++spins) {
                if (mbar_try_wait(drained, 0u)) break;
                if ((spins & 31u) == 31u && tc_now() - t0 > 2000000ull) break;      // 2 ms
            }
        }
    } else if (warp >= 2) {
        // ---- epilogue of this CTA's 128 rows ----
        const int quarter = warp & 3;
        uint32_t local = 0;
        for (long t = pair; t < total; t += pairs, ++local) {
            const Tile2 tile = tile_of(a, tm, t, BN);
            const uint32_t buf = ACCS == 2 ? (local & 1u) : 0u, use = ACCS == 2 ? (local >> 1) : local;
            if (!mbar_wait_warp(acc_full + buf, use & 1u, guard, 5u)) break;
            fence_after();
            const int row = tile.m0 + (int)rank * HALF + quarter * 32 + lane;
            const int shard_end = (tile.shard + 1) * a.shard_rows;
            #pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * 256 + c, r);
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
            fence_before();
            __syncwarp();
            if (lane == 0) bar_arrive_cluster(in_cta(s32(acc_empty + buf), 0));
        }
    }
    fence_before();
    __syncthreads();
    pair_sync();                                   // nobody leaves while the peer still computes
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                     :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
}

typedef CUresult (*EncodeTiled2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                 const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool make_map2(CUtensorMap* map, const void* base, int rows, int K) {
    static EncodeTiled2 encode = nullptr;
    if (encode == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) !=
                cudaSuccess || status != cudaDriverEntryPointSuccess)
            return false;
        encode = reinterpret_cast<EncodeTiled2>(ptr);
    }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)HALF};
    cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
           CUDA_SUCCESS;
}

}  // namespace

// Same contract as gb_allgather_gemm; gemm_blocks and comm_blocks must be even (the grid is
// launched as clusters of two CTAs).
extern "C" int gb_allgather_gemm_pair(const GbTeam* team, void* y, const void* x, const void* shard,
                                      void* gathered, unsigned int* flags, unsigned int* error,
                                      unsigned int epoch, int M, int N, int K, size_t ws_off,
                                      size_t ws_half, int gemm_blocks, int comm_blocks, cudaStream_t stream) {
    // tuning switches for measurements: the tile walk and the operand-ingest probe
    static const int tile_group = []{ const char* v = getenv("GPUBRIDGE_GEMM_GROUP"); return v ? atoi(v) : 8; }();
    static const int ingest_probe = []{ const char* v = getenv("GPUBRIDGE_GEMM_PROBE"); return v ? atoi(v) : 0; }();
    if (M <= 0 || N <= 0 || K <= 0 || (K & 7) || N % team->world || gemm_blocks < 2 ||
        comm_blocks < 2 || (gemm_blocks & 1) || (comm_blocks & 1))
        return (int)cudaErrorInvalidValue;
    CUtensorMap map_x, map_w;
    if (!make_map2(&map_x, x, M, K) || !make_map2(&map_w, gathered, N, K)) return -3;
    Gemm2Args a;
    a.y = static_cast<__nv_bfloat16*>(y);
    a.shard = static_cast<const __nv_bfloat16*>(shard);
    a.gathered = static_cast<__nv_bfloat16*>(gathered);
    a.flags = flags; a.error = error; a.epoch = epoch;
    a.M = M; a.N = N; a.K = K;
    a.shard_rows = N / team->world;
    a.ws_off = ws_off;
    a.ws_half = ws_half;
    a.group = tile_group;
    a.probe = ingest_probe;
    const size_t smem = SMEM_TILES + 256 + 1024;
    // 256 x 512 tiles have one accumulator, so their epilogue does not overlap the next tile's
    // products: they pay off for a long K only (measured: 8192 wins, 2048 and 4096 lose).
    // GPUBRIDGE_GEMM_WIDE: 1 = always wide, 0 = always 256 x 256 with two accumulators, unset = by K
    static const int wide_choice = []{ const char* v = getenv("GPUBRIDGE_GEMM_WIDE"); return v ? atoi(v) : -1; }();
    const int wide = wide_choice >= 0 ? (wide_choice != 0) : (K >= 8192 && N % 512 == 0);
    typedef void (*Kernel)(const CUtensorMap, const CUtensorMap, GbTeam, Gemm2Args);
    Kernel kernel = wide ? allgather_gemm_pair_kernel<2> : allgather_gemm_pair_kernel<1>;
    static bool configured[2] = {false, false};
    static int resident[2] = {0, 0};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    if (!configured[wide]) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
        // every CTA must be resident at once (pairs wait for the communication CTAs' flags)
        cudaLaunchConfig_t probe = {};
        probe.gridDim = dim3(2); probe.blockDim = dim3(THREADS2); probe.dynamicSmemBytes = smem;
        probe.attrs = attr; probe.numAttrs = 1;
        err = cudaOccupancyMaxActiveClusters(&resident[wide], kernel, &probe);
        if (err != cudaSuccess) return (int)err;
        configured[wide] = true;
    }
    const int resident_clusters = resident[wide];
    if (gemm_blocks + comm_blocks > 2 * resident_clusters) gemm_blocks = 2 * resident_clusters - comm_blocks;
    if (gemm_blocks < 2) return (int)cudaErrorInvalidConfiguration;
    a.gemm_blocks = gemm_blocks;
    a.comm_blocks = comm_blocks;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)(gemm_blocks + comm_blocks));
    config.blockDim = dim3(THREADS2);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    config.attrs = attr;
    config.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&config, kernel, map_x, map_w, *team, a);
}

GB_BOUNDS_HOST(gemm2)
