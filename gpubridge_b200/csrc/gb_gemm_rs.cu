// A tcgen05 GEMM whose epilogue is the first half of a reduce-scatter:
//     out[rows of this rank, Q] = (1 / divide) * sum over ranks s of  A_s[P, R] * B_s[Q, R]^T
// with the P rows of the product owned in equal blocks by the ranks of the team - the weight
// gradient of a row-sharded Linear, dW = dY^T X (P = out_features, Q = in_features, R = tokens),
// averaged over the data-parallel ranks and left sharded.  It replaces "GEMM, then
// reduce_scatter_tensor, then div_" (reference: the reduce-scatter of
// src/gpubridge/policies.py:409-429 plus collectives.py:218).
//
// One persistent kernel.  The GEMM part is the main loop of the all-gather GEMM (gb_gemm.cu):
// warp 0 feeds a 4-stage shared-memory ring with TMA, warp 1 issues tcgen05.mma into one of two
// accumulators in tensor memory, warps 2-5 drain the other one.  What differs is where a drained
// tile goes: every row of the product belongs to one rank, and the epilogue stores the row's
// values - rounded to bf16, the precision a bf16 reduce-scatter exchanges - straight into that
// rank's workspace over NVLink, into the slot of the sending rank.  Tiles are walked starting
// behind this rank's own rows, so every remote tile's transfer overlaps the math of the tiles
// that follow and the own rows, which travel nowhere, come last.  Then the team meets (grid
// barrier + peer barrier, bounded), and every rank adds the slots of its rows in rank order in
// fp32, divides, rounds once and writes its shard.
//
// Workspace: [2 parities][world slots][rows_per_rank * Q] bf16 inside the team's workspaces; the
// parity is the team's collective counter's, as for every region written before a kernel's
// first barrier, and the two parities are the two halves of the region whatever the shapes - the
// same halves the reduce-scatter kernel uses when it shares the region, so a collective never
// writes where a slow peer may still read the one before it.  Every wait has a deadline (the
// team's wait limit) and ends early once the error word or the team's abort word is set; the
// role then leaves its tile loop, tensor memory is freed and the kernel returns.
#include "gb_common.cuh"
#include "gb_tc_tile.cuh"

namespace {

struct RsArgs {
    void* out;                       // [rows_per_rank, Q], bf16 or fp32
    unsigned int* error;             // set when an mbarrier wait ran out
    int P, Q, R;
    int rows_per_rank;               // P / world
    int divide;                      // > 0: divide the sum by it
    int out_fp32;                    // element type of `out`
    size_t ws_off;                   // start of the region inside the workspaces
    size_t slot_bytes;               // rows_per_rank * Q * 2
    size_t half_bytes;               // distance between the two parities of the region
};

// Tile t of the schedule: row tiles start at the first one that lies wholly behind this rank's
// rows and wrap around; inside a row tile the column tiles.
struct RsTile { int p0, q0; };
__device__ __forceinline__ RsTile rs_tile_at(const RsArgs& a, const GbTeam& tm, long t, int p_tiles,
                                             int q_tiles) {
    const int first = (int)((((long)(tm.rank + 1) * a.rows_per_rank + BM - 1) / BM) % p_tiles);
    RsTile tile;
    tile.p0 = (int)((first + t / q_tiles) % p_tiles) * BM;
    tile.q0 = (int)(t % q_tiles) * BN;
    return tile;
}

__global__ void __launch_bounds__(GEMM_THREADS)
gemm_reduce_scatter_kernel(const __grid_constant__ CUtensorMap map_a,
                           const __grid_constant__ CUtensorMap map_b, GbTeam tm, RsArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the half of the region this collective writes (read before the barrier below advances it)
    const unsigned parity = gb_ld_volatile(&tm.ctrl->epoch) & 1u;
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

    const int p_tiles = (a.P + BM - 1) / BM, q_tiles = (a.Q + BN - 1) / BN;
    const long total = (long)p_tiles * q_tiles;
    const int k_blocks = (a.R + BK - 1) / BK;
    const long stride = (long)gridDim.x;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        uint32_t stage = 0, phase = 0, issued = 0;
        bool alive = true;
        for (long t = blockIdx.x; alive && t < total; t += stride) {
            const RsTile tile = rs_tile_at(a, tm, t, p_tiles, q_tiles);
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(empty + stage, phase ^ 1u, guard, 1u)) { alive = false; break; }
                unsigned char* sa = tiles + stage * STAGE_BYTES;
                mbar_expect_tx(full + stage, STAGE_BYTES);
                tma_load_2d(sa, &map_a, kb * BK, tile.p0, full + stage);
                tma_load_2d(sa + A_BYTES, &map_b, kb * BK, tile.q0, full + stage);
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
        for (long t = blockIdx.x; alive && t < total; t += stride, ++local) {
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
                for (int kk = 0; kk < BK / 16; ++kk)           // 32 bytes along the contraction per step
                    tc_mma(tmem_d, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
                tc_commit(empty + stage);                      // frees the stage when they finish
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (alive) tc_commit(acc_full + buf);
        }
        if (!alive) tc_drain_mma(drained);
    } else if (warp >= 2) {
        // ---- epilogue: tensor memory -> registers -> bf16 -> the row owner's workspace ----
        const int quarter = warp & 3;                          // the lanes this warp may read
        const size_t half = a.half_bytes;                      // one parity of the region
        uint32_t local = 0;
        for (long t = blockIdx.x; t < total; t += stride, ++local) {
            const RsTile tile = rs_tile_at(a, tm, t, p_tiles, q_tiles);
            const uint32_t buf = local & 1u, use = local >> 1;
            if (!mbar_wait_warp(acc_full + buf, use & 1u, guard, 5u)) break;
            tc_fence_after();
            const int row = tile.p0 + quarter * 32 + lane;
            const bool live = row < a.P;
            const int owner = live ? row / a.rows_per_rank : 0;
            const int at = live ? row - owner * a.rows_per_rank : 0;
            __nv_bfloat16* slot_row = reinterpret_cast<__nv_bfloat16*>(
                tm.ws[owner] + a.ws_off + (size_t)parity * half + (size_t)tm.rank * a.slot_bytes)
                + (size_t)at * a.Q;
            #pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + c, r);
                const int col = tile.q0 + c;
                if (live && col < a.Q) {
                    __nv_bfloat16* dst = slot_row + col;       // 16-byte aligned: Q and col are multiples of 8
                    if (col + 32 <= a.Q) {
                        #pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            uint4 out;
                            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
                            #pragma unroll
                            for (int j = 0; j < 4; ++j)
                                h[j] = __floats2bfloat162_rn(__uint_as_float(r[8 * g + 2 * j]),
                                                             __uint_as_float(r[8 * g + 2 * j + 1]));
                            gb_st16(dst + 8 * g, out);
                        }
                    } else {
                        for (int j = 0; j < 32 && col + j < a.Q; ++j)
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

    // ---- every rank's partial rows have been sent: meet, then add the slots of the own rows ----
    // A block whose GEMM part gave up raises the team's abort word first, so that the barrier
    // below ends at once on this rank and the peers' waits for it run into their deadline with
    // a status record instead of adding slots that were never filled.
    if (threadIdx.x == 0 && gb_ld_volatile(a.error) != 0u) gb_fail(tm, GB_TIMEOUT_TENSOR, 0u, 0u, 0u);
    if (!gb_sync_all(tm, 0, true)) return;
    const char* slots = tm.ws[tm.rank] + a.ws_off + (size_t)parity * a.half_bytes;
    const size_t nvec = a.slot_bytes >> 4;                     // vectors of eight bf16 values
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nth = (size_t)gridDim.x * blockDim.x;
    for (size_t v = tid; v < nvec; v += nth) {
        float acc[8];
        #pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
        for (int s = 0; s < tm.world; ++s) {                   // rank order: the same sum whoever asks
            const uint4 w = gb_ld16(slots + (size_t)s * a.slot_bytes + (v << 4), tm.ld_mode);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h[j]);
                acc[2 * j] = __fadd_rn(acc[2 * j], f.x);
                acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], f.y);
            }
        }
        if (a.divide > 0) {
            #pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = gb_divide<float>(acc[j], a.divide);
        }
        if (a.out_fp32) {
            float4* dst = reinterpret_cast<float4*>(static_cast<float*>(a.out) + (v << 3));
            dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
        } else {
            uint4 out;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
            #pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.out) + (v << 3)) = out;
        }
    }
}

}  // namespace

// Bytes of workspace the kernel needs at `ws_off` for these shapes (both halves).
extern "C" size_t gb_gemm_reduce_scatter_bytes(int world, int P, int Q) {
    if (world < 1 || P <= 0 || Q <= 0 || P % world) return 0;
    return (size_t)2 * world * ((size_t)(P / world) * Q * 2);
}

// out[P / world, Q] = (1 / divide) * sum over the team of a[P, R] * b[Q, R]^T, rows of the
// product owned in equal blocks by the team's ranks.  a, b: bf16, row-major, 16-byte aligned;
// R and Q multiples of 8; out: bf16 (out_fp32 = 0) or fp32, 16-byte aligned.  The region
// [ws_off, ws_off + ws_len) of every rank's workspace is the staging area (ws_off a multiple of
// 16).  blocks <= 0: one block per SM that can hold one.  Returns a cudaError_t, -3 when the
// tensor maps could not be built, -4 when the staging area is too small.
extern "C" int gb_gemm_reduce_scatter(const GbTeam* team, void* out, const void* a, const void* b,
                                      unsigned int* error, int P, int Q, int R, size_t ws_off,
                                      size_t ws_len, int divide, int out_fp32, int blocks,
                                      cudaStream_t stream) {
    if (P <= 0 || Q <= 0 || R <= 0 || (R & 7) || (Q & 7) || P % team->world || (ws_off & 15))
        return (int)cudaErrorInvalidValue;
    const size_t need = gb_gemm_reduce_scatter_bytes(team->world, P, Q);
    const size_t half = (ws_len / 2) & ~(size_t)15;
    if (need == 0 || need / 2 > half) return -4;
    CUtensorMap map_a, map_b;
    if (!make_map(&map_a, a, P, R, BM) || !make_map(&map_b, b, Q, R, BN)) return -3;
    RsArgs args;
    args.out = out;
    args.error = error;
    args.P = P; args.Q = Q; args.R = R;
    args.rows_per_rank = P / team->world;
    args.divide = divide;
    args.out_fp32 = out_fp32;
    args.ws_off = ws_off;
    args.slot_bytes = (size_t)args.rows_per_rank * Q * 2;
    args.half_bytes = half;
    const size_t smem = STAGES * STAGE_BYTES + 256 + 1024;
    static int resident = 0;                       // blocks the device holds at once (the grid barrier needs all)
    if (resident == 0) {
        cudaError_t err = cudaFuncSetAttribute(gemm_reduce_scatter_kernel,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
        int device = 0, sms = 0, per_sm = 0;
        if ((err = cudaGetDevice(&device)) != cudaSuccess) return (int)err;
        if ((err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess)
            return (int)err;
        if ((err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_reduce_scatter_kernel,
                                                                 GEMM_THREADS, smem)) != cudaSuccess)
            return (int)err;
        if (per_sm < 1) return (int)cudaErrorLaunchOutOfResources;
        resident = sms;                            // one block per SM: each takes all of its tensor memory
    }
    const long tiles = (long)((P + BM - 1) / BM) * ((Q + BN - 1) / BN);
    int grid = blocks > 0 && blocks < resident ? blocks : resident;
    if ((long)grid > tiles) grid = (int)tiles;
    gemm_reduce_scatter_kernel<<<grid, GEMM_THREADS, smem, stream>>>(map_a, map_b, *team, args);
    return (int)cudaGetLastError();
}

GB_BOUNDS_HOST(gemm_rs)
