// All-reduce through the NVSwitch (NVLS) with block-level barriers: SUM / AVG of f32, bf16, f16.
//
// Every rank owns staging memory bound to a multicast object of its group (gb_mcast.cu).  A
// multimem.ld_reduce on the group's multicast address returns the sum over the group, computed
// inside the switch; a multimem.st writes every member's copy at once.  A GPU then sends and
// receives about 9/8 of the tensor instead of the 14/8 of a reduce-scatter + all-gather over
// peer memory, and the adding costs no SM time.
//
// The tensor is cut into tiles; tile j belongs to block j mod B of EVERY rank (all ranks launch
// the same grid).  A block works through its tiles as a software pipeline over `depth` staging
// buffers of its own, with ONE barrier per step - and that barrier joins only the blocks of the
// same index on the other ranks (a flag row per block in the peers' workspaces), never the
// grid.  Blocks therefore drift apart and the steps of different blocks overlap: while some
// copy, others have their requests in the switch.  Inside a block the first half of the warps
// does the local copies and the second half the switch step, side by side.
//
// One group (a team of one island, or the flat mode of a team of several), depth 3; step i:
//     A  copy tile i from the input into the own staging buffer              (local)
//     B  member p: ld_reduce stripe p of tile i-1, divide for AVG, multimem.st it back   (switch)
//     C  copy tile i-2 from the own staging buffer to the output             (local)
// Several islands (hierarchical order: island sums first, rounded to the tensor's type, then
// the islands in island order), the group is the island, depth 4; step i:
//     A  copy tile i in
//     B  owner p: ld_reduce stripe p of tile i-1 over the island and store the island sum into a
//        slot of owner p of every island                                     (switch + NVLink)
//     C  owner p: add the islands' slots of tile i-2 in island order, divide, multimem.st to the
//        island                                                              (switch)
//     D  copy tile i-3 out
// Owners: positions 0 .. k-1 of every island, k the size of the smallest island.
//
// Why the buffers do not collide: a buffer is rewritten `depth` steps after it was first
// written, and every barrier in between needs every member's arrival, so nobody is ever more
// than one step ahead of the slowest member; the proof by cases is the CPU model in
// tests/test_switch_model.py.  Every element is reduced by exactly one rank and then
// multicast, so all ranks end with identical bits; the order of the addends inside a group is
// the switch's, and integer-valued data is exact.
//
// Every wait is bounded (gb_wait_flag: spin limit + globaltimer deadline); on expiry the block
// records the failure in the team's status block, raises the abort word and returns.
#include <stdlib.h>

#include "gb_common.cuh"
#include "gb_switch.h"

extern "C" int gb_switch_plan_copy(const GbSwitch* sw, int nsub, size_t piece, int max_blocks,
                                   GbSwitchPlan* plan);

namespace {

// Two launch shapes: 512 threads (one block per SM) with four switch requests in flight per
// thread, or 256 threads (two blocks per SM, so one block's barrier wait is covered by the
// other's work) with eight.  GPUBRIDGE_SWITCH_SHAPE picks; the default is the second.
constexpr int SW_MAX_THREADS = 512;

template <typename T> struct SwVec {
    static constexpr int N = 16 / sizeof(T);
    union { uint4 u; T e[16 / sizeof(T)]; };
};

template <typename T> struct SwitchSum;
template <> struct SwitchSum<float> {
    static __device__ __forceinline__ uint4 load(const char* mc) {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
        return v;
    }
};
template <> struct SwitchSum<__nv_bfloat16> {
    static __device__ __forceinline__ uint4 load(const char* mc) {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
        return v;
    }
};
template <> struct SwitchSum<__half> {
    static __device__ __forceinline__ uint4 load(const char* mc) {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
        return v;
    }
};
__device__ __forceinline__ void switch_store(char* mc, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
                 :: "l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ size_t sw_round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }

// Barrier of block `b` with the blocks `b` of every other rank of the team.  Row b of the flag
// area of rank q holds, at index r, the last step rank r's block b announced to q.
__device__ __forceinline__ bool sw_block_sync(const GbTeam& tm, const GbSwitch& sw, int b,
                                              unsigned seq) {
    __syncthreads();                                      // this block's stores are issued
    const int q = (int)threadIdx.x;
    if (q < tm.world && q != tm.rank) {
        __threadfence_system();                           // ... and ordered before the flag, everywhere
        unsigned* theirs = reinterpret_cast<unsigned*>(tm.ws[q] + sw.off_flags) +
                           (size_t)b * GB_MAX_RANKS + tm.rank;
        gb_st_release_sys(theirs, seq);
        const unsigned* mine = reinterpret_cast<const unsigned*>(tm.ws[tm.rank] + sw.off_flags) +
                               (size_t)b * GB_MAX_RANKS + q;
        if (!gb_wait_flag(tm, mine, seq, true, tm.timeout_ns))
            gb_fail(tm, GB_TIMEOUT_PEER, (unsigned)q, seq, 8u + (unsigned)(b & 7));
    }
    __syncthreads();
    return gb_ld_volatile(&tm.ctrl->abort) == 0u;
}

struct SwTile { size_t off, len, padded; };
__device__ __forceinline__ SwTile sw_tile(const SwArgs& a, int owners, int b, int B, int i) {
    SwTile t;
    t.off = ((size_t)i * B + b) * a.tile;
    t.len = a.nbytes - t.off < a.tile ? a.nbytes - t.off : a.tile;
    t.padded = sw_round_up(t.len, 16 * (size_t)owners);      // stripes are whole 16-byte vectors
    return t;
}

// Zero [lo, hi) of a staging buffer (hi - lo < 16 * owners): the padding of a short last tile.
__device__ __forceinline__ void sw_zero(char* base, size_t lo, size_t hi, int tid, int nth) {
    for (size_t x = lo + tid; x < hi; x += nth) base[x] = 0;
}

template <typename T, bool HIER, int SW_THREADS, int U>
__global__ void __launch_bounds__(SW_THREADS, SW_MAX_THREADS / SW_THREADS)
allreduce_switch_kernel(GbTeam tm, GbSwitch sw, SwArgs a) {
    typedef typename GbAcc<T>::type A;
    constexpr int V = SwVec<T>::N;
    constexpr int DEPTH = HIER ? 4 : 3;
    constexpr int SW_HALF = SW_THREADS / 2;                    // U: switch requests in flight per thread
    const int b = (int)blockIdx.x, B = (int)gridDim.x;
    const int mine = (a.ntiles - b + B - 1) / B;               // tiles b, b + B, ... (b < ntiles)
    const int steps = mine + DEPTH - 1;
    unsigned seq = gb_ld_volatile(sw.bseq + b);
    char* stage = sw.uc + (size_t)b * DEPTH * a.tile;          // this block's buffers, local address
    char* stage_mc = sw.mc + (size_t)b * DEPTH * a.tile;       // the same buffers on the whole group
    const int owners = sw.owners;
    const bool owner = sw.group_pos < owners;
    const bool copier = (int)threadIdx.x < SW_HALF;
    const int tid = (int)threadIdx.x - (copier ? 0 : SW_HALF);
    GbLane L;
    L.tid = (size_t)tid; L.nth = SW_HALF; L.ld = tm.ld_mode;
    // the bridge slots of this block: [2 parities][islands] of one stripe each
    const size_t slot = a.tile / (size_t)owners;
    const size_t bridge0 = sw.off_bridge + (size_t)b * 2 * tm.n_islands * slot;

    for (int i = 0; i < steps; ++i) {
        if (copier) {
            if (i < mine) {                                                   // A
                const SwTile t = sw_tile(a, owners, b, B, i);
                char* dst = stage + (size_t)(i % DEPTH) * a.tile;
                gb_copy_bytes(L, dst, a.in + t.off, t.len, false);
                sw_zero(dst, t.len, t.padded, tid, SW_HALF);
            }
            const int c = i - (DEPTH - 1);
            if (c >= 0) {                                                     // C (D when HIER)
                const SwTile t = sw_tile(a, owners, b, B, c);
                gb_copy_bytes(L, a.out + t.off, stage + (size_t)(c % DEPTH) * a.tile, t.len, true);
            }
        } else if (owner) {
            const int r = i - 1;
            if (r >= 0 && r < mine) {                                         // B
                const SwTile t = sw_tile(a, owners, b, B, r);
                const size_t stripe = t.padded / (size_t)owners;
                const size_t s0 = (size_t)(r % DEPTH) * a.tile + (size_t)sw.group_pos * stripe;
                const size_t nvec = stripe >> 4;
                for (size_t v0 = (size_t)tid; v0 < nvec; v0 += (size_t)U * SW_HALF) {
                    SwVec<T> w[U];
                    #pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const size_t v = v0 + (size_t)u * SW_HALF;
                        if (v < nvec) w[u].u = SwitchSum<T>::load(stage_mc + s0 + (v << 4));
                    }
                    #pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const size_t v = v0 + (size_t)u * SW_HALF;
                        if (v >= nvec) continue;
                        if (!HIER) {
                            if (a.divide > 0) {
                                #pragma unroll
                                for (int j = 0; j < V; ++j)
                                    w[u].e[j] = gb_down<T>(gb_divide<A>(gb_up<T>(w[u].e[j]), a.divide));
                            }
                            switch_store(stage_mc + s0 + (v << 4), w[u].u);
                        } else {
                            // the island's sum of this stripe goes to owner p of every island
                            const size_t at = bridge0 + ((size_t)(r & 1) * tm.n_islands + tm.my_island) * slot
                                              + (v << 4);
                            for (int g = 0; g < tm.n_islands; ++g) {
                                const int peer = tm.order[tm.island_off[g] + sw.group_pos];
                                gb_st16(tm.ws[peer] + at, w[u].u);
                            }
                        }
                    }
                }
            }
            const int s = i - 2;
            if (HIER && s >= 0 && s < mine) {                                 // C
                const SwTile t = sw_tile(a, owners, b, B, s);
                const size_t stripe = t.padded / (size_t)owners;
                const size_t s0 = (size_t)(s % DEPTH) * a.tile + (size_t)sw.group_pos * stripe;
                const size_t nvec = stripe >> 4;
                const char* slots = tm.ws[tm.rank] + bridge0 + (size_t)(s & 1) * tm.n_islands * slot;
                for (size_t v = (size_t)tid; v < nvec; v += SW_HALF) {
                    A acc[V];
                    for (int g = 0; g < tm.n_islands; ++g) {                   // island order
                        SwVec<T> w;
                        w.u = gb_ld16(slots + (size_t)g * slot + (v << 4), tm.ld_mode);
                        #pragma unroll
                        for (int j = 0; j < V; ++j)
                            acc[j] = g == 0 ? gb_up<T>(w.e[j]) : acc[j] + gb_up<T>(w.e[j]);
                    }
                    SwVec<T> out;
                    #pragma unroll
                    for (int j = 0; j < V; ++j)
                        out.e[j] = gb_down<T>(a.divide > 0 ? gb_divide<A>(acc[j], a.divide) : acc[j]);
                    switch_store(stage_mc + s0 + (v << 4), out.u);
                }
            }
        }
        if (i + 1 < steps && !sw_block_sync(tm, sw, b, ++seq)) return;
        if (b == 0 && threadIdx.x == 0 && i == 0) tm.ctrl->stamps[0] = gb_now();   // first tiles staged
    }
    if (threadIdx.x == 0) {
        sw.bseq[b] = seq;
        if (b == 0) tm.ctrl->stamps[1] = gb_now();             // block 0's last tile is out
    }
}

// In place, for a tensor that lives IN the group's switch memory at the same offset on every
// rank (Fabric.switch_empty hands such tensors out; a trainer keeps its gradients there): no
// staging and no copies.  Block b owns tiles b, b + B, ... of the tensor; it meets the same
// block of every rank once (every rank's values are written), reduces its rank's share of
// each of its tiles in the switch and multicasts the result back in place, and meets them
// again (every share is written) before anybody reads.  One group, flat order.
template <typename T, int SW_THREADS, int U>
__global__ void __launch_bounds__(SW_THREADS, SW_MAX_THREADS / SW_THREADS)
allreduce_switch_inplace_kernel(GbTeam tm, GbSwitch sw, SwArgs a, size_t offset) {
    typedef typename GbAcc<T>::type A;
    constexpr int V = SwVec<T>::N;
    const int b = (int)blockIdx.x, B = (int)gridDim.x;
    unsigned seq = gb_ld_volatile(sw.bseq + b);
    if (!sw_block_sync(tm, sw, b, ++seq)) return;
    char* everyone = sw.mc + offset;
    for (int i = b; i < a.ntiles; i += B) {
        const size_t t0 = (size_t)i * a.tile;
        const size_t len = a.nbytes - t0 < a.tile ? a.nbytes - t0 : a.tile;      // a multiple of 16
        const size_t nvec = len >> 4;
        const size_t share = (nvec + (size_t)sw.owners - 1) / (size_t)sw.owners;
        const size_t lo = (size_t)sw.group_pos * share;
        const size_t hi = lo + share < nvec ? lo + share : nvec;
        for (size_t v0 = lo + threadIdx.x; v0 < hi; v0 += (size_t)U * SW_THREADS) {
            SwVec<T> w[U];
            #pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t v = v0 + (size_t)u * SW_THREADS;
                if (v < hi) w[u].u = SwitchSum<T>::load(everyone + t0 + (v << 4));
            }
            #pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t v = v0 + (size_t)u * SW_THREADS;
                if (v >= hi) continue;
                if (a.divide > 0) {
                    #pragma unroll
                    for (int j = 0; j < V; ++j)
                        w[u].e[j] = gb_down<T>(gb_divide<A>(gb_up<T>(w[u].e[j]), a.divide));
                }
                switch_store(everyone + t0 + (v << 4), w[u].u);
            }
        }
    }
    if (!sw_block_sync(tm, sw, b, ++seq)) return;
    if (threadIdx.x == 0) sw.bseq[b] = seq;
}

int switch_shape() {
    static const int shape = []{ const char* v = getenv("GPUBRIDGE_SWITCH_SHAPE"); return v ? atoi(v) : 1; }();
    return shape;
}

template <typename T>
cudaError_t launch_switch(const GbTeam& tm, const GbSwitch& sw, const SwArgs& a, int grid,
                          cudaStream_t stream) {
    if (switch_shape() == 0) {
        if (sw.hier) allreduce_switch_kernel<T, true, 512, 4><<<grid, 512, 0, stream>>>(tm, sw, a);
        else allreduce_switch_kernel<T, false, 512, 4><<<grid, 512, 0, stream>>>(tm, sw, a);
    } else {
        if (sw.hier) allreduce_switch_kernel<T, true, 256, 8><<<grid, 256, 0, stream>>>(tm, sw, a);
        else allreduce_switch_kernel<T, false, 256, 8><<<grid, 256, 0, stream>>>(tm, sw, a);
    }
    return cudaGetLastError();
}

template <typename T>
cudaError_t launch_inplace(const GbTeam& tm, const GbSwitch& sw, const SwArgs& a, size_t offset, int grid,
                           cudaStream_t stream) {
    if (switch_shape() == 0) allreduce_switch_inplace_kernel<T, 512, 4><<<grid, 512, 0, stream>>>(tm, sw, a, offset);
    else allreduce_switch_inplace_kernel<T, 256, 8><<<grid, 256, 0, stream>>>(tm, sw, a, offset);
    return cudaGetLastError();
}


// ---- all-reduce in one step, for small and medium tensors -------------------------------------------
//
// Block b copies its tile of the input into ITS slot of the reserved tail of the switch memory,
// meets block b of every other rank once, and then ld_reduces the whole tile - not a share of
// it - straight into the output: one barrier instead of two, no copy out, at the price of every
// rank pulling every byte through the switch (n times the traffic of the two-step form, which
// is why this is for a few MiB at most).  Every rank adds the same values in the switch's order,
// so all ranks still end with identical bits.
// A slot has two halves; a block uses half (its barrier number & 1).  Two calls in a row
// therefore use different halves, and by the time a half comes round again the block has been
// through a barrier that every peer joined after finishing the earlier call - so nobody still
// reads what is overwritten.  Any other kernel in between only adds barriers.  The slots are
// per block index and fixed in place, whatever the tile size of a call.
template <typename T, int SW_THREADS, int U>
__global__ void __launch_bounds__(SW_THREADS, SW_MAX_THREADS / SW_THREADS)
allreduce_switch_oneshot_kernel(GbTeam tm, GbSwitch sw, SwArgs a) {
    typedef typename GbAcc<T>::type A;
    constexpr int V = SwVec<T>::N;
    const int b = (int)blockIdx.x;
    unsigned seq = gb_ld_volatile(sw.bseq + b) + 1u;
    const size_t slot = sw.bytes + (size_t)(seq & 1u) * GB_SWITCH_ONESHOT_SLOT * GB_SWITCH_ONESHOT_BLOCKS +
                        (size_t)b * GB_SWITCH_ONESHOT_SLOT;
    char* mine = sw.uc + slot;
    const char* everyone = sw.mc + slot;
    const size_t off = (size_t)b * a.tile;
    const size_t len = a.nbytes - off < a.tile ? a.nbytes - off : a.tile;
    const size_t padded = sw_round_up(len, 16);
    GbLane whole;
    whole.tid = threadIdx.x; whole.nth = SW_THREADS; whole.ld = tm.ld_mode;
    gb_copy_bytes(whole, mine, a.in + off, len, false);
    sw_zero(mine, len, padded, (int)threadIdx.x, SW_THREADS);
    if (!sw_block_sync(tm, sw, b, seq)) return;
    if (b == 0 && threadIdx.x == 0) tm.ctrl->stamps[0] = gb_now();
    char* out = a.out + off;
    const bool aligned = (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
    const size_t nvec = padded >> 4;
    for (size_t v0 = threadIdx.x; v0 < nvec; v0 += (size_t)U * SW_THREADS) {
        SwVec<T> w[U];
        #pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t v = v0 + (size_t)u * SW_THREADS;
            if (v < nvec) w[u].u = SwitchSum<T>::load(everyone + (v << 4));
        }
        #pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t v = v0 + (size_t)u * SW_THREADS;
            if (v >= nvec) continue;
            if (a.divide > 0) {
                #pragma unroll
                for (int j = 0; j < V; ++j)
                    w[u].e[j] = gb_down<T>(gb_divide<A>(gb_up<T>(w[u].e[j]), a.divide));
            }
            if (aligned && ((v + 1) << 4) <= len) {
                gb_st16(out + (v << 4), w[u].u);
            } else {                                                   // a ragged end or an odd address
                const unsigned char* bytes = reinterpret_cast<const unsigned char*>(&w[u].u);
                for (size_t j = 0; j < 16 && (v << 4) + j < len; ++j) out[(v << 4) + j] = (char)bytes[j];
            }
        }
    }
    if (threadIdx.x == 0) {
        sw.bseq[b] = seq;
        if (b == 0) tm.ctrl->stamps[1] = gb_now();
    }
}

// ---- reduce-scatter, all-gather and broadcast through the switch -----------------------------------
//
// The same staging memory, block-level barriers and tile ownership as the all-reduce (one group:
// the team), depth 3, every step ends with the barrier - the last one too, so that when a block
// leaves nobody reads or writes its staging buffers any more and the next kernel may start with
// a remote write.  A staging buffer holds `nsub` sub-tiles, one per member's piece.
//   reduce-scatter  A  copy tile i of every member's piece of the input into the own buffer (local)
//                   B  ld_reduce the own piece's sub-tile of tile i-1 over the team, divide for AVG,
//                      store it straight into the output                       (switch; no copy out)
//   all-gather      A  multimem.st tile i of the own input into the own sub-tile of every
//                      member's buffer                                          (switch; no copy in)
//                   B  copy every sub-tile of tile i-1 from the own buffer to the output   (local)
//   broadcast       A  root: multimem.st tile i of the tensor into every member's buffer
//                   B  the others: copy tile i-1 from the own buffer into the tensor
// Traffic per GPU: what the collective has to move and no more - a reduce-scatter receives 1/n
// of the input instead of (n-1)/n of it, an all-gather and a broadcast send one copy instead of
// n-1 - and the local copies run at memory speed beside the switch requests.
// All pointers and the piece size are multiples of 16 bytes (the host checks).
template <typename T, int MODE, int SW_THREADS, int U>
__global__ void __launch_bounds__(SW_THREADS, SW_MAX_THREADS / SW_THREADS)
switch_copy_kernel(GbTeam tm, GbSwitch sw, SwCopyArgs a) {
    typedef typename GbAcc<T>::type A;
    constexpr int V = SwVec<T>::N;
    constexpr int DEPTH = 3;
    constexpr int SW_HALF = SW_THREADS / 2;
    const int b = (int)blockIdx.x, B = (int)gridDim.x;
    const int mine = (a.ntiles - b + B - 1) / B;
    unsigned seq = gb_ld_volatile(sw.bseq + b);
    const size_t buf = (size_t)a.nsub * a.tile;
    char* stage = sw.uc + (size_t)b * DEPTH * buf;
    char* stage_mc = sw.mc + (size_t)b * DEPTH * buf;
    const int n = tm.world, me = tm.rank;
    const bool front = (int)threadIdx.x < SW_HALF;
    const int tid = (int)threadIdx.x - (front ? 0 : SW_HALF);
    GbLane half;
    half.tid = (size_t)tid; half.nth = SW_HALF; half.ld = tm.ld_mode;
    GbLane whole;
    whole.tid = threadIdx.x; whole.nth = SW_THREADS; whole.ld = tm.ld_mode;

    for (int s = 0; s <= mine; ++s) {
        const size_t off = ((size_t)s * B + b) * a.tile;                       // tile s, inside a piece
        const size_t len = s < mine ? (a.piece - off < a.tile ? a.piece - off : a.tile) : 0;
        const size_t poff = ((size_t)(s - 1) * B + b) * a.tile;                // tile s - 1
        const size_t plen = s >= 1 ? (a.piece - poff < a.tile ? a.piece - poff : a.tile) : 0;
        char* now = stage + (size_t)(s % DEPTH) * buf;
        char* now_mc = stage_mc + (size_t)(s % DEPTH) * buf;
        char* before = stage + (size_t)((s + DEPTH - 1) % DEPTH) * buf;
        char* before_mc = stage_mc + (size_t)((s + DEPTH - 1) % DEPTH) * buf;
        if (MODE == 0) {
            if (front) {
                if (len)
                    for (int q = 0; q < n; ++q)
                        gb_copy_bytes(half, now + (size_t)q * a.tile, a.in + (size_t)q * a.piece + off, len, false);
            } else if (plen) {
                const char* src = before_mc + (size_t)me * a.tile;
                const size_t nvec = plen >> 4;
                for (size_t v0 = (size_t)tid; v0 < nvec; v0 += (size_t)U * SW_HALF) {
                    SwVec<T> w[U];
                    #pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const size_t v = v0 + (size_t)u * SW_HALF;
                        if (v < nvec) w[u].u = SwitchSum<T>::load(src + (v << 4));
                    }
                    #pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const size_t v = v0 + (size_t)u * SW_HALF;
                        if (v >= nvec) continue;
                        if (a.divide > 0) {
                            #pragma unroll
                            for (int j = 0; j < V; ++j)
                                w[u].e[j] = gb_down<T>(gb_divide<A>(gb_up<T>(w[u].e[j]), a.divide));
                        }
                        gb_st16(a.out + poff + (v << 4), w[u].u);
                    }
                }
            }
        } else if (MODE == 1) {
            if (!front) {
                if (len) {
                    const char* src = a.in + off;
                    char* dst = now_mc + (size_t)me * a.tile;
                    const size_t nvec = len >> 4;
                    for (size_t v0 = (size_t)tid; v0 < nvec; v0 += (size_t)U * SW_HALF) {
                        uint4 w[U];
                        #pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const size_t v = v0 + (size_t)u * SW_HALF;
                            if (v < nvec) w[u] = __ldg(reinterpret_cast<const uint4*>(src + (v << 4)));
                        }
                        #pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const size_t v = v0 + (size_t)u * SW_HALF;
                            if (v < nvec) switch_store(dst + (v << 4), w[u]);
                        }
                    }
                }
            } else if (plen) {
                for (int q = 0; q < n; ++q)
                    gb_copy_bytes(half, a.out + (size_t)q * a.piece + poff, before + (size_t)q * a.tile, plen, true);
            }
        } else {
            if (me == a.root) {
                if (len) {
                    const size_t nvec = len >> 4;
                    for (size_t v0 = threadIdx.x; v0 < nvec; v0 += (size_t)U * SW_THREADS) {
                        uint4 w[U];
                        #pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const size_t v = v0 + (size_t)u * SW_THREADS;
                            if (v < nvec) w[u] = __ldg(reinterpret_cast<const uint4*>(a.in + off + (v << 4)));
                        }
                        #pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const size_t v = v0 + (size_t)u * SW_THREADS;
                            if (v < nvec) switch_store(now_mc + (v << 4), w[u]);
                        }
                    }
                }
            } else if (plen) {
                gb_copy_bytes(whole, a.out + poff, before, plen, true);
            }
        }
        if (!sw_block_sync(tm, sw, b, ++seq)) return;
        if (b == 0 && threadIdx.x == 0 && s == 0) tm.ctrl->stamps[0] = gb_now();
    }
    if (threadIdx.x == 0) {
        sw.bseq[b] = seq;
        if (b == 0) tm.ctrl->stamps[1] = gb_now();
    }
}

template <typename T, int MODE>
cudaError_t launch_copy(const GbTeam& tm, const GbSwitch& sw, const SwCopyArgs& a, int grid,
                        cudaStream_t stream) {
    if (switch_shape() == 0) switch_copy_kernel<T, MODE, 512, 4><<<grid, 512, 0, stream>>>(tm, sw, a);
    else switch_copy_kernel<T, MODE, 256, 8><<<grid, 256, 0, stream>>>(tm, sw, a);
    return cudaGetLastError();
}

// Shared preparation of the three: checks, plan, arguments.  Returns 0, -1 (does not fit) or -3
// (alignment: the caller takes the peer-memory kernel).
int prepare_copy(const GbTeam* team, const GbSwitch* sw, const void* in, void* out, size_t piece,
                 int nsub, int max_blocks, SwCopyArgs* a, int* grid) {
    if (sw->hier || sw->group_size != team->world) return -1;
    if (piece == 0 || (piece & 15) || ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15))
        return -3;
    GbSwitchPlan plan;
    if (gb_switch_plan_copy(sw, nsub, piece, max_blocks, &plan) != 0) return -1;
    a->in = static_cast<const char*>(in);
    a->out = static_cast<char*>(out);
    a->piece = piece;
    a->tile = plan.tile;
    a->ntiles = plan.ntiles;
    a->nsub = nsub;
    a->divide = 0;
    a->root = 0;
    *grid = plan.grid;
    return 0;
}

}  // namespace

// Tile size and grid for `nbytes` with at most `max_blocks` blocks: every rank of the team
// computes this from values they all share.  Returns 0, or -1 when the regions are too small
// for even one tile per block.
extern "C" int gb_switch_plan(const GbSwitch* sw, int n_islands, size_t nbytes, int max_blocks,
                              GbSwitchPlan* plan) {
    const int depth = sw->hier ? 4 : 3;
    const size_t unit = 16 * (size_t)sw->owners * 8;           // stripes of whole 128-byte lines
    // half-size blocks, two per SM - from 64 MiB on: below that the barrier (whose cost grows with
    // the number of blocks) weighs more than the second block per SM gains (measured on four
    // B200s: 8 / 16 / 32 MiB in 58 / 84 / 128 us on 128 blocks against 69 / 90 / 137 us on 256;
    // 256 MiB in 707 us on 256 against 765 us on 128)
    if (switch_shape() != 0 && nbytes >= ((size_t)64 << 20)) max_blocks *= 2;
    if (max_blocks > GB_SWITCH_MAX_BLOCKS) max_blocks = GB_SWITCH_MAX_BLOCKS;
    if (max_blocks < 1 || nbytes == 0) return -1;
    const size_t floor_tile = (8192 + unit - 1) / unit * unit;
    // as many blocks as have at least a floor-sized tile each
    size_t want_blocks = (nbytes + floor_tile - 1) / floor_tile;
    int grid = (int)(want_blocks < (size_t)max_blocks ? want_blocks : (size_t)max_blocks);
    size_t cap = sw->bytes / ((size_t)grid * depth) / unit * unit;
    if (sw->hier) {
        const size_t per_block = sw->len_bridge / (size_t)grid / (2 * (size_t)n_islands);   // one slot
        const size_t by_bridge = per_block * (size_t)sw->owners / unit * unit;
        if (by_bridge < cap) cap = by_bridge;
    }
    if (cap > GB_SWITCH_MAX_TILE) cap = GB_SWITCH_MAX_TILE / unit * unit;
    if (cap < unit) return -1;
    size_t tile = ((nbytes + grid - 1) / grid + unit - 1) / unit * unit;
    if (tile < floor_tile) tile = floor_tile;
    if (tile > cap) tile = cap;
    const size_t ntiles = (nbytes + tile - 1) / tile;
    if (ntiles > 0x7fffffffu) return -1;
    if ((size_t)grid > ntiles) grid = (int)ntiles;
    plan->tile = tile;
    plan->ntiles = (int)ntiles;
    plan->grid = grid;
    return 0;
}

// out = sum over the team of in (divided by `divide` when > 0).  dtype: 0 f32, 1 bf16, 2 f16;
// n elements; in / out any alignment (16-byte aligned runs fastest).  `sw`: the group's
// switch memory (the team's, or this rank's island's with sw->hier = 1).  Every rank passes the
// same n, dtype, divide and max_blocks.  Returns a cudaError_t, or -2 for a type the switch
// cannot add, -1 when the plan does not fit.
extern "C" int gb_switch_all_reduce(const GbTeam* team, const GbSwitch* sw, const void* in, void* out,
                                    size_t n, int dtype, int divide, int max_blocks,
                                    cudaStream_t stream) {
    const size_t esize = dtype == 0 ? 4 : 2;
    if (dtype < 0 || dtype > 2) return -2;
    GbSwitchPlan plan;
    if (gb_switch_plan(sw, team->n_islands, n * esize, max_blocks, &plan) != 0) return -1;
    SwArgs a;
    a.in = static_cast<const char*>(in);
    a.out = static_cast<char*>(out);
    a.nbytes = n * esize;
    a.tile = plan.tile;
    a.ntiles = plan.ntiles;
    a.divide = divide;
    if (dtype == 0) return (int)launch_switch<float>(*team, *sw, a, plan.grid, stream);
    if (dtype == 1) return (int)launch_switch<__nv_bfloat16>(*team, *sw, a, plan.grid, stream);
    return (int)launch_switch<__half>(*team, *sw, a, plan.grid, stream);
}

// The same sum in one step (see allreduce_switch_oneshot_kernel): for tensors of at most
// max_blocks x 32 KiB (max_blocks doubled for the half-size launch shape, 128 at most), one
// group, flat order.  The group's memory must have GB_SWITCH_ONESHOT_RESERVE bytes behind
// sw->bytes.  Returns a cudaError_t, -2 for a type the switch cannot add, -1 when it does not fit.
extern "C" int gb_switch_all_reduce_oneshot(const GbTeam* team, const GbSwitch* sw, const void* in, void* out,
                                            size_t n, int dtype, int divide, int max_blocks,
                                            cudaStream_t stream) {
    if (dtype < 0 || dtype > 2) return -2;
    const size_t nbytes = n * (dtype == 0 ? 4 : 2);
    if (switch_shape() != 0) max_blocks *= 2;
    if (max_blocks > GB_SWITCH_ONESHOT_BLOCKS) max_blocks = GB_SWITCH_ONESHOT_BLOCKS;
    if (sw->hier || nbytes == 0 || max_blocks < 1 || nbytes > (size_t)max_blocks * GB_SWITCH_ONESHOT_SLOT)
        return -1;
    SwArgs a;
    a.in = static_cast<const char*>(in);
    a.out = static_cast<char*>(out);
    a.nbytes = nbytes;
    a.divide = divide;
    size_t tile = ((nbytes + max_blocks - 1) / max_blocks + 127) / 128 * 128;
    if (tile < 2048) tile = 2048;
    a.tile = tile;
    a.ntiles = (int)((nbytes + tile - 1) / tile);
    const int grid = a.ntiles;
    cudaError_t err;
    if (switch_shape() == 0) {
        if (dtype == 0) allreduce_switch_oneshot_kernel<float, 512, 4><<<grid, 512, 0, stream>>>(*team, *sw, a);
        else if (dtype == 1) allreduce_switch_oneshot_kernel<__nv_bfloat16, 512, 4><<<grid, 512, 0, stream>>>(*team, *sw, a);
        else allreduce_switch_oneshot_kernel<__half, 512, 4><<<grid, 512, 0, stream>>>(*team, *sw, a);
    } else {
        if (dtype == 0) allreduce_switch_oneshot_kernel<float, 256, 8><<<grid, 256, 0, stream>>>(*team, *sw, a);
        else if (dtype == 1) allreduce_switch_oneshot_kernel<__nv_bfloat16, 256, 8><<<grid, 256, 0, stream>>>(*team, *sw, a);
        else allreduce_switch_oneshot_kernel<__half, 256, 8><<<grid, 256, 0, stream>>>(*team, *sw, a);
    }
    err = cudaGetLastError();
    return (int)err;
}

// The same sum for a tensor inside the group's switch memory, `offset` bytes from its start on
// every rank (a multiple of 16, like the tensor's size in bytes): in place, nothing copied.
// Returns a cudaError_t, -2 for a type the switch cannot add, -1 for a range outside the memory
// or a group that is an island of several (the in-place form is flat).
extern "C" int gb_switch_all_reduce_inplace(const GbTeam* team, const GbSwitch* sw, size_t offset,
                                            size_t n, int dtype, int divide, int max_blocks,
                                            cudaStream_t stream) {
    if (dtype < 0 || dtype > 2) return -2;
    const size_t nbytes = n * (dtype == 0 ? 4 : 2);
    if (sw->hier || (offset & 15) || (nbytes & 15) || nbytes == 0 || offset + nbytes > sw->bytes) return -1;
    if (switch_shape() != 0) max_blocks *= 2;
    if (max_blocks > GB_SWITCH_MAX_BLOCKS) max_blocks = GB_SWITCH_MAX_BLOCKS;
    if (max_blocks < 1) return -1;
    SwArgs a;
    a.in = nullptr;
    a.out = nullptr;
    a.nbytes = nbytes;
    a.divide = divide;
    // tiles of at least 16 KiB per owner-share sweep, at most one per block and step
    const size_t unit = 16 * (size_t)sw->owners * 8;
    size_t tile = ((nbytes + max_blocks - 1) / max_blocks + unit - 1) / unit * unit;
    const size_t floor_tile = (65536 + unit - 1) / unit * unit;
    if (tile < floor_tile) tile = floor_tile;
    if (tile > (4u << 20)) tile = (4u << 20) / unit * unit;
    a.tile = tile;
    a.ntiles = (int)((nbytes + tile - 1) / tile);
    const int grid = a.ntiles < max_blocks ? a.ntiles : max_blocks;
    if (dtype == 0) return (int)launch_inplace<float>(*team, *sw, a, offset, grid, stream);
    if (dtype == 1) return (int)launch_inplace<__nv_bfloat16>(*team, *sw, a, offset, grid, stream);
    return (int)launch_inplace<__half>(*team, *sw, a, offset, grid, stream);
}

// Tiles and grid of a copy-shaped collective: `nsub` sub-tiles per staging buffer, pieces of
// `piece` bytes.  Every rank computes this from values they all share.
extern "C" int gb_switch_plan_copy(const GbSwitch* sw, int nsub, size_t piece, int max_blocks,
                                   GbSwitchPlan* plan) {
    const size_t unit = 128;
    if (switch_shape() != 0) max_blocks *= 2;
    if (max_blocks > GB_SWITCH_MAX_BLOCKS) max_blocks = GB_SWITCH_MAX_BLOCKS;
    if (max_blocks < 1 || piece == 0 || nsub < 1) return -1;
    const size_t floor_tile = nsub > 1 ? 4096 : 16384;
    const size_t want_blocks = (piece + floor_tile - 1) / floor_tile;
    int grid = (int)(want_blocks < (size_t)max_blocks ? want_blocks : (size_t)max_blocks);
    size_t cap = sw->bytes / ((size_t)grid * 3 * (size_t)nsub) / unit * unit;
    const size_t most = (size_t)(2 * GB_SWITCH_MAX_TILE) / (size_t)nsub / unit * unit;   // 512 KiB per buffer
    if (cap > most) cap = most;
    if (cap < unit) return -1;
    size_t tile = ((piece + grid - 1) / grid + unit - 1) / unit * unit;
    if (tile < floor_tile) tile = floor_tile;
    if (tile > cap) tile = cap;
    const size_t ntiles = (piece + tile - 1) / tile;
    if (ntiles > 0x7fffffffu) return -1;
    if ((size_t)grid > ntiles) grid = (int)ntiles;
    plan->tile = tile;
    plan->ntiles = (int)ntiles;
    plan->grid = grid;
    return 0;
}

// out = this rank's piece (n_out elements) of the sum over the team of in (world pieces back to
// back), divided by `divide` when > 0.  dtype: 0 f32, 1 bf16, 2 f16.  Returns a cudaError_t, -2
// for a type the switch cannot add, -1 when it does not fit, -3 for pointers or a piece size
// that are not multiples of 16 bytes (take the peer-memory kernel then).
extern "C" int gb_switch_reduce_scatter(const GbTeam* team, const GbSwitch* sw, const void* in, void* out,
                                        size_t n_out, int dtype, int divide, int max_blocks,
                                        cudaStream_t stream) {
    if (dtype < 0 || dtype > 2) return -2;
    SwCopyArgs a;
    int grid = 0;
    const int rc = prepare_copy(team, sw, in, out, n_out * (dtype == 0 ? 4 : 2), team->world, max_blocks, &a, &grid);
    if (rc != 0) return rc;
    a.divide = divide;
    if (dtype == 0) return (int)launch_copy<float, 0>(*team, *sw, a, grid, stream);
    if (dtype == 1) return (int)launch_copy<__nv_bfloat16, 0>(*team, *sw, a, grid, stream);
    return (int)launch_copy<__half, 0>(*team, *sw, a, grid, stream);
}

// out = every rank's `in` (in_bytes each) back to back in team order.
extern "C" int gb_switch_all_gather(const GbTeam* team, const GbSwitch* sw, const void* in, void* out,
                                    size_t in_bytes, int max_blocks, cudaStream_t stream) {
    SwCopyArgs a;
    int grid = 0;
    const int rc = prepare_copy(team, sw, in, out, in_bytes, team->world, max_blocks, &a, &grid);
    if (rc != 0) return rc;
    return (int)launch_copy<float, 1>(*team, *sw, a, grid, stream);
}

// Every rank's `buffer` becomes the root's.
extern "C" int gb_switch_broadcast(const GbTeam* team, const GbSwitch* sw, void* buffer, size_t nbytes,
                                   int root, int max_blocks, cudaStream_t stream) {
    SwCopyArgs a;
    int grid = 0;
    const int rc = prepare_copy(team, sw, buffer, buffer, nbytes, 1, max_blocks, &a, &grid);
    if (rc != 0) return rc;
    a.root = root;
    return (int)launch_copy<float, 2>(*team, *sw, a, grid, stream);
}

extern "C" size_t gb_sizeof_switch() { return sizeof(GbSwitch); }

GB_BOUNDS_HOST(switch)
