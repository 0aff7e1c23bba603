// Shared device-side definitions of the fabric kernels (sm_100a).
//
// A "team" is the group of ranks one collective runs over.  Every rank owns a symmetric
// workspace that is mapped into every peer (CUDA IPC or cuMem handles), so a kernel can
// store into and load from any peer's workspace over NVLink.  All synchronisation between
// GPUs goes through one primitive, gb_sync_all(): a grid barrier on this GPU whose last
// arriving block also runs a barrier with every peer (a release store of a sequence number
// into each peer's flag row, an acquire poll of the own row).  Every wait is bounded by a
// spin limit and a globaltimer deadline; when one runs out the kernel records
// {code, peer, sequence, phase} in a host-mapped status block, raises the abort word and
// returns normally - it never traps and never spins forever.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#define GB_MAX_RANKS 16
#define GB_MAX_CHANNELS 8           // independent pipelines (control blocks, flag rows)
#define GB_FLAG_BYTES 4096          // start of every workspace: the flag rows
#define GB_STATUS_WORDS 8

// Local (not shared with peers) control block of one team.
struct GbCtrl {
    unsigned int grid_arrive;       // blocks that reached the current grid barrier
    unsigned int grid_gen;          // grid barrier generation
    unsigned int seq;               // last completed team barrier
    unsigned int epoch;             // collectives completed (parity selects buffer halves)
    unsigned int abort;             // a wait ran out in this or an earlier kernel
    unsigned int pad[3];
    unsigned long long stamps[8];   // globaltimer at the barriers of the last collective
};

struct GbTeam {
    int rank, world;                // this rank's position in the team, team size
    int n_islands;
    int my_island, my_pos;          // island of this rank, position inside it
    int island_off[GB_MAX_RANKS + 1];   // island i = order[island_off[i] .. island_off[i+1])
    int order[GB_MAX_RANKS];        // team ranks sorted by (island, position)
    char* ws[GB_MAX_RANKS];         // workspace base of every team rank (ws[rank] is local)
    GbCtrl* ctrl;
    volatile unsigned int* status;  // host-mapped: code, peer, seq, phase, ...
    unsigned long long timeout_ns;
    int ld_mode;                    // how peer-written data is loaded: 0 ld.relaxed.sys, 1 ld.global.cg
    int pad;
};

// (3 is GB_TIMEOUT_COPY, a bulk copy of the ring that never landed: gb_bulk.cuh)
enum GbStatus { GB_OK = 0, GB_TIMEOUT_PEER = 1, GB_TIMEOUT_GRID = 2, GB_TIMEOUT_TENSOR = 4 };

// ---- memory-order helpers ---------------------------------------------------------------
__device__ __forceinline__ unsigned long long gb_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned int gb_ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void gb_st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int gb_ld_volatile(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// 16-byte load of data another GPU wrote (or that lives in a peer's memory): never from L1.
// Mode 1 (the default) is a weak load that bypasses L1 (ld.global.cg): L2 is a memory-side
// cache, so it is coherent for local memory and not involved for a peer's; the barrier that
// precedes every such load orders it.  Mode 0 is a system-scope relaxed load.
#ifdef GB_BOUNDS
// The checked build (-DGB_BOUNDS, a library of its own): every 16-byte access of the fabric
// kernels and every source of a bulk copy is compared with the address ranges the host allowed
// for the launch (the workspaces of all ranks as mapped here, switch memory, the caller's
// tensors).  An access outside them is not made: the first one is recorded (address, kind,
// block, thread) and counted, a load returns zeros, a bulk copy reads the start of the first
// range instead.  One table per translation unit; the host fills and reads each through the
// functions GB_BOUNDS_HOST defines.  An empty table allows everything.
#define GB_BOUNDS_RANGES 40
struct GbBoundsTable {
    unsigned long long lo[GB_BOUNDS_RANGES], hi[GB_BOUNDS_RANGES];
    int n, pad;
    unsigned long long first[4];    // address, kind (0 load, 1 store, 2 bulk copy), block, thread
    unsigned int violations, pad2;
};
static __device__ GbBoundsTable gb_bounds_table;
__device__ __forceinline__ bool gb_in_bounds(const void* p, unsigned bytes, unsigned kind) {
    const unsigned long long a = reinterpret_cast<unsigned long long>(p);
    const int n = gb_bounds_table.n;
    if (n == 0) return true;
    for (int i = 0; i < n; ++i)
        if (a >= gb_bounds_table.lo[i] && a + bytes <= gb_bounds_table.hi[i]) return true;
    if (atomicAdd(&gb_bounds_table.violations, 1u) == 0) {
        gb_bounds_table.first[0] = a; gb_bounds_table.first[1] = kind;
        gb_bounds_table.first[2] = blockIdx.x; gb_bounds_table.first[3] = threadIdx.x;
    }
    return false;
}
__device__ __forceinline__ const char* gb_bounds_source(const char* p, unsigned bytes) {
    return gb_in_bounds(p, bytes, 2) ? p : reinterpret_cast<const char*>(gb_bounds_table.lo[0]);
}
#define GB_BOUNDS_HOST(unit)                                                                    \
    extern "C" int gb_bounds_set_##unit(const GbBoundsTable* t) {                               \
        return (int)cudaMemcpyToSymbol(gb_bounds_table, t, sizeof(GbBoundsTable));              \
    }                                                                                           \
    extern "C" int gb_bounds_get_##unit(GbBoundsTable* t) {                                     \
        return (int)cudaMemcpyFromSymbol(t, gb_bounds_table, sizeof(GbBoundsTable));            \
    }
#else
#define GB_BOUNDS_HOST(unit)
#endif

__device__ __forceinline__ uint4 gb_ld16(const void* p, int mode = 1) {
#ifdef GB_BOUNDS
    if (!gb_in_bounds(p, 16, 0)) return make_uint4(0u, 0u, 0u, 0u);
#endif
    if (mode == 0) {
        uint4 v;
        asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
        return v;
    }
    return __ldcg(reinterpret_cast<const uint4*>(p));      // ld.global.cg.v4: schedulable
}
__device__ __forceinline__ void gb_st16(void* p, uint4 v) {
#ifdef GB_BOUNDS
    if (!gb_in_bounds(p, 16, 1)) return;
#endif
    *reinterpret_cast<uint4*>(p) = v;
}

__device__ __forceinline__ unsigned int* gb_flag_row(const GbTeam& tm, int owner) {
    return reinterpret_cast<unsigned int*>(tm.ws[owner]);
}

__device__ __forceinline__ void gb_fail(const GbTeam& tm, unsigned code, unsigned peer,
                                        unsigned seq, unsigned phase) {
    if (atomicExch(&tm.ctrl->abort, 1u) == 0u) {
        tm.status[1] = peer; tm.status[2] = seq; tm.status[3] = phase;
        tm.status[4] = (unsigned)tm.rank;
        __threadfence_system();
        tm.status[0] = code;
    }
}

// Poll `addr` until it reaches `want` (sequence numbers compare by signed difference).
__device__ __forceinline__ bool gb_wait_flag(const GbTeam& tm, const unsigned int* addr,
                                             unsigned want, bool sys, unsigned long long limit_ns) {
    unsigned long long t0 = 0;
    for (unsigned spins = 0;; ++spins) {
        unsigned v = sys ? gb_ld_acquire_sys(addr) : gb_ld_volatile(addr);
        if ((int)(v - want) >= 0) return true;
        if (spins > 32) __nanosleep(spins > 4096 ? 400 : 40);
        if ((spins & 255u) == 255u) {
            unsigned long long now = gb_now();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) return false;
            if (gb_ld_volatile(&tm.ctrl->abort)) return false;
        }
        if (spins > 0x3fffffffu) return false;
    }
}

// Barrier of `nblocks` blocks of this grid and - with `with_peers` - of the same blocks on
// every peer.  `channel` selects the control block and the flag row, so independent groups of
// blocks (channels) can run their own pipelines and barriers inside one kernel.  Returns false
// when this or an earlier wait ran out; the caller must then return without touching peers
// again.  `phase` only labels a failure and selects a timestamp slot.
__device__ __forceinline__ bool gb_sync(const GbTeam& tm, int channel, unsigned nblocks,
                                        unsigned phase, bool first, bool with_peers = true) {
    __shared__ unsigned s_gen, s_last, s_seq;
    GbCtrl* c = tm.ctrl + channel;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();                       // this block's stores, local and remote
        s_gen = gb_ld_volatile(&c->grid_gen);         // read the generation before arriving
        unsigned arrived = atomicAdd(&c->grid_arrive, 1u) + 1u;
        s_last = (arrived == nblocks);
        s_seq = gb_ld_volatile(&c->seq) + 1u;
    }
    __syncthreads();
    if (s_last) {
        // The last block to arrive meets the peers on behalf of its channel.
        const unsigned seq = s_seq;
        const int t = threadIdx.x;
        const int row = channel * GB_MAX_RANKS;
        // A rank that has already given up (in this kernel or an earlier one) tells nobody that
        // it arrived: its data may be incomplete, and the peers' own deadlines then report it.
        const bool dead = gb_ld_volatile(&tm.ctrl->abort) != 0u;
        if (with_peers && !dead && t < tm.world && t != tm.rank) {
            __threadfence_system();
            gb_st_release_sys(gb_flag_row(tm, t) + row + tm.rank, seq);
        }
        if (with_peers && t < tm.world && t != tm.rank) {
            if (!gb_wait_flag(tm, gb_flag_row(tm, tm.rank) + row + t, seq, true, tm.timeout_ns))
                gb_fail(tm, GB_TIMEOUT_PEER, (unsigned)t, seq, phase);
        }
        __syncthreads();
        if (t == 0) {
            if (with_peers) c->seq = seq;
            if (first) c->epoch += 1u;
            if (phase < 8u) c->stamps[phase] = gb_now();
            c->grid_arrive = 0u;
            __threadfence();
            atomicAdd(&c->grid_gen, 1u);              // release the channel's blocks
        }
    } else if (threadIdx.x == 0) {
        if (!gb_wait_flag(tm, &c->grid_gen, s_gen + 1u, false, 2ull * tm.timeout_ns))
            gb_fail(tm, GB_TIMEOUT_GRID, 0u, s_seq, phase);
        __threadfence();
    }
    __syncthreads();
    return gb_ld_volatile(&tm.ctrl->abort) == 0u;
}

// The whole grid as one channel.
__device__ __forceinline__ bool gb_sync_all(const GbTeam& tm, unsigned phase, bool first) {
    return gb_sync(tm, 0, gridDim.x, phase, first, true);
}

__device__ __forceinline__ unsigned int gb_ld_acquire_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void gb_st_release_gpu(unsigned int* p, unsigned int v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}

// ---- element types -------------------------------------------------------------------------
enum GbDtype { GB_F32 = 0, GB_BF16 = 1, GB_F16 = 2, GB_F64 = 3, GB_I8 = 4, GB_U8 = 5,
               GB_I32 = 6, GB_I64 = 7 };
enum GbOp { GB_SUM = 0, GB_MAX = 1, GB_MIN = 2 };

template <typename T> struct GbAcc { typedef T type; };
template <> struct GbAcc<__nv_bfloat16> { typedef float type; };
template <> struct GbAcc<__half> { typedef float type; };

template <typename T> __device__ __forceinline__ typename GbAcc<T>::type gb_up(T v) { return v; }
template <> __device__ __forceinline__ float gb_up<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}
template <> __device__ __forceinline__ float gb_up<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T gb_down(typename GbAcc<T>::type v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 gb_down<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ __half gb_down<__half>(float v) { return __float2half_rn(v); }

template <int OP, typename A> __device__ __forceinline__ A gb_combine(A a, A b) {
    if (OP == GB_SUM) return a + b;
    if (OP == GB_MAX) return a > b ? a : b;
    return a < b ? a : b;
}
// NaN propagates through MAX/MIN the way torch's maximum/minimum do.
template <int OP> __device__ __forceinline__ float gb_combine_f(float a, float b) {
    if (OP == GB_SUM) return __fadd_rn(a, b);
    if (a != a) return a;
    if (b != b) return b;
    if (OP == GB_MAX) return a > b ? a : b;
    return a < b ? a : b;
}
template <int OP> __device__ __forceinline__ double gb_combine_d(double a, double b) {
    if (OP == GB_SUM) return a + b;
    if (a != a) return a;
    if (b != b) return b;
    if (OP == GB_MAX) return a > b ? a : b;
    return a < b ? a : b;
}
template <int OP, typename A> struct GbFold {
    static __device__ __forceinline__ A run(A a, A b) { return gb_combine<OP, A>(a, b); }
};
template <int OP> struct GbFold<OP, float> {
    static __device__ __forceinline__ float run(float a, float b) { return gb_combine_f<OP>(a, b); }
};
template <int OP> struct GbFold<OP, double> {
    static __device__ __forceinline__ double run(double a, double b) { return gb_combine_d<OP>(a, b); }
};

// AVG: the sum divided by the team size, as one correctly rounded division.
template <typename A> __device__ __forceinline__ A gb_divide(A v, int by) { return v / (A)by; }
template <> __device__ __forceinline__ float gb_divide<float>(float v, int by) {
    return __fdiv_rn(v, (float)by);
}

// ---- lanes --------------------------------------------------------------------------------------
// The threads that share one piece of work: the whole grid, or the blocks of one role when a
// kernel splits its grid so that different pipeline steps run at the same time.
struct GbLane {
    size_t tid, nth;      // this thread's index among the lane's threads, and their number
    int ld;               // load mode for peer-written data (GbTeam::ld_mode)
};
__device__ __forceinline__ GbLane gb_lane_all(int ld = 1) {
    GbLane l;
    l.ld = ld;
    l.tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    l.nth = (size_t)gridDim.x * blockDim.x;
    return l;
}
__device__ __forceinline__ GbLane gb_lane_blocks(int first, int count, int ld = 1) {
    GbLane l;
    l.ld = ld;
    l.tid = (size_t)(blockIdx.x - first) * blockDim.x + threadIdx.x;
    l.nth = (size_t)count * blockDim.x;
    return l;
}

// ---- byte copies -----------------------------------------------------------------------------
// Copy `nbytes` with the threads of a lane.  `peer_src`: the source was written by another GPU
// (or is remote), so it is read past L1.  Eight independent 16-byte transfers are in flight per
// thread, which is what hides the NVLink round trip of a remote load.  Falls back to narrower
// accesses for unaligned user tensors.
__device__ __forceinline__ void gb_copy_bytes(const GbLane& L, void* dst, const void* src,
                                              size_t nbytes, bool peer_src) {
    const size_t tid = L.tid, nth = L.nth;
    char* d = static_cast<char*>(dst);
    const char* s = static_cast<const char*>(src);
    if ((((uintptr_t)d | (uintptr_t)s) & 15u) == 0) {
        const size_t nv = nbytes >> 4;
        size_t i = tid;
        for (; i + 7 * nth < nv; i += 8 * nth) {
            uint4 r[8];
            #pragma unroll
            for (int u = 0; u < 8; ++u)
                r[u] = peer_src ? gb_ld16(s + ((i + u * nth) << 4), L.ld)
                                : __ldg((const uint4*)(s + ((i + u * nth) << 4)));
            #pragma unroll
            for (int u = 0; u < 8; ++u) gb_st16(d + ((i + u * nth) << 4), r[u]);
        }
        for (; i < nv; i += nth) {
            uint4 a = peer_src ? gb_ld16(s + (i << 4), L.ld) : __ldg((const uint4*)(s + (i << 4)));
            gb_st16(d + (i << 4), a);
        }
        for (size_t b = (nv << 4) + tid; b < nbytes; b += nth)
            d[b] = peer_src ? *(volatile const char*)(s + b) : s[b];
        return;
    }
    if ((((uintptr_t)d | (uintptr_t)s) & 3u) == 0) {
        const size_t nw = nbytes >> 2;
        for (size_t i = tid; i < nw; i += nth) {
            unsigned v = peer_src ? *(volatile const unsigned*)(s + (i << 2))
                                  : *(const unsigned*)(s + (i << 2));
            *(unsigned*)(d + (i << 2)) = v;
        }
        for (size_t b = (nw << 2) + tid; b < nbytes; b += nth)
            d[b] = peer_src ? *(volatile const char*)(s + b) : s[b];
        return;
    }
    for (size_t b = tid; b < nbytes; b += nth)
        d[b] = peer_src ? *(volatile const char*)(s + b) : s[b];
}
