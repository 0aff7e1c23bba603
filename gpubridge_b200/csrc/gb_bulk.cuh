// Bulk-copy ring: every read of a fabric kernel goes through the TMA unit.
//
// A block owns a ring of GB_RING_STAGES shared-memory stages.  One thread issues bulk
// asynchronous copies (cp.async.bulk, global -> shared, completion counted in bytes on an
// mbarrier) several stages ahead; all threads then consume a stage from shared memory and
// write results with ordinary 16-byte stores, to local memory or over NVLink.  Compared with
// loads into registers this keeps ~150 KB in flight per SM at almost no register cost, which
// is what a latency of one to two microseconds (HBM under load, NVLink round trip) needs to
// run a link or HBM at full rate from few SMs.  Sources may be local or a peer's memory;
// the copies are plain (no cluster fan-out), and stores never go through the copy engine, so
// nothing here needs completion tracking on the writing side.
//
// Every wait is bounded (try_wait spins with a globaltimer deadline).  When one runs out the
// block records GB_TIMEOUT_COPY, waits - bounded again - for its other copies in flight, and
// the caller returns.
#pragma once
#include "gb_common.cuh"

#define GB_RING_STAGES 4
#define GB_RING_STAGE_BYTES 49152
#define GB_RING_SMEM (GB_RING_STAGES * GB_RING_STAGE_BYTES + 1024)
#define GB_RING_MAX_SRC 16
#define GB_TIMEOUT_COPY 3

struct GbRing {
    unsigned char* buf;             // GB_RING_STAGES stages of GB_RING_STAGE_BYTES, 1024-aligned
    unsigned long long* full;       // one mbarrier per stage
    unsigned* fail;                 // block-wide failure word in shared memory
    unsigned uses;                  // stages used so far (equal in every thread of the block)
};

__device__ __forceinline__ unsigned gb_smem_u32(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}

// Call once at the top of the kernel, by every thread.
__device__ __forceinline__ GbRing gb_ring_init() {
    extern __shared__ unsigned char gb_dynamic_smem[];
    __shared__ __align__(8) unsigned long long bars[GB_RING_STAGES];
    __shared__ unsigned failed;
    GbRing r;
    r.buf = reinterpret_cast<unsigned char*>(
        ((uintptr_t)gb_dynamic_smem + 1023u) & ~(uintptr_t)1023u);
    r.full = bars;
    r.fail = &failed;
    r.uses = 0u;
    if (threadIdx.x == 0) {
        failed = 0u;
        for (int s = 0; s < GB_RING_STAGES; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(gb_smem_u32(&bars[s])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    return r;
}

__device__ __forceinline__ bool gb_mbar_try(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(gb_smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0u;
}

__device__ __forceinline__ bool gb_mbar_wait(unsigned long long* bar, unsigned parity,
                                             unsigned long long limit_ns) {
    unsigned long long t0 = 0;
    for (unsigned spins = 0; spins < 0x40000000u; ++spins) {
        if (gb_mbar_try(bar, parity)) return true;
        if ((spins & 63u) == 63u) {
            const unsigned long long now = gb_now();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) return false;
        }
    }
    return false;
}

// One stage's loads: `m` pieces of `len` bytes, piece p from src + p * src_stride + off, into
// stage + p * pitch.  len and every address are multiples of 16.
__device__ __forceinline__ void gb_ring_issue(const GbRing& R, unsigned use, const char* src,
                                              size_t src_stride, int m, size_t off, unsigned len,
                                              unsigned pitch) {
    const unsigned stage = use % GB_RING_STAGES;
    const unsigned bar = gb_smem_u32(&R.full[stage]);
    const unsigned dst = gb_smem_u32(R.buf + (size_t)stage * GB_RING_STAGE_BYTES);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                 :: "r"(bar), "r"(len * (unsigned)m) : "memory");
    for (int p = 0; p < m; ++p) {
        const char* from = src + (size_t)p * src_stride + off;
#ifdef GB_BOUNDS
        from = gb_bounds_source(from, len);
#endif
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
            :: "r"(dst + (unsigned)p * pitch), "l"(from), "r"(len), "r"(bar) : "memory");
    }
}

// The tile size a transfer of `bytes` per source is cut into when `nblocks` blocks share it
// and each stage holds `m` pieces: as large as a stage allows, smaller when that would leave
// blocks without work; a multiple of 1024.
__device__ __forceinline__ unsigned gb_ring_tile(size_t bytes, int m, int nblocks) {
    unsigned cap = (GB_RING_STAGE_BYTES / (unsigned)m) & ~1023u;
    size_t even = (bytes / (size_t)nblocks + 1023u) & ~(size_t)1023u;
    if (even < 2048u) even = 2048u;
    return even < cap ? (unsigned)even : cap;
}

// Stream `bytes` (a multiple of 16) from each of `m` sources (source p starts at
// src + p * src_stride) through the ring.  Block `bi` of
// `nb` takes tiles bi, bi + nb, ...; for every tile all threads call
//     consume(stage_base, pitch, offset, len)
// where piece p of the tile starts at stage_base + p * pitch and covers bytes
// [offset, offset + len) of every source.  `after_peer_writes`: the sources were written
// during this kernel (by peers or by other blocks), so the copy engine's reads are ordered
// after the barrier the caller has just passed.  Returns false after a timeout.
template <typename F>
__device__ __forceinline__ bool gb_ring_run(GbRing& R, const GbTeam& tm, int bi, int nb,
                                            const char* src, size_t src_stride, int m,
                                            size_t bytes, bool after_peer_writes, F&& consume) {
    if (bytes == 0) return true;
    const unsigned tile = gb_ring_tile(bytes, m, nb);
    const size_t ntiles = (bytes + tile - 1) / tile;
    const size_t mine = ntiles > (size_t)bi ? (ntiles - bi + nb - 1) / nb : 0;
    if (mine == 0) return true;
    const unsigned base = R.uses;
    const bool issuer = threadIdx.x == 0;
    auto tile_off = [&](size_t i) { return ((size_t)bi + i * nb) * tile; };
    auto tile_len = [&](size_t i) {
        const size_t o = tile_off(i);
        return (unsigned)(bytes - o < tile ? bytes - o : tile);
    };
    if (issuer) {
        if (after_peer_writes) asm volatile("fence.proxy.async.global;" ::: "memory");
        const size_t ahead = mine < GB_RING_STAGES - 1 ? mine : GB_RING_STAGES - 1;
        for (size_t i = 0; i < ahead; ++i)
            gb_ring_issue(R, base + (unsigned)i, src, src_stride, m, tile_off(i), tile_len(i), tile);
    }
    size_t failed_at = mine;
    for (size_t i = 0; i < mine; ++i) {
        const size_t next = i + GB_RING_STAGES - 1;
        if (issuer && next < mine)
            gb_ring_issue(R, base + (unsigned)next, src, src_stride, m, tile_off(next), tile_len(next), tile);
        const unsigned use = base + (unsigned)i;
        const unsigned stage = use % GB_RING_STAGES;
        if (!gb_mbar_wait(&R.full[stage], (use / GB_RING_STAGES) & 1u, tm.timeout_ns))
            *R.fail = 1u;
        else
            consume(R.buf + (size_t)stage * GB_RING_STAGE_BYTES, tile, tile_off(i), tile_len(i));
        __syncthreads();                       // the stage is free again; the verdict is shared
        if (*R.fail) { failed_at = i; break; }
    }
    if (failed_at < mine) {
        // Copies already issued (tiles failed_at .. failed_at + STAGES - 1) may still land:
        // give each its own bounded wait before the block leaves.
        if (issuer) {
            gb_fail(tm, GB_TIMEOUT_COPY, (unsigned)tm.rank, R.uses, 0u);
            for (size_t i = failed_at; i < mine && i < failed_at + GB_RING_STAGES; ++i) {
                const unsigned use = base + (unsigned)i;
                gb_mbar_wait(&R.full[use % GB_RING_STAGES], (use / GB_RING_STAGES) & 1u,
                             tm.timeout_ns / 4u + 1u);
            }
        }
        __syncthreads();
        return false;
    }
    R.uses = base + (unsigned)mine;
    return true;
}

// Copy with the ring: src -> dst, any sizes; the part that is not 16-byte aligned on both
// sides, or shorter than 16 bytes, goes through gb_copy_bytes.
__device__ __forceinline__ bool gb_ring_copy(GbRing& R, const GbTeam& tm, const GbLane& L, int bi,
                                             int nb, void* dst, const void* src, size_t nbytes,
                                             bool after_peer_writes) {
    char* d = static_cast<char*>(dst);
    const char* s = static_cast<const char*>(src);
    if ((((uintptr_t)d | (uintptr_t)s) & 15u) != 0 || nbytes < 4096) {
        gb_copy_bytes(L, d, s, nbytes, after_peer_writes);
        return true;
    }
    const size_t body = nbytes & ~(size_t)15;
    const bool ok = gb_ring_run(R, tm, bi, nb, s, 0, 1, body, after_peer_writes,
        [&](const unsigned char* stage, unsigned, size_t off, unsigned len) {
            const unsigned nv = len >> 4;
            char* out = d + off;
            for (unsigned v = threadIdx.x; v < nv; v += blockDim.x)
                gb_st16(out + ((size_t)v << 4), *reinterpret_cast<const uint4*>(stage + ((size_t)v << 4)));
        });
    if (!ok) return false;
    if (body < nbytes) gb_copy_bytes(L, d + body, s + body, nbytes - body, after_peer_writes);
    return true;
}

// ---- several transfers through one pipeline -----------------------------------------------------
// The steps a pipelined collective runs between two barriers are independent of each other, so
// their tiles are queued back to back: the ring stays full across step boundaries instead of
// draining and refilling (a refill costs one memory latency per step and block).
struct GbJob {
    const char* src;        // source p of the job starts at src + p * src_stride
    size_t src_stride;
    size_t bytes;           // per source; a multiple of 16
    char* dst;              // kind-specific (copy: destination of byte 0)
    int m;                  // sources
    int kind;               // meaning is the caller's
    int arg;                // kind-specific
    unsigned tile;          // derived by gb_jobs_plan
    unsigned first;         // block that takes tile 0
    size_t ntiles;
};

#define GB_MAX_JOBS (2 * GB_MAX_RANKS + 2)

// Tile sizes and a round-robin assignment that continues from job to job.
__device__ __forceinline__ void gb_jobs_plan(GbJob* jobs, int njobs, int nb) {
    size_t total = 0;
    for (int j = 0; j < njobs; ++j) total += jobs[j].bytes * (size_t)jobs[j].m;
    size_t seen = 0;
    for (int j = 0; j < njobs; ++j) {
        GbJob& job = jobs[j];
        // size tiles as if the whole queue were one transfer, so small jobs do not get
        // needlessly small tiles and large queues use whole stages
        unsigned cap = (GB_RING_STAGE_BYTES / (unsigned)job.m) & ~1023u;
        size_t even = (total / (size_t)job.m / (size_t)nb + 1023u) & ~(size_t)1023u;
        if (even < 4096u) even = 4096u;
        job.tile = even < cap ? (unsigned)even : cap;
        job.ntiles = (job.bytes + job.tile - 1) / job.tile;
        job.first = (unsigned)(seen % (size_t)nb);
        seen += job.ntiles;
    }
}

struct GbCursor { int j; size_t t; };

__device__ __forceinline__ void gb_cursor_settle(GbCursor& c, const GbJob* jobs, int njobs, int bi,
                                                 int nb) {
    while (c.j < njobs && c.t >= jobs[c.j].ntiles) {
        ++c.j;
        if (c.j < njobs) c.t = (size_t)((bi - (int)jobs[c.j].first + nb) % nb);
    }
}

// Run the queue.  `jobs` lives in shared memory and was planned by gb_jobs_plan.  For every
// tile all threads call consume(job, stage_base, pitch, offset, len).
template <typename F>
__device__ __forceinline__ bool gb_ring_run_jobs(GbRing& R, const GbTeam& tm, int bi, int nb,
                                                 const GbJob* jobs, int njobs, F&& consume) {
    if (njobs == 0) return true;
    const bool issuer = threadIdx.x == 0;
    GbCursor cc;
    cc.j = 0;
    cc.t = (size_t)((bi - (int)jobs[0].first + nb) % nb);
    gb_cursor_settle(cc, jobs, njobs, bi, nb);
    GbCursor ic = cc;
    unsigned issued = R.uses, use = R.uses;
    auto issue_one = [&]() {
        const GbJob& job = jobs[ic.j];
        const size_t off = ic.t * job.tile;
        const unsigned len = (unsigned)(job.bytes - off < job.tile ? job.bytes - off : job.tile);
        gb_ring_issue(R, issued, job.src, job.src_stride, job.m, off, len, job.tile);
        ++issued;
        ic.t += (size_t)nb;
        gb_cursor_settle(ic, jobs, njobs, bi, nb);
    };
    if (issuer) {
        asm volatile("fence.proxy.async.global;" ::: "memory");
        for (int a = 0; a < GB_RING_STAGES - 1 && ic.j < njobs; ++a) issue_one();
    }
    bool failed = false;
    while (cc.j < njobs) {
        if (issuer && ic.j < njobs) issue_one();
        const GbJob& job = jobs[cc.j];
        const size_t off = cc.t * job.tile;
        const unsigned len = (unsigned)(job.bytes - off < job.tile ? job.bytes - off : job.tile);
        const unsigned stage = use % GB_RING_STAGES;
        if (!gb_mbar_wait(&R.full[stage], (use / GB_RING_STAGES) & 1u, tm.timeout_ns))
            *R.fail = 1u;
        else
            consume(job, R.buf + (size_t)stage * GB_RING_STAGE_BYTES, job.tile, off, len);
        __syncthreads();
        if (*R.fail) { failed = true; break; }
        ++use;
        cc.t += (size_t)nb;
        gb_cursor_settle(cc, jobs, njobs, bi, nb);
    }
    if (failed) {
        if (issuer) {
            gb_fail(tm, GB_TIMEOUT_COPY, (unsigned)tm.rank, use, 1u);
            for (unsigned u = use; u != issued; ++u)      // copies still in flight
                gb_mbar_wait(&R.full[u % GB_RING_STAGES], (u / GB_RING_STAGES) & 1u,
                             tm.timeout_ns / 4u + 1u);
        }
        __syncthreads();
        return false;
    }
    R.uses = use;
    return true;
}
