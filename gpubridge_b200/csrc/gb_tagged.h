// Collectives over any worker that moves tagged byte ranges (send / recv / wait): the algorithms
// the host-staged bridges share, whatever carries the bytes - the multi-stream TCP worker
// (gb_tcp.cpp) or the RDMA-style endpoint (gb_rdma.cpp).
//
// Two members: every chunk's receive and send are posted at once and chunk i is folded as soon
// as both have completed, while later chunks are still on the wire.  More members: a ring
// reduce-scatter followed by a ring all-gather over near-equal segments (the first
// count % members segments hold one element more); segment j starts at member j and walks
// upward, every member folding what arrives into its own values.  Broadcast: the root sends to
// every other member.  Tags are sequence (24) | step (12) | sender (8) | chunk (20).  Any
// failure stops the worker before returning, so nothing still points into the caller's buffers.
// (Role of the reference's src/gpubridge/tagged.py, run natively.)
#pragma once
#include <cstddef>
#include <cstdint>

struct GbTaggedWorker {
    virtual ~GbTaggedWorker() {}
    virtual int members() const = 0;
    virtual int index() const = 0;
    // Operation ids (> 0), or < 0 on failure.  The buffers stay the caller's until wait() returns.
    virtual long send(int peer, const void* data, uint64_t length, uint64_t tag) = 0;
    virtual long recv(int peer, void* data, uint64_t length, uint64_t tag) = 0;
    virtual int wait(const long* ids, int count, double timeout_s) = 0;      // 0: all done
    virtual void stop() = 0;                                                 // after a failed post
    virtual void fail(const char* why) = 0;
};

// dtype: 0 f32, 1 bf16, 2 f16, 3 f64, 4 i8, 5 u8, 6 i32, 7 i64.  op: 0 sum, 1 max, 2 min.
size_t gb_tagged_dtype_size(int dtype);
void gb_tagged_fold(int dtype, void* into, const void* from, size_t n, int op);
uint64_t gb_tagged_tag(uint64_t seq, uint64_t step, uint64_t sender, uint64_t chunk);
// 0 on success, -1 after a failure (the worker has been stopped and holds the reason).
int gb_tagged_all_reduce(GbTaggedWorker& w, void* data, uint64_t count, int dtype, int op,
                         uint64_t chunk_elems, uint64_t seq, double timeout_s);
int gb_tagged_broadcast(GbTaggedWorker& w, void* data, uint64_t nbytes, int root, uint64_t chunk_bytes,
                        uint64_t seq, double timeout_s);
