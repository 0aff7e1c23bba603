// Host-side engine: planner and launches of the fused collectives (see gb_engine.h).
#include <atomic>
#include <cmath>
#include <cstring>
#include <new>

#include "gb_common.cuh"
#include "gb_engine.h"
#include "gb_switch.h"

extern "C" int gb_launch_reduce(int kind, int dtype, int op, int codec, const GbTeam* team,
                                const GbArgs* args, int grid, cudaStream_t stream);
extern "C" int gb_launch_copy(int kind, const GbTeam* team, const GbArgs* args, int grid,
                              cudaStream_t stream);
extern "C" int gb_switch_all_reduce(const GbTeam* team, const GbSwitch* sw, const void* in, void* out,
                                    size_t n, int dtype, int divide, int max_blocks,
                                    cudaStream_t stream);
extern "C" int gb_switch_all_reduce_oneshot(const GbTeam* team, const GbSwitch* sw, const void* in, void* out,
                                            size_t n, int dtype, int divide, int max_blocks,
                                            cudaStream_t stream);
extern "C" int gb_switch_reduce_scatter(const GbTeam* team, const GbSwitch* sw, const void* in, void* out,
                                        size_t n_out, int dtype, int divide, int max_blocks,
                                        cudaStream_t stream);
extern "C" int gb_switch_all_gather(const GbTeam* team, const GbSwitch* sw, const void* in, void* out,
                                    size_t in_bytes, int max_blocks, cudaStream_t stream);
extern "C" int gb_switch_broadcast(const GbTeam* team, const GbSwitch* sw, void* buffer, size_t nbytes,
                                   int root, int max_blocks, cudaStream_t stream);

namespace {

constexpr int kThreads = 512;
// One link direction saturates near 650 GB/s; a team barrier inside a kernel costs ~10 us
// (both measured with the link probe).  The pipeline depth is sized from these.
constexpr double kLinkBytesPerS = 650e9, kBarrierS = 10e-6;
constexpr int kElemSize[8] = {4, 2, 2, 8, 1, 1, 4, 8};   // GbDtype order: f32 bf16 f16 f64 i8 u8 i32 i64

struct Engine {
    GbTeam team;
    GbEngineConfig c;
    // in-switch all-reduce: the team's group (flat) and this rank's island's (hierarchical order)
    GbSwitch sw_team{}, sw_island{};
    bool has_team = false, has_island = false;
    size_t sw_min_bytes = 0;
    int sw_min_ranks = 3;
    size_t sw_copy_min_bytes = ~size_t(0);      // broadcast through the switch from this size on
    size_t sw_gather_min_bytes = ~size_t(0);    // reduce-scatter and all-gather
    size_t sw_oneshot_max = 0;                  // the one-step all-reduce up to this size
    std::atomic<unsigned long long> launches{0};
};

inline size_t down(size_t v, size_t m) { return v / m * m; }
inline size_t up(size_t v, size_t m) { return (v + m - 1) / m * m; }
inline size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

// Whether a copy-shaped collective of `total` bytes in pieces of `piece` bytes takes the switch
// (the team's group; pieces and pointers in multiples of 16 bytes): the same rule as
// Fabric._switch_copy.
bool switch_copy(const Engine& e, size_t total, size_t piece, const void* p0, const void* p1,
                 bool gather = true) {
    const size_t least = gather ? e.sw_gather_min_bytes : e.sw_copy_min_bytes;
    return e.has_team && e.team.world >= e.sw_min_ranks && e.c.algo == 0 && total >= least &&
           (piece & 15) == 0 &&
           ((reinterpret_cast<uintptr_t>(p0) | reinterpret_cast<uintptr_t>(p1)) & 15) == 0;
}

void switch_grid(const Engine& e, int grid_cap, GbLaunch* L, int kind) {
    L->family = 2;
    L->kind = kind;
    L->grid = e.c.max_blocks;
    if (grid_cap > 0 && grid_cap < L->grid) L->grid = grid_cap;
}

int grid_for(const Engine& e, size_t nbytes, int cap, int grid_cap) {
    const size_t blocks = ceil_div(nbytes, size_t(kThreads) * 16 * 4);
    int limit = e.c.max_blocks;
    if (cap > 0 && cap < limit) limit = cap;
    if (grid_cap > 0 && grid_cap < limit) limit = grid_cap;
    const size_t g = blocks < size_t(limit) ? blocks : size_t(limit);
    return g < 1 ? 1 : int(g);
}

}  // namespace

extern "C" int gb_plan_hier(size_t n, int esize, int k, int m_max, int n_islands, size_t len_ha,
                            size_t len_hb, size_t len_hc, int grid, size_t chunk_bytes,
                            int force_channels, int force_chunks, int stripe_multiple,
                            GbHierPlanOut* out) {
    const size_t nbytes = n * size_t(esize);
    int channels = force_channels > 0 ? force_channels
                   : nbytes < (size_t(4) << 20) ? 1 : nbytes < (size_t(32) << 20) ? 2 : 4;
    const int by_grid = grid / 8 > 0 ? grid / 8 : 1;
    if (channels > by_grid) channels = by_grid;
    if (channels > 8) channels = 8;
    if (channels < 1) channels = 1;
    const int whole = grid / channels * channels;
    grid = whole > channels ? whole : channels;
    const size_t len_a = len_ha / channels / 4096 * 4096;
    const size_t len_b = len_hb / channels / 4096 * 4096;
    const size_t len_c = len_hc / channels / 4096 * 4096;
    size_t slot = len_a / m_max;
    if (len_b / n_islands < slot) slot = len_b / n_islands;
    if (len_c < slot) slot = len_c;
    const size_t sm = size_t(stripe_multiple);
    const size_t stripe_cap = down(slot / esize, sm);
    if (stripe_cap < sm) return GB_ENGINE_WORKSPACE;
    size_t want;
    if (chunk_bytes) {
        want = chunk_bytes / esize / k;
        if (want < 256) want = 256;
    } else {
        // per channel T(c) = (c + depth) (barrier + link time / c) is least at
        // c = sqrt(depth * link time / barrier)
        double share = double(m_max - 1) / m_max;
        const double across = n_islands > 1 ? double(n_islands - 1) / k : 0.0;
        if (across > share) share = across;
        const int depth = n_islands > 1 ? 3 : 2;
        const double link_s = double(nbytes) / channels * share / kLinkBytesPerS;
        long long chunks = force_chunks > 0 ? force_chunks
                                            : (long long)std::nearbyint(std::sqrt(depth * link_s / kBarrierS));
        if (chunks < 1) chunks = 1;
        want = ceil_div(n, size_t(chunks) * channels * k);
    }
    const size_t per_k = ceil_div(n, size_t(k));
    size_t target = want < per_k ? want : per_k;
    if (target < 1) target = 1;
    size_t stripe = up(target, sm);
    if (stripe > stripe_cap) stripe = stripe_cap;
    out->channels = channels;
    out->grid = grid;
    out->stripe = stripe;
    out->nchunks = ceil_div(n, stripe * k);
    out->len_a = len_a;
    out->len_b = len_b;
    out->len_c = len_c;
    return GB_ENGINE_OK;
}

extern "C" void* gb_engine_create(const GbTeam* team, const GbEngineConfig* config) {
    Engine* e = new (std::nothrow) Engine();
    if (e == nullptr) return nullptr;
    e->team = *team;
    e->c = *config;
    return e;
}

extern "C" void gb_engine_destroy(void* engine) { delete static_cast<Engine*>(engine); }

extern "C" unsigned long long gb_engine_launches(void* engine) {
    return static_cast<Engine*>(engine)->launches.load();
}

extern "C" size_t gb_sizeof_engine_config() { return sizeof(GbEngineConfig); }
extern "C" size_t gb_sizeof_launch() { return sizeof(GbLaunch); }

extern "C" unsigned int gb_engine_status(void* engine) {
    const Engine& e = *static_cast<Engine*>(engine);
    return e.team.status ? e.team.status[0] : 0u;
}

extern "C" int gb_engine_prepare_all_reduce(void* engine, const void* in, void* out, size_t n, int dtype,
                                            int op, int divide, int grid_cap, GbLaunch* L) {
    const Engine& e = *static_cast<Engine*>(engine);
    if (dtype < 0 || dtype > 7 || op < 0 || op > 2 || n == 0) return GB_ENGINE_UNSUPPORTED;
    const int esize = kElemSize[dtype];
    const size_t nbytes = n * size_t(esize);
    std::memset(L, 0, sizeof(*L));
    GbArgs& a = L->args;
    a.in = in;
    a.out = out;
    a.n = n;
    a.divide = divide > 0 ? divide : 0;
    L->family = 0;
    if ((e.has_island || e.has_team) && op == 0 && dtype <= 2 && nbytes >= e.sw_min_bytes &&
        e.team.world >= e.sw_min_ranks) {
        L->family = 2;
        L->kind = e.has_island ? 1 : 0;
        L->grid = e.c.max_blocks;
        if (grid_cap > 0 && grid_cap < L->grid) L->grid = grid_cap;
        // one step (kind 5): the flat group, small enough, inside the slots this grid has
        size_t blocks = 2 * size_t(L->grid);
        if (blocks > GB_SWITCH_ONESHOT_BLOCKS) blocks = GB_SWITCH_ONESHOT_BLOCKS;
        if (!e.has_island && nbytes <= e.sw_oneshot_max && nbytes <= blocks * GB_SWITCH_ONESHOT_SLOT)
            L->kind = 5;
        return GB_ENGINE_OK;
    }
    if (nbytes <= e.c.oneshot_slot && e.c.algo != 2) {
        a.off_a = e.c.off_oneshot;
        a.len_a = e.c.len_oneshot;
        L->kind = 0;
        L->grid = grid_for(e, nbytes, 32, grid_cap);
        return GB_ENGINE_OK;
    }
    const bool aligned = ((reinterpret_cast<size_t>(in) | reinterpret_cast<size_t>(out)) % 16) == 0;
    const bool ring = e.c.ring != 0 && aligned;
    const bool two_shot = ring && e.c.ring == 2 && e.team.n_islands >= 3 && e.c.two_shot != 0;
    GbHierPlanOut p;
    const int rc = gb_plan_hier(n, esize, e.c.k, e.c.m_max, e.team.n_islands, e.c.len_ha, e.c.len_hb,
                                e.c.len_hc, grid_for(e, nbytes * 2, 0, grid_cap), 0, e.c.force_channels,
                                e.c.force_chunks, two_shot ? 256 * e.team.n_islands : 256, &p);
    if (rc != GB_ENGINE_OK) return rc;
    a.role_b = two_shot ? 1 : 0;
    a.stripe = p.stripe;
    a.k = e.c.k;
    a.chunk = p.stripe * size_t(e.c.k);
    a.off_a = e.c.off_ha; a.len_a = p.len_a;
    a.off_b = e.c.off_hb; a.len_b = p.len_b;
    a.off_c = e.c.off_hc; a.len_c = p.len_c;
    a.role_a = p.channels;
    L->kind = ring ? (e.c.ring == 2 ? 4 : 3) : 1;
    L->grid = p.grid;
    return GB_ENGINE_OK;
}

extern "C" int gb_engine_prepare_reduce_scatter(void* engine, const void* in, void* out, size_t n_out,
                                                int dtype, int divide, int grid_cap, GbLaunch* L) {
    const Engine& e = *static_cast<Engine*>(engine);
    if (dtype < 0 || dtype > 7 || n_out == 0) return GB_ENGINE_UNSUPPORTED;
    const int esize = kElemSize[dtype];
    std::memset(L, 0, sizeof(*L));
    GbArgs& a = L->args;
    a.in = in;
    a.out = out;
    a.n = n_out;
    a.divide = divide > 0 ? divide : 0;
    if (dtype <= 2 && switch_copy(e, n_out * size_t(esize) * e.team.world, n_out * size_t(esize), in, out)) {
        switch_grid(e, grid_cap, L, 2);
        return GB_ENGINE_OK;
    }
    const size_t cap = down(e.c.rs_chunk_bytes / esize, 256), whole = up(n_out, 256);
    a.chunk = cap < whole ? cap : whole;
    if (a.chunk == 0) return GB_ENGINE_WORKSPACE;
    a.off_a = e.c.off_rs;
    a.len_a = e.c.len_rs;
    const int limit = e.c.scatter_blocks < e.c.max_blocks ? e.c.scatter_blocks : e.c.max_blocks;
    const int grid = grid_for(e, n_out * size_t(esize) * e.team.world, limit, grid_cap);
    if (ceil_div(n_out, a.chunk) >= 4 && grid >= 8) a.role_a = grid * 3 / 4;
    L->family = 0;
    L->kind = 2;
    L->grid = grid;
    return GB_ENGINE_OK;
}

extern "C" int gb_engine_prepare_all_gather(void* engine, const void* in, void* out, size_t in_bytes,
                                            int grid_cap, GbLaunch* L) {
    const Engine& e = *static_cast<Engine*>(engine);
    if (in_bytes == 0) return GB_ENGINE_UNSUPPORTED;
    std::memset(L, 0, sizeof(*L));
    GbArgs& a = L->args;
    a.in = in;
    a.out = out;
    a.n = in_bytes;
    if (switch_copy(e, in_bytes * size_t(e.team.world), in_bytes, in, out)) {
        switch_grid(e, grid_cap, L, 3);
        return GB_ENGINE_OK;
    }
    const size_t whole = up(in_bytes, 16);
    a.chunk = e.c.ag_chunk_bytes < whole ? e.c.ag_chunk_bytes : whole;
    a.off_a = e.c.off_ag;
    a.len_a = e.c.len_ag;
    const int limit = e.c.copy_blocks < e.c.max_blocks ? e.c.copy_blocks : e.c.max_blocks;
    L->family = 1;
    L->kind = 0;
    L->grid = grid_for(e, in_bytes * size_t(e.team.world), limit, grid_cap);
    return GB_ENGINE_OK;
}

extern "C" int gb_engine_prepare_broadcast(void* engine, void* buffer, size_t nbytes, int root,
                                           int grid_cap, GbLaunch* L) {
    const Engine& e = *static_cast<Engine*>(engine);
    if (nbytes == 0 || root < 0 || root >= e.team.world) return GB_ENGINE_UNSUPPORTED;
    std::memset(L, 0, sizeof(*L));
    GbArgs& a = L->args;
    a.out = buffer;
    a.n = nbytes;
    a.root = root;
    if (switch_copy(e, nbytes, nbytes, buffer, buffer, /*gather=*/false)) {
        switch_grid(e, grid_cap, L, 4);
        return GB_ENGINE_OK;
    }
    const size_t share = up(ceil_div(nbytes, size_t(e.team.world)), 16);
    const size_t stripe = e.c.bc_stripe_bytes < share ? e.c.bc_stripe_bytes : share;
    a.stripe = stripe;
    a.chunk = stripe * size_t(e.team.world);
    a.off_a = e.c.off_bc;
    a.len_a = e.c.len_bc;
    const int limit = e.c.copy_blocks < e.c.max_blocks ? e.c.copy_blocks : e.c.max_blocks;
    L->family = 1;
    L->kind = 1;
    L->grid = grid_for(e, nbytes * 2, limit, grid_cap);
    return GB_ENGINE_OK;
}

// The team's switch memory, once it has been bound: `team` for the flat order, `island` for the
// hierarchical one (either may be null); SUM / AVG of floats of at least min_bytes then go
// through the switch.  The island group wins when both are given.
extern "C" void gb_engine_set_switch(void* engine, const GbSwitch* team, const GbSwitch* island,
                                     size_t min_bytes, int min_ranks) {
    Engine& e = *static_cast<Engine*>(engine);
    e.has_team = team != nullptr;
    e.has_island = island != nullptr;
    if (team) e.sw_team = *team;
    if (island) e.sw_island = *island;
    e.sw_min_bytes = min_bytes;
    e.sw_min_ranks = min_ranks;
}

// Up to how many bytes an all-reduce through the flat group takes the one-step kernel (0: never).
extern "C" void gb_engine_set_switch_oneshot(void* engine, size_t max_bytes) {
    static_cast<Engine*>(engine)->sw_oneshot_max = max_bytes;
}

// From how many bytes on a broadcast, and a reduce-scatter or all-gather, go through the team's
// switch group (never, until this is called).
extern "C" void gb_engine_set_switch_copy(void* engine, size_t broadcast_min_bytes, size_t gather_min_bytes) {
    static_cast<Engine*>(engine)->sw_copy_min_bytes = broadcast_min_bytes;
    static_cast<Engine*>(engine)->sw_gather_min_bytes = gather_min_bytes;
}

namespace {
int launch(Engine& e, const GbLaunch& L, int dtype, int op, void* stream) {
    if (L.family == 2 && L.kind >= 2) {
        cudaStream_t on = static_cast<cudaStream_t>(stream);
        const int rc = L.kind == 5
            ? gb_switch_all_reduce_oneshot(&e.team, &e.sw_team, L.args.in, L.args.out, L.args.n, dtype,
                                           L.args.divide, L.grid, on)
            : L.kind == 2
            ? gb_switch_reduce_scatter(&e.team, &e.sw_team, L.args.in, L.args.out, L.args.n, dtype,
                                       L.args.divide, L.grid, on)
            : L.kind == 3
            ? gb_switch_all_gather(&e.team, &e.sw_team, L.args.in, L.args.out, L.args.n, L.grid, on)
            : gb_switch_broadcast(&e.team, &e.sw_team, L.args.out, L.args.n, L.args.root, L.grid, on);
        if (rc == 0) e.launches.fetch_add(1, std::memory_order_relaxed);
        return rc;
    }
    if (L.family == 2) {
        const int rc = gb_switch_all_reduce(&e.team, L.kind == 1 ? &e.sw_island : &e.sw_team, L.args.in,
                                            L.args.out, L.args.n, dtype, L.args.divide, L.grid,
                                            static_cast<cudaStream_t>(stream));
        if (rc == 0) e.launches.fetch_add(1, std::memory_order_relaxed);
        return rc;
    }
    const int rc = L.family == 0
        ? gb_launch_reduce(L.kind, dtype, op, /*codec=*/0, &e.team, &L.args, L.grid, static_cast<cudaStream_t>(stream))
        : gb_launch_copy(L.kind, &e.team, &L.args, L.grid, static_cast<cudaStream_t>(stream));
    if (rc == 0) e.launches.fetch_add(1, std::memory_order_relaxed);
    return rc;
}
}  // namespace

extern "C" int gb_engine_all_reduce(void* engine, const void* in, void* out, size_t n, int dtype, int op,
                                    int divide, int grid_cap, void* stream) {
    GbLaunch L;
    const int rc = gb_engine_prepare_all_reduce(engine, in, out, n, dtype, op, divide, grid_cap, &L);
    return rc != GB_ENGINE_OK ? rc : launch(*static_cast<Engine*>(engine), L, dtype, op, stream);
}

extern "C" int gb_engine_reduce_scatter(void* engine, const void* in, void* out, size_t n_out, int dtype,
                                        int divide, int grid_cap, void* stream) {
    GbLaunch L;
    const int rc = gb_engine_prepare_reduce_scatter(engine, in, out, n_out, dtype, divide, grid_cap, &L);
    return rc != GB_ENGINE_OK ? rc : launch(*static_cast<Engine*>(engine), L, dtype, /*op=*/0, stream);
}

extern "C" int gb_engine_all_gather(void* engine, const void* in, void* out, size_t in_bytes, int grid_cap,
                                    void* stream) {
    GbLaunch L;
    const int rc = gb_engine_prepare_all_gather(engine, in, out, in_bytes, grid_cap, &L);
    return rc != GB_ENGINE_OK ? rc : launch(*static_cast<Engine*>(engine), L, 0, 0, stream);
}

extern "C" int gb_engine_broadcast(void* engine, void* buffer, size_t nbytes, int root, int grid_cap,
                                   void* stream) {
    GbLaunch L;
    const int rc = gb_engine_prepare_broadcast(engine, buffer, nbytes, root, grid_cap, &L);
    return rc != GB_ENGINE_OK ? rc : launch(*static_cast<Engine*>(engine), L, 0, 0, stream);
}

extern "C" int gb_engine_barrier(void* engine, void* stream) {
    GbLaunch L;
    std::memset(&L, 0, sizeof(L));
    L.family = 1;
    L.kind = 2;
    L.grid = 1;
    return launch(*static_cast<Engine*>(engine), L, 0, 0, stream);
}
