// The host-side engine of one team: from a tensor to a kernel launch without Python.
//
// The planner (channels, chunking, regions, grid) and the launch of every fused collective,
// behind a C ABI with an opaque handle, so that a C++ front end (the c10d backend) issues a
// collective on a CUDA stream in a few hundred nanoseconds of host time.  The arithmetic is
// the same as the Python planner's (ops/fabric.py), and a CPU test holds the two together:
// every rank of a team must come out with the same plan whichever side computed it.
#pragma once
#include <cstddef>
#include "gb_args.h"

struct GbTeam;

struct GbEngineConfig {
    size_t ws_bytes;
    int k, m_max;                       // smallest and largest island of the team
    int max_blocks, copy_blocks, scatter_blocks, overlap_blocks;
    int ring;                           // 0 register loads, 1 bulk-copy ring (job queue), 2 ring (phased)
    int two_shot;                       // two-shot bridge between three or more islands
    int force_chunks, force_channels;   // 0 = planned
    int algo;                           // 0 auto, 1 one-shot whenever it fits, 2 never one-shot
    size_t oneshot_slot, off_oneshot, len_oneshot;
    size_t off_ha, len_ha, off_hb, len_hb, off_hc, len_hc;
    size_t off_rs, len_rs, rs_chunk_bytes;
    size_t off_ag, len_ag, ag_chunk_bytes;
    size_t off_bc, len_bc, bc_stripe_bytes;
};

struct GbLaunch {                       // what a prepare call decided
    int family;                         // 0 gb_launch_reduce, 1 gb_launch_copy, 2 in-switch all-reduce
    int kind, grid;                     // family 2: kind 1 = hierarchical order, grid = block limit
    GbArgs args;
};

struct GbHierPlanOut { int channels, grid; size_t stripe, nchunks, len_a, len_b, len_c; };

enum { GB_ENGINE_OK = 0, GB_ENGINE_UNSUPPORTED = -1, GB_ENGINE_WORKSPACE = -2 };

extern "C" {
// Pure arithmetic; returns GB_ENGINE_WORKSPACE when a stripe does not fit the workspace.
int gb_plan_hier(size_t n, int esize, int k, int m_max, int n_islands, size_t len_ha, size_t len_hb,
                 size_t len_hc, int grid, size_t chunk_bytes, int force_channels, int force_chunks,
                 int stripe_multiple, GbHierPlanOut* out);

void* gb_engine_create(const GbTeam* team, const GbEngineConfig* config);
void gb_engine_destroy(void* engine);
struct GbSwitch;
void gb_engine_set_switch(void* engine, const GbSwitch* team, const GbSwitch* island, size_t min_bytes,
                          int min_ranks);
unsigned long long gb_engine_launches(void* engine);
size_t gb_sizeof_engine_config();
size_t gb_sizeof_launch();

// prepare_*: fill `launch` without touching the device.  grid_cap <= 0: the team's full grid.
// Return GB_ENGINE_OK, or a negative code when this call must take another path.
int gb_engine_prepare_all_reduce(void* engine, const void* in, void* out, size_t n, int dtype, int op,
                                 int divide, int grid_cap, GbLaunch* launch);
int gb_engine_prepare_reduce_scatter(void* engine, const void* in, void* out, size_t n_out, int dtype,
                                     int divide, int grid_cap, GbLaunch* launch);
int gb_engine_prepare_all_gather(void* engine, const void* in, void* out, size_t in_bytes,
                                 int grid_cap, GbLaunch* launch);
int gb_engine_prepare_broadcast(void* engine, void* buffer, size_t nbytes, int root, int grid_cap,
                                GbLaunch* launch);

// The same, then the launch on `stream` (a cudaStream_t).  Return GB_ENGINE_* (< 0) or a cudaError_t.
int gb_engine_all_reduce(void* engine, const void* in, void* out, size_t n, int dtype, int op,
                         int divide, int grid_cap, void* stream);
int gb_engine_reduce_scatter(void* engine, const void* in, void* out, size_t n_out, int dtype,
                             int divide, int grid_cap, void* stream);
int gb_engine_all_gather(void* engine, const void* in, void* out, size_t in_bytes, int grid_cap,
                         void* stream);
int gb_engine_broadcast(void* engine, void* buffer, size_t nbytes, int root, int grid_cap, void* stream);
int gb_engine_barrier(void* engine, void* stream);
// 0 while no device-side wait of this team has run out, else the status code the kernel left.
unsigned int gb_engine_status(void* engine);
}
