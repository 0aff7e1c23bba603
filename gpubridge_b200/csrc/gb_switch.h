// The in-switch all-reduce (gb_switch.cu): what host code and the kernel share.
#pragma once
#include <cstddef>

#define GB_SWITCH_MAX_BLOCKS 320                 // rows of the per-block flag area
#define GB_SWITCH_MAX_TILE (256u << 10)          // bytes of one tile of the pipeline

// The one-step all-reduce keeps two halves of fixed per-block slots BEHIND `bytes` of a group's
// switch memory (the host reserves them: GbSwitch::bytes excludes this tail).
#define GB_SWITCH_ONESHOT_SLOT (32u << 10)       // bytes of one block's slot
#define GB_SWITCH_ONESHOT_BLOCKS 128             // slots per half (more blocks cost more at the barrier than they gain)
#define GB_SWITCH_ONESHOT_RESERVE (2u * GB_SWITCH_ONESHOT_SLOT * GB_SWITCH_ONESHOT_BLOCKS)   // 8 MiB

// One rank's view of the switch memory of its group (the team, or its island).
struct GbSwitch {
    char* uc;                 // this rank's memory bound to the group's multicast object
    char* mc;                 // the multicast address of that memory on every member
    size_t bytes;             // size of the bound memory
    size_t off_flags;         // in the team's workspaces: [GB_SWITCH_MAX_BLOCKS][GB_MAX_RANKS] flags
    size_t off_bridge;        // in the team's workspaces: the islands' sums of a stripe (hier only)
    size_t len_bridge;
    unsigned int* bseq;       // local: the last barrier number of every block index
    int group_size;           // members of the group
    int group_pos;            // this rank's position in it
    int owners;               // members that reduce a stripe: positions 0 .. owners - 1
    int hier;                 // 1: the group is an island of a team of several; bridge between them
};

struct GbSwitchPlan {
    size_t tile;              // bytes; a multiple of 128 * owners
    int ntiles;
    int grid;
};

struct SwArgs {
    const char* in;
    char* out;
    size_t nbytes;
    size_t tile;
    int ntiles;
    int divide;
};

// The copy-shaped collectives through the switch (reduce-scatter, all-gather, broadcast).
struct SwCopyArgs {
    const char* in;
    char* out;
    size_t piece;             // bytes of one member's piece (broadcast: of the whole tensor)
    size_t tile;              // bytes of one piece's share of a staging buffer; a multiple of 128
    int ntiles;               // tiles per piece
    int nsub;                 // pieces per staging buffer: the team size (broadcast: 1)
    int divide;               // reduce-scatter: > 0 divides the sum
    int root;                 // broadcast: the team rank that has the data
};
