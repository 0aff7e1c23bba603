// Arguments of one collective launch (plain data: host code and kernels share it).
#pragma once
#include <cstddef>

struct GbArgs {
    const void* in;
    void* out;
    size_t n;                 // elements (all-reduce, reduce-scatter: per slice) or bytes (copies)
    size_t chunk;             // elements / bytes per chunk
    size_t stripe;            // elements per stripe of a chunk (a multiple of 256)
    int k;                    // stripes per chunk
    int divide;               // > 0: divide the sum by it (AVG)
    int root;                 // broadcast source (team rank)
    int role_a;               // all-reduce: channels (0 = 1); reduce-scatter: blocks that store
    int role_b;               // all-reduce: 1 = two-shot bridge between three or more islands
    int pad;
    size_t off_a, off_b, off_c;   // regions
    size_t len_a, len_b, len_c;   // bytes of one buffer of each region
    float* residual;          // error feedback of this rank's stripes (compressed all-reduce)
    char* sym;                // NVLS all-reduce: this rank's multicast-bound buffer ...
    char* mc;                 // ... and the multicast address of the same buffer on every rank
    size_t keep_lo, keep_n;   // hierarchical all-reduce: the element range this rank wants in `out`
                              // (out[0] is element keep_lo); keep_n = 0: the whole tensor
};
