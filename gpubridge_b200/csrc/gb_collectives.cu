// Fused collectives over NVLink peer memory (sm_100a).
//
// Every kernel here is persistent (one wave of blocks), moves data with 16-byte loads and
// stores to and from the peers' symmetric workspaces, and separates its steps with
// gb_sync_all().  Summation order is fixed and the same on every rank: members of an
// island in rank order, the island result rounded to the tensor's dtype, island results in
// island order - so every rank ends with identical bits and integer-valued data is exact.
//
//   allreduce_oneshot  small tensors: every rank stores its tensor into a slot of every
//                      peer, one barrier, every rank reduces the slots locally.
//   allreduce_hier     the three-phase hierarchical all-reduce in one launch, software
//                      pipelined over chunks.  A chunk is k stripes (k = size of the smallest
//                      island); island member j owns stripe j.  Per chunk:
//                        A  every rank stores stripe j of its input into a slot of its
//                           island's owner j                            (island reduce)
//                        B  owner j reduces its island's slots and stores the island result
//                           - raw, bf16 or block-scaled fp8 with error feedback - into
//                           owner j of every island                     (bridge, send)
//                        C  owner j adds the island results in island order, applies AVG and
//                           rounds once                                 (bridge, reduce)
//                        D  every rank loads stripe j from its island's owner j into its
//                           output                                      (island broadcast)
//                      Iteration t runs A(t), B(t-1), C(t-2), D(t-3) and then one barrier, so
//                      the steps of neighbouring chunks share the links.  With one island B
//                      writes the result directly and C is skipped.
//   allgather          every rank stages its input, barrier, every rank loads every peer's.
//   reduce_scatter     every rank stores slice r into rank r, barrier, rank r reduces.
//   broadcast          the source scatters stripes over the ranks, barrier, all-gather.
//   barrier            gb_sync_all() alone.
//
// Buffer reuse.  A region written before a kernel's first barrier (one-shot slots, all-gather
// staging, reduce-scatter slots, broadcast stripes) has two copies selected by the parity of
// the team's collective counter; everything else is written only after a barrier of the same
// kernel, when every peer has left the previous collective.  Inside a pipelined kernel the
// two buffers of a region alternate with the chunk index.
#include "gb_codec.cuh"
#include "gb_bulk.cuh"

// Byte offsets are into a workspace; every offset and length is a multiple of 16.
#include "gb_args.h"

namespace {

constexpr int THREADS = 512;

template <typename T> struct Vec {
    static constexpr int N = 16 / sizeof(T);
    union { uint4 u; T e[16 / sizeof(T)]; };
};

__device__ __forceinline__ size_t round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }

// Values of stripe j of the chunk starting at c0 that lie inside the tensor.
__device__ __forceinline__ size_t stripe_valid(const GbArgs& a, size_t c0, int j) {
    const size_t s0 = c0 + (size_t)j * a.stripe;
    if (s0 >= a.n) return 0;
    const size_t left = a.n - s0;
    return left < a.stripe ? left : a.stripe;
}

// V results of type TO to dst: as 16-byte (or, for 8 bytes in all, one 8-byte) stores when
// `aligned` says dst + this vector is aligned to its own size, else one by one.
template <typename TO, int V>
__device__ __forceinline__ void store_results(TO* dst, const TO (&vals)[V], bool aligned) {
    constexpr int BYTES = V * (int)sizeof(TO);
    if (aligned && BYTES >= 16) {
        union { uint4 q[BYTES / 16 > 0 ? BYTES / 16 : 1]; TO e[V]; } pack;
        #pragma unroll
        for (int j = 0; j < V; ++j) pack.e[j] = vals[j];
        #pragma unroll
        for (int q = 0; q < BYTES / 16; ++q) gb_st16(reinterpret_cast<char*>(dst) + 16 * q, pack.q[q]);
    } else if (aligned && BYTES == 8) {
        union { uint2 q; TO e[V]; } pack;
        #pragma unroll
        for (int j = 0; j < V; ++j) pack.e[j] = vals[j];
        *reinterpret_cast<uint2*>(dst) = pack.q;
    } else {
        #pragma unroll
        for (int j = 0; j < V; ++j) dst[j] = vals[j];
    }
}

// Reduce local slots in hierarchical order into out[0 .. count).
//   slot s lives at slots + s * slot_bytes; island g is slot_of[bounds[g] .. bounds[g+1]).
// TO: the type of `out`; when it differs from T (float <-> bf16) the sum - island sums rounded
// to T, islands added in the accumulator type, divided - is rounded once, to TO.
template <typename T, int OP, typename TO = T>
__device__ __forceinline__ void reduce_slots(const GbLane& L, const char* slots, size_t slot_bytes,
                                             const int* slot_of, const int* bounds, int n_groups,
                                             size_t count, TO* out, int divide) {
    typedef typename GbAcc<T>::type A;
    constexpr int V = Vec<T>::N;
    const size_t tid = L.tid, nth = L.nth;
    const size_t nvec = count / V;
    const bool out_aligned = ((uintptr_t)out & (V * sizeof(TO) >= 16 ? 15u : V * sizeof(TO) - 1u)) == 0;
    // U vectors per thread and step, so U loads are in flight per slot (a single vector per
    // step leaves the loop bound by memory latency)
    constexpr int U = V >= 8 ? 4 : 8;
    for (size_t v0 = tid; v0 < nvec; v0 += (size_t)U * nth) {
        A total[U][V];
        for (int g = 0; g < n_groups; ++g) {
            A part[U][V];
            for (int s = bounds[g]; s < bounds[g + 1]; ++s) {
                Vec<T> w[U];
                const char* base = slots + (size_t)slot_of[s] * slot_bytes;
                #pragma unroll
                for (int u = 0; u < U; ++u) {
                    const size_t v = v0 + (size_t)u * nth;
                    if (v < nvec) w[u].u = gb_ld16(base + v * 16, L.ld);
                }
                #pragma unroll
                for (int u = 0; u < U; ++u) {
                    #pragma unroll
                    for (int j = 0; j < V; ++j)
                        part[u][j] = (s == bounds[g]) ? gb_up<T>(w[u].e[j])
                                     : GbFold<OP, A>::run(part[u][j], gb_up<T>(w[u].e[j]));
                }
            }
            #pragma unroll
            for (int u = 0; u < U; ++u) {
                #pragma unroll
                for (int j = 0; j < V; ++j) {
                    A rounded = gb_up<T>(gb_down<T>(part[u][j]));   // the island result, in T
                    total[u][j] = (g == 0) ? rounded : GbFold<OP, A>::run(total[u][j], rounded);
                }
            }
        }
        #pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t v = v0 + (size_t)u * nth;
            if (v >= nvec) continue;
            TO r[V];
            #pragma unroll
            for (int j = 0; j < V; ++j)
                r[j] = gb_down<TO>(divide > 0 ? gb_divide<A>(total[u][j], divide) : total[u][j]);
            store_results<TO, V>(out + v * V, r, out_aligned);
        }
    }
    // ragged tail: count is not a multiple of a 16-byte vector
    for (size_t i = nvec * V + tid; i < count; i += nth) {
        A total = A();
        for (int g = 0; g < n_groups; ++g) {
            A part = A();
            for (int s = bounds[g]; s < bounds[g + 1]; ++s) {
                const volatile unsigned char* p = reinterpret_cast<const volatile unsigned char*>(
                    slots + (size_t)slot_of[s] * slot_bytes + i * sizeof(T));
                union { T t; unsigned char b[sizeof(T)]; } cell;
                #pragma unroll
                for (unsigned q = 0; q < sizeof(T); ++q) cell.b[q] = p[q];
                A x = gb_up<T>(cell.t);
                part = (s == bounds[g]) ? x : GbFold<OP, A>::run(part, x);
            }
            A rounded = gb_up<T>(gb_down<T>(part));
            total = (g == 0) ? rounded : GbFold<OP, A>::run(total, rounded);
        }
        out[i] = gb_down<TO>(divide > 0 ? gb_divide<A>(total, divide) : total);
    }
}

// Zero [lo, hi) bytes of a 16-byte aligned buffer with the whole grid.
__device__ __forceinline__ void zero_range(const GbLane& L, char* base, size_t lo, size_t hi) {
    if (hi <= lo) return;
    const size_t tid = L.tid, nth = L.nth;
    size_t head = round_up(lo, 16);
    if (head > hi) head = hi;
    if (tid < head - lo) base[lo + tid] = 0;
    const size_t nv = (hi - head) >> 4;
    for (size_t i = tid; i < nv; i += nth) gb_st16(base + head + (i << 4), make_uint4(0, 0, 0, 0));
    for (size_t b = head + (nv << 4) + tid; b < hi; b += nth) base[b] = 0;
}

// ---- one-shot all-reduce ----------------------------------------------------------------------
// Region A: [2 parities][world slots] of len_a / world bytes each.
template <typename T, int OP>
__global__ void __launch_bounds__(THREADS)
allreduce_oneshot_kernel(GbTeam tm, GbArgs a) {
    const unsigned parity = gb_ld_volatile(&tm.ctrl->epoch) & 1u;
    const size_t nbytes = a.n * sizeof(T);
    const size_t base = a.off_a + parity * a.len_a;
    const size_t slot = a.len_a / (size_t)tm.world;
    const GbLane L = gb_lane_all(tm.ld_mode);
    for (int d = 0; d < tm.world; ++d) {
        const int peer = (tm.rank + d) % tm.world;
        gb_copy_bytes(L, tm.ws[peer] + base + (size_t)tm.rank * slot, a.in, nbytes, false);
    }
    if (!gb_sync_all(tm, 0, true)) return;
    reduce_slots<T, OP>(L, tm.ws[tm.rank] + base, slot, tm.order, tm.island_off, tm.n_islands,
                        a.n, static_cast<T*>(a.out), a.divide);
}

// ---- hierarchical all-reduce ------------------------------------------------------------------
// Region A: [2][island slots] of stripe bytes     (step A targets, on the owner)
// Region B: [2][n_islands] of payload bytes       (step B targets, on the owner)
// Region C: [2] of stripe bytes                   (step C output, on the owner)
template <typename T, int CODEC> __host__ __device__ inline size_t payload_bytes(size_t stripe) {
    if (CODEC == GB_RAW) return stripe * sizeof(T);
    if (CODEC == GB_C_BF16) return stripe * 2;
    return (stripe + 4 * (stripe / GbBlock<CODEC>::size) + 15) / 16 * 16;   // codes, then scales
}

template <typename T> __device__ __forceinline__ T coded_out(float v) { return (T)v; }
template <> __device__ __forceinline__ float coded_out<float>(float v) { return v; }
template <> __device__ __forceinline__ double coded_out<double>(float v) { return (double)v; }
template <> __device__ __forceinline__ __half coded_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 coded_out<__nv_bfloat16>(float v) {
    __nv_bfloat16_raw raw;
    raw.x = (unsigned short)gb_bf16_bits(v);
    return __nv_bfloat16(raw);
}

template <typename T> __device__ __forceinline__ float as_float_sat(T v, bool& finite) {
    float x = (float)gb_up<T>(v);
    finite = isfinite(x);
    return x;
}
template <> __device__ __forceinline__ float as_float_sat<double>(double v, bool& finite) {
    finite = isfinite(v);
    if (!finite) return (float)v;
    return __double2float_rn(fmin(fmax(v, -(double)GB_FLT_MAX), (double)GB_FLT_MAX));
}

// Step B without compression: reduce the island's slots, round to T, store into every owner
// (or, with a single island, straight into the result buffer with AVG applied).
template <typename T, int OP>
__device__ __forceinline__ void island_reduce_raw(const GbLane& L, const GbTeam& tm,
                                                  const GbArgs& a, const char* slots,
                                                  size_t count, int buf) {
    typedef typename GbAcc<T>::type A;
    constexpr int V = Vec<T>::N;
    const int m = tm.island_off[tm.my_island + 1] - tm.island_off[tm.my_island];
    const bool bridged = tm.n_islands > 1;
    const size_t sbytes = a.stripe * sizeof(T);
    const size_t tid = L.tid, nth = L.nth;
    const size_t nvec = count / V;                       // count is a multiple of 256
    constexpr int U = V >= 8 ? 4 : 8;                    // vectors in flight per thread
    for (size_t v0 = tid; v0 < nvec; v0 += (size_t)U * nth) {
        A part[U][V];
        for (int p = 0; p < m; ++p) {
            Vec<T> w[U];
            #pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t v = v0 + (size_t)u * nth;
                if (v < nvec) w[u].u = gb_ld16(slots + (size_t)p * sbytes + v * 16, L.ld);
            }
            #pragma unroll
            for (int u = 0; u < U; ++u) {
                #pragma unroll
                for (int j = 0; j < V; ++j)
                    part[u][j] = (p == 0) ? gb_up<T>(w[u].e[j])
                                 : GbFold<OP, A>::run(part[u][j], gb_up<T>(w[u].e[j]));
            }
        }
        #pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t v = v0 + (size_t)u * nth;
            if (v >= nvec) continue;
            Vec<T> r;
            #pragma unroll
            for (int j = 0; j < V; ++j) r.e[j] = gb_down<T>(part[u][j]);
            if (!bridged) {
                if (a.divide > 0) {
                    #pragma unroll
                    for (int j = 0; j < V; ++j)
                        r.e[j] = gb_down<T>(gb_divide<A>(gb_up<T>(r.e[j]), a.divide));
                }
                gb_st16(tm.ws[tm.rank] + a.off_c + (size_t)buf * a.len_c + v * 16, r.u);
            } else {
                for (int d = 0; d < tm.n_islands; ++d) {
                    const int isl = (tm.my_island + d) % tm.n_islands;
                    const int owner = tm.order[tm.island_off[isl] + tm.my_pos];
                    gb_st16(tm.ws[owner] + a.off_b + (size_t)buf * a.len_b
                            + (size_t)tm.my_island * sbytes + v * 16, r.u);
                }
            }
        }
    }
}

// EPL consecutive values of type T, read past L1, as floats (saturated for double).
template <typename T, int EPL>
__device__ __forceinline__ void load_run(const T* src, float (&x)[EPL], bool (&fin)[EPL], bool first,
                                         float (&acc)[EPL]) {
    constexpr int BYTES = EPL * (int)sizeof(T);
    union { uint4 q[(BYTES + 15) / 16]; uint2 d; T e[EPL]; } w;
    if (BYTES >= 16) {
        #pragma unroll
        for (int g = 0; g < BYTES / 16; ++g) w.q[g] = gb_ld16(reinterpret_cast<const char*>(src) + 16 * g);
    } else {
        asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];"
                     : "=r"(w.d.x), "=r"(w.d.y) : "l"(src) : "memory");
    }
    #pragma unroll
    for (int j = 0; j < EPL; ++j) {
        x[j] = as_float_sat<T>(w.e[j], fin[j]);
        acc[j] = first ? x[j] : __fadd_rn(acc[j], x[j]);
    }
}

// Step B with compression: one warp per quantisation block; payload = codes, then scales.
template <typename T, int CODEC>
__device__ __forceinline__ void island_reduce_coded(const GbLane& L, const GbTeam& tm,
                                                    const GbArgs& a, const char* slots,
                                                    size_t count, int buf, float* residual) {
    constexpr int BS = GbBlock<CODEC>::size;
    constexpr int EPL = BS / 32;
    const int m = tm.island_off[tm.my_island + 1] - tm.island_off[tm.my_island];
    const size_t sbytes = a.stripe * sizeof(T);
    const size_t pbytes = payload_bytes<T, CODEC>(a.stripe);
    const int lane = threadIdx.x & 31;
    const size_t warp = L.tid >> 5;
    const size_t nwarps = L.nth >> 5;
    const size_t nblk = count / BS;
    for (size_t blk = warp; blk < nblk; blk += nwarps) {
        const size_t i0 = blk * BS + (size_t)lane * EPL;
        float v[EPL], acc[EPL]; bool fin[EPL];
        for (int p = 0; p < m; ++p)
            load_run<T, EPL>(reinterpret_cast<const T*>(slots + (size_t)p * sbytes) + i0, v, fin,
                             p == 0, acc);
        float amax = 0.0f;
        #pragma unroll
        for (int j = 0; j < EPL; ++j) {
            // the island result in T, as the uncompressed path would hand it to the bridge
            bool xf;
            float x = as_float_sat<T>(gb_down<T>((typename GbAcc<T>::type)acc[j]), xf);
            bool f;
            v[j] = gb_prepare(x, xf, residual[i0 + j], f);
            fin[j] = f;
            if (f) amax = fmaxf(amax, fabsf(v[j]));
        }
        if (CODEC == GB_C_BF16) {
            unsigned words[EPL / 2];
            #pragma unroll
            for (int j = 0; j < EPL; ++j) {
                unsigned code = gb_bf16_code(v[j], fin[j]);
                residual[i0 + j] = fin[j] ? __fsub_rn(v[j], gb_from_bf16_bits(code)) : 0.0f;
                if (j & 1) words[j / 2] |= code << 16; else words[j / 2] = code;
            }
            for (int d = 0; d < tm.n_islands; ++d) {
                const int isl = (tm.my_island + d) % tm.n_islands;
                const int owner = tm.order[tm.island_off[isl] + tm.my_pos];
                char* dst = tm.ws[owner] + a.off_b + (size_t)buf * a.len_b
                            + (size_t)tm.my_island * pbytes + i0 * 2;
                gb_st16(dst, make_uint4(words[0], words[1], words[2], words[3]));
            }
        } else {
            amax = gb_warp_max(amax);
            float scale, mult;
            gb_block_scale<CODEC>(amax, scale, mult);
            unsigned words[2] = {0u, 0u};
            #pragma unroll
            for (int j = 0; j < EPL; ++j) {
                unsigned code = fin[j] ? gb_e4m3_encode(__fmul_rn(v[j], mult)) : 0x7Fu;
                float sent = __fmul_rn(gb_e4m3_decode(code), scale);
                residual[i0 + j] = fin[j] ? __fsub_rn(v[j], sent) : 0.0f;
                words[j / 4] |= code << (8 * (j & 3));
            }
            for (int d = 0; d < tm.n_islands; ++d) {
                const int isl = (tm.my_island + d) % tm.n_islands;
                const int owner = tm.order[tm.island_off[isl] + tm.my_pos];
                char* dst = tm.ws[owner] + a.off_b + (size_t)buf * a.len_b
                            + (size_t)tm.my_island * pbytes;
                if (EPL == 8) *reinterpret_cast<uint2*>(dst + i0) = make_uint2(words[0], words[1]);
                else *reinterpret_cast<unsigned*>(dst + i0) = words[0];
                if (lane == 0) reinterpret_cast<float*>(dst + a.stripe)[blk] = scale;
            }
        }
    }
}

// Step C: add the island results in island order, AVG, round once, into region C.
template <typename T, int OP, int CODEC>
__device__ __forceinline__ void bridge_reduce(const GbLane& L, const GbTeam& tm, const GbArgs& a,
                                              size_t count, int buf) {
    typedef typename GbAcc<T>::type A;
    constexpr int V = Vec<T>::N;
    const size_t tid = L.tid, nth = L.nth;
    const size_t pbytes = payload_bytes<T, CODEC>(a.stripe);
    const char* parts = tm.ws[tm.rank] + a.off_b + (size_t)buf * a.len_b;
    char* result = tm.ws[tm.rank] + a.off_c + (size_t)buf * a.len_c;
    const size_t nvec = count / V;
    if (CODEC == GB_RAW) {
        constexpr int U = V >= 8 ? 4 : 8;
        for (size_t v0 = tid; v0 < nvec; v0 += (size_t)U * nth) {
            A total[U][V];
            for (int g = 0; g < tm.n_islands; ++g) {
                Vec<T> w[U];
                #pragma unroll
                for (int u = 0; u < U; ++u) {
                    const size_t v = v0 + (size_t)u * nth;
                    if (v < nvec) w[u].u = gb_ld16(parts + (size_t)g * pbytes + v * 16, L.ld);
                }
                #pragma unroll
                for (int u = 0; u < U; ++u) {
                    #pragma unroll
                    for (int j = 0; j < V; ++j)
                        total[u][j] = (g == 0) ? gb_up<T>(w[u].e[j])
                                      : GbFold<OP, A>::run(total[u][j], gb_up<T>(w[u].e[j]));
                }
            }
            #pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t v = v0 + (size_t)u * nth;
                if (v >= nvec) continue;
                Vec<T> r;
                #pragma unroll
                for (int j = 0; j < V; ++j)
                    r.e[j] = gb_down<T>(a.divide > 0 ? gb_divide<A>(total[u][j], a.divide)
                                                     : total[u][j]);
                gb_st16(result + v * 16, r.u);
            }
        }
        return;
    }
    for (size_t v = tid; v < nvec; v += nth) {
        Vec<T> r;
        {
            float acc[V];
            #pragma unroll
            for (int j = 0; j < V; ++j) acc[j] = 0.0f;
            const size_t e0 = v * V;
            for (int g = 0; g < tm.n_islands; ++g) {
                const char* row = parts + (size_t)g * pbytes;
                if (CODEC == GB_C_BF16) {
                    #pragma unroll
                    for (int j = 0; j < V; j += 2) {
                        unsigned w = *reinterpret_cast<const volatile unsigned*>(row + (e0 + j) * 2);
                        acc[j] = gb_flush(__fadd_rn(acc[j], gb_from_bf16_bits(w & 0xFFFFu)));
                        acc[j + 1] = gb_flush(__fadd_rn(acc[j + 1], gb_from_bf16_bits(w >> 16)));
                    }
                } else {
                    const float scale = reinterpret_cast<const volatile float*>(row + a.stripe)
                        [e0 / GbBlock<CODEC>::size];
                    if (V >= 4) {
                        #pragma unroll
                        for (int j = 0; j < V; j += 4) {
                            unsigned w = *reinterpret_cast<const volatile unsigned*>(row + e0 + j);
                            #pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                if (j + q < V) {
                                    float d = __fmul_rn(gb_e4m3_decode((w >> (8 * q)) & 0xFFu), scale);
                                    acc[j + q] = gb_flush(__fadd_rn(acc[j + q], d));
                                }
                            }
                        }
                    } else {                              // double: two codes per vector
                        #pragma unroll
                        for (int j = 0; j < V; ++j) {
                            unsigned c = *reinterpret_cast<const volatile unsigned char*>(row + e0 + j);
                            float d = __fmul_rn(gb_e4m3_decode(c), scale);
                            acc[j] = gb_flush(__fadd_rn(acc[j], d));
                        }
                    }
                }
            }
            #pragma unroll
            for (int j = 0; j < V; ++j)
                r.e[j] = coded_out<T>(a.divide > 0 ? __fdiv_rn(acc[j], (float)a.divide) : acc[j]);
        }
        gb_st16(result + v * 16, r.u);
    }
}

template <typename T, int OP, int CODEC>
__global__ void __launch_bounds__(THREADS)
allreduce_hier_kernel(GbTeam tm, GbArgs a) {
    const T* in = static_cast<const T*>(a.in);
    T* out = static_cast<T*>(a.out);
    const bool owner = tm.my_pos < a.k;
    const bool bridged = tm.n_islands > 1;
    const size_t sbytes = a.stripe * sizeof(T);
    const long nchunks = (long)((a.n + a.chunk - 1) / a.chunk);
    const int depth = bridged ? 3 : 2;                   // iterations between A and D
    // Channels: the grid is cut into `channels` equal groups of blocks.  Channel c takes the
    // chunks c, c + channels, ... through its own pipeline, with its own barrier (control
    // block and flag row c) and its own buffers, so while one channel sits in a barrier or
    // reduces locally the others keep the links busy.
    const int channels = a.role_a > 0 ? a.role_a : 1;
    const int per = (int)gridDim.x / channels;
    const int ch = (int)blockIdx.x / per;
    if (ch >= channels) return;                          // grid not a multiple: idle blocks
    const GbLane L = gb_lane_blocks(ch * per, per, tm.ld_mode);
    const long mine = nchunks > ch ? (nchunks - ch + channels - 1) / channels : 0;
    if (mine == 0) return;
    const long iters = mine + depth;
    const size_t off_a = a.off_a + (size_t)ch * 2 * a.len_a;
    const size_t off_b = a.off_b + (size_t)ch * 2 * a.len_b;
    const size_t off_c = a.off_c + (size_t)ch * 2 * a.len_c;
    GbArgs b = a;                                        // this channel's regions
    b.off_a = off_a; b.off_b = off_b; b.off_c = off_c;
    for (long i = 0; i < iters; ++i) {
        if (i < mine) {                                  // A(i)
            const size_t c0 = (size_t)(ch + i * channels) * a.chunk;
            for (int dj = 0; dj < a.k; ++dj) {
                const int j = (tm.my_pos + dj) % a.k;
                const int own = tm.order[tm.island_off[tm.my_island] + j];
                char* dst = tm.ws[own] + off_a + (size_t)(i & 1) * a.len_a
                            + (size_t)tm.my_pos * sbytes;
                const size_t valid = stripe_valid(a, c0, j);
                if (valid)
                    gb_copy_bytes(L, dst, in + c0 + (size_t)j * a.stripe, valid * sizeof(T), false);
                // zeros up to the next quantisation block: padding reduces only with padding
                zero_range(L, dst, valid * sizeof(T), round_up(valid, 256) * sizeof(T));
            }
        }
        if (owner && i >= 1 && i - 1 < mine) {           // B(i-1)
            const long c = ch + (i - 1) * channels;
            const size_t need = round_up(stripe_valid(a, (size_t)c * a.chunk, tm.my_pos), 256);
            const char* slots = tm.ws[tm.rank] + off_a + (size_t)((i - 1) & 1) * a.len_a;
            if (CODEC == GB_RAW)
                island_reduce_raw<T, OP>(L, tm, b, slots, need, (int)((i - 1) & 1));
            else
                island_reduce_coded<T, CODEC>(L, tm, b, slots, need, (int)((i - 1) & 1),
                                              a.residual + (size_t)c * a.stripe);
        }
        if (bridged && owner && i >= 2 && i - 2 < mine) {        // C(i-2)
            const long c = ch + (i - 2) * channels;
            const size_t need = round_up(stripe_valid(a, (size_t)c * a.chunk, tm.my_pos), 256);
            bridge_reduce<T, OP, CODEC>(L, tm, b, need, (int)((i - 2) & 1));
        }
        if (i >= depth) {                                // D(i-depth)
            const long c = ch + (i - depth) * channels;
            const size_t c0 = (size_t)c * a.chunk;
            for (int dj = 0; dj < a.k; ++dj) {
                const int j = (tm.my_pos + dj) % a.k;
                const int own = tm.order[tm.island_off[tm.my_island] + j];
                const size_t valid = stripe_valid(a, c0, j);
                if (!valid) continue;
                // A reduce-scatter keeps only its own slice of the result: the part of this
                // stripe inside [keep_lo, keep_lo + keep_n) goes to out[element - keep_lo].
                const size_t s0 = c0 + (size_t)j * a.stripe;
                const size_t keep_hi = a.keep_n ? a.keep_lo + a.keep_n : a.n;
                const size_t lo = s0 > a.keep_lo ? s0 : a.keep_lo;
                const size_t hi = s0 + valid < keep_hi ? s0 + valid : keep_hi;
                if (lo < hi)
                    gb_copy_bytes(L, out + (lo - a.keep_lo),
                                  tm.ws[own] + off_c + (size_t)((i - depth) & 1) * a.len_c
                                  + (lo - s0) * sizeof(T),
                                  (hi - lo) * sizeof(T), true);
            }
        }
        if (i + 1 < iters &&
            !gb_sync(tm, ch, (unsigned)per, (unsigned)(i < 7 ? i : 7), i == 0 && ch == 0))
            return;
    }
}

// ---- hierarchical all-reduce through the bulk-copy ring -----------------------------------------
// The same steps, buffers and summation order as allreduce_hier_kernel without compression;
// every read (input stripes, island slots, island results, the owner's result) is a bulk copy
// into shared memory issued ahead of its use, every write an ordinary store from there.

// One tile of step B: fold the island's slots in member order, round to T, store.
template <typename T, int OP>
__device__ __forceinline__ void island_reduce_tile(const GbTeam& tm, const GbArgs& a, int buf,
                                                   const unsigned char* stage, unsigned pitch,
                                                   size_t off, unsigned len) {
    typedef typename GbAcc<T>::type A;
    constexpr int V = Vec<T>::N;
    const int m = tm.island_off[tm.my_island + 1] - tm.island_off[tm.my_island];
    const bool bridged = tm.n_islands > 1;
    const size_t sbytes = a.stripe * sizeof(T);
    const unsigned nv = len >> 4;
    for (unsigned v = threadIdx.x; v < nv; v += THREADS) {
        A part[V];
        for (int p = 0; p < m; ++p) {
            Vec<T> w;
            w.u = *reinterpret_cast<const uint4*>(stage + (size_t)p * pitch + ((size_t)v << 4));
            #pragma unroll
            for (int j = 0; j < V; ++j)
                part[j] = (p == 0) ? gb_up<T>(w.e[j]) : GbFold<OP, A>::run(part[j], gb_up<T>(w.e[j]));
        }
        Vec<T> r;
        #pragma unroll
        for (int j = 0; j < V; ++j) r.e[j] = gb_down<T>(part[j]);
        const size_t at = off + ((size_t)v << 4);
        if (!bridged) {
            if (a.divide > 0) {
                #pragma unroll
                for (int j = 0; j < V; ++j)
                    r.e[j] = gb_down<T>(gb_divide<A>(gb_up<T>(r.e[j]), a.divide));
            }
            gb_st16(tm.ws[tm.rank] + a.off_c + (size_t)buf * a.len_c + at, r.u);
        } else {
            for (int d = 0; d < tm.n_islands; ++d) {
                const int isl = (tm.my_island + d) % tm.n_islands;
                const int owner = tm.order[tm.island_off[isl] + tm.my_pos];
                gb_st16(tm.ws[owner] + a.off_b + (size_t)buf * a.len_b
                        + (size_t)tm.my_island * sbytes + at, r.u);
            }
        }
    }
}

// One tile of step C: add the island results in island order, AVG, one rounding, into region C.
template <typename T, int OP>
__device__ __forceinline__ void bridge_reduce_tile(const GbTeam& tm, const GbArgs& a, int buf,
                                                   const unsigned char* stage, unsigned pitch,
                                                   size_t off, unsigned len) {
    typedef typename GbAcc<T>::type A;
    constexpr int V = Vec<T>::N;
    char* result = tm.ws[tm.rank] + a.off_c + (size_t)buf * a.len_c;
    const int groups = tm.n_islands;
    const unsigned nv = len >> 4;
    for (unsigned v = threadIdx.x; v < nv; v += THREADS) {
        A total[V];
        for (int g = 0; g < groups; ++g) {
            Vec<T> w;
            w.u = *reinterpret_cast<const uint4*>(stage + (size_t)g * pitch + ((size_t)v << 4));
            #pragma unroll
            for (int j = 0; j < V; ++j)
                total[j] = (g == 0) ? gb_up<T>(w.e[j]) : GbFold<OP, A>::run(total[j], gb_up<T>(w.e[j]));
        }
        Vec<T> r;
        #pragma unroll
        for (int j = 0; j < V; ++j)
            r.e[j] = gb_down<T>(a.divide > 0 ? gb_divide<A>(total[j], a.divide) : total[j]);
        gb_st16(result + off + ((size_t)v << 4), r.u);
    }
}

__device__ __forceinline__ void copy_tile(char* dst, const unsigned char* stage, size_t off,
                                          unsigned len) {
    const unsigned nv = len >> 4;
    char* out = dst + off;
    for (unsigned v = threadIdx.x; v < nv; v += THREADS)
        gb_st16(out + ((size_t)v << 4), *reinterpret_cast<const uint4*>(stage + ((size_t)v << 4)));
}

enum { JOB_COPY = 0, JOB_ISLAND = 1, JOB_BRIDGE = 2 };

__device__ __forceinline__ void job_set(GbJob& job, int kind, const char* src, size_t stride, int m,
                                        size_t bytes, char* dst, int arg) {
    job.kind = kind; job.src = src; job.src_stride = stride; job.m = m; job.bytes = bytes;
    job.dst = dst; job.arg = arg;
}

template <typename T, int OP>
__global__ void __launch_bounds__(THREADS)
allreduce_ring_kernel(GbTeam tm, GbArgs a) {
    __shared__ GbJob jobs[GB_MAX_JOBS];
    __shared__ int njobs;
    GbRing R = gb_ring_init();
    const T* in = static_cast<const T*>(a.in);
    T* out = static_cast<T*>(a.out);
    const bool owner = tm.my_pos < a.k;
    const bool bridged = tm.n_islands > 1;
    const size_t sbytes = a.stripe * sizeof(T);
    const long nchunks = (long)((a.n + a.chunk - 1) / a.chunk);
    const int depth = bridged ? 3 : 2;
    const int channels = a.role_a > 0 ? a.role_a : 1;
    const int per = (int)gridDim.x / channels;
    const int ch = (int)blockIdx.x / per;
    if (ch >= channels) return;
    const int bi = (int)blockIdx.x - ch * per;
    const GbLane L = gb_lane_blocks(ch * per, per, tm.ld_mode);
    const long mine = nchunks > ch ? (nchunks - ch + channels - 1) / channels : 0;
    if (mine == 0) return;
    const long iters = mine + depth;
    const int members = tm.island_off[tm.my_island + 1] - tm.island_off[tm.my_island];
    GbArgs b = a;                                        // this channel's regions
    b.off_a = a.off_a + (size_t)ch * 2 * a.len_a;
    b.off_b = a.off_b + (size_t)ch * 2 * a.len_b;
    b.off_c = a.off_c + (size_t)ch * 2 * a.len_c;
    for (long i = 0; i < iters; ++i) {
        const bool do_a = i < mine;
        const bool do_b = owner && i >= 1 && i - 1 < mine;
        const bool do_c = bridged && owner && i >= 2 && i - 2 < mine;
        const bool do_d = i >= depth;
        const size_t a0 = (size_t)(ch + i * channels) * a.chunk;          // chunk of step A
        const size_t d0 = (size_t)(ch + (i - depth) * channels) * a.chunk; // chunk of step D
        __syncthreads();                                 // the last queue is no longer read
        if (threadIdx.x == 0) {
            int n = 0;
            if (do_d) {
                for (int dj = 0; dj < a.k; ++dj) {
                    const int j = (tm.my_pos + dj) % a.k;
                    const int own = tm.order[tm.island_off[tm.my_island] + j];
                    const size_t body = (stripe_valid(a, d0, j) * sizeof(T)) & ~(size_t)15;
                    if (body)
                        job_set(jobs[n++], JOB_COPY,
                                tm.ws[own] + b.off_c + (size_t)((i - depth) & 1) * a.len_c, 0, 1, body,
                                reinterpret_cast<char*>(out + d0 + (size_t)j * a.stripe), 0);
                }
            }
            if (do_c) {
                const long c = ch + (i - 2) * channels;
                const size_t need = round_up(stripe_valid(a, (size_t)c * a.chunk, tm.my_pos), 256);
                if (need)
                    job_set(jobs[n++], JOB_BRIDGE,
                            tm.ws[tm.rank] + b.off_b + (size_t)((i - 2) & 1) * a.len_b, sbytes,
                            tm.n_islands, need * sizeof(T), nullptr, (int)((i - 2) & 1));
            }
            if (do_b) {
                const long c = ch + (i - 1) * channels;
                const size_t need = round_up(stripe_valid(a, (size_t)c * a.chunk, tm.my_pos), 256);
                if (need)
                    job_set(jobs[n++], JOB_ISLAND,
                            tm.ws[tm.rank] + b.off_a + (size_t)((i - 1) & 1) * a.len_a, sbytes,
                            members, need * sizeof(T), nullptr, (int)((i - 1) & 1));
            }
            if (do_a) {
                for (int dj = 0; dj < a.k; ++dj) {
                    const int j = (tm.my_pos + dj) % a.k;
                    const int own = tm.order[tm.island_off[tm.my_island] + j];
                    const size_t body = (stripe_valid(a, a0, j) * sizeof(T)) & ~(size_t)15;
                    if (body)
                        job_set(jobs[n++], JOB_COPY,
                                reinterpret_cast<const char*>(in + a0 + (size_t)j * a.stripe), 0, 1,
                                body, tm.ws[own] + b.off_a + (size_t)(i & 1) * a.len_a
                                      + (size_t)tm.my_pos * sbytes, 0);
                }
            }
            gb_jobs_plan(jobs, n, per);
            njobs = n;
        }
        __syncthreads();
        // what the copy engine cannot take: ends shorter than 16 bytes, and the zero padding
        // up to the next quantisation block (padding reduces only with padding)
        if (do_a) {
            for (int j = 0; j < a.k; ++j) {
                const int own = tm.order[tm.island_off[tm.my_island] + j];
                char* dst = tm.ws[own] + b.off_a + (size_t)(i & 1) * a.len_a
                            + (size_t)tm.my_pos * sbytes;
                const size_t vb = stripe_valid(a, a0, j) * sizeof(T);
                const size_t body = vb & ~(size_t)15;
                if (vb > body)
                    gb_copy_bytes(L, dst + body,
                                  reinterpret_cast<const char*>(in + a0 + (size_t)j * a.stripe) + body,
                                  vb - body, false);
                zero_range(L, dst, vb, round_up(vb / sizeof(T), 256) * sizeof(T));
            }
        }
        if (do_d) {
            for (int j = 0; j < a.k; ++j) {
                const int own = tm.order[tm.island_off[tm.my_island] + j];
                const size_t vb = stripe_valid(a, d0, j) * sizeof(T);
                const size_t body = vb & ~(size_t)15;
                if (vb > body)
                    gb_copy_bytes(L, reinterpret_cast<char*>(out + d0 + (size_t)j * a.stripe) + body,
                                  tm.ws[own] + b.off_c + (size_t)((i - depth) & 1) * a.len_c + body,
                                  vb - body, true);
            }
        }
        const bool ok = gb_ring_run_jobs(R, tm, bi, per, jobs, njobs,
            [&](const GbJob& job, const unsigned char* stage, unsigned pitch, size_t off, unsigned len) {
                if (job.kind == JOB_COPY) copy_tile(job.dst, stage, off, len);
                else if (job.kind == JOB_ISLAND)
                    island_reduce_tile<T, OP>(tm, b, job.arg, stage, pitch, off, len);
                else bridge_reduce_tile<T, OP>(tm, b, job.arg, stage, pitch, off, len);
            });
        if (!ok) return;
        if (i + 1 < iters &&
            !gb_sync(tm, ch, (unsigned)per, (unsigned)(i < 7 ? i : 7), i == 0 && ch == 0))
            return;
    }
}

// ---- the same kernel with one ring run per step ---------------------------------------------------
// With more than two islands the bridge can run "two-shot" (a.role_b != 0): owner j of island g
// sends sub-stripe h of its island result only to owner j of island h, which adds the islands'
// sub-stripes in leader order and sends the finished sub-stripe to owner j of every island.
// That moves 2 (I - 1) / I stripes per owner instead of I - 1, with the same number of steps
// and barriers and the same order of additions.
// Step B: fold the island's slots in member order, round to T, store.
template <typename T, int OP>
__device__ __forceinline__ bool island_reduce_ring(GbRing& R, const GbTeam& tm, const GbArgs& a,
                                                   int bi, int nb, const char* slots, size_t count,
                                                   int buf) {
    typedef typename GbAcc<T>::type A;
    constexpr int V = Vec<T>::N;
    const int m = tm.island_off[tm.my_island + 1] - tm.island_off[tm.my_island];
    const bool bridged = tm.n_islands > 1;
    const size_t sbytes = a.stripe * sizeof(T);
    return gb_ring_run(R, tm, bi, nb, slots, sbytes, m, count * sizeof(T), true,
        [&](const unsigned char* stage, unsigned pitch, size_t off, unsigned len) {
            const unsigned nv = len >> 4;
            for (unsigned v = threadIdx.x; v < nv; v += THREADS) {
                A part[V];
                for (int p = 0; p < m; ++p) {
                    Vec<T> w;
                    w.u = *reinterpret_cast<const uint4*>(stage + (size_t)p * pitch + ((size_t)v << 4));
                    #pragma unroll
                    for (int j = 0; j < V; ++j)
                        part[j] = (p == 0) ? gb_up<T>(w.e[j])
                                           : GbFold<OP, A>::run(part[j], gb_up<T>(w.e[j]));
                }
                Vec<T> r;
                #pragma unroll
                for (int j = 0; j < V; ++j) r.e[j] = gb_down<T>(part[j]);
                const size_t at = off + ((size_t)v << 4);
                if (!bridged) {
                    if (a.divide > 0) {
                        #pragma unroll
                        for (int j = 0; j < V; ++j)
                            r.e[j] = gb_down<T>(gb_divide<A>(gb_up<T>(r.e[j]), a.divide));
                    }
                    gb_st16(tm.ws[tm.rank] + a.off_c + (size_t)buf * a.len_c + at, r.u);
                } else if (a.role_b != 0) {
                    const size_t subbytes = sbytes / (size_t)tm.n_islands;
                    const size_t h = at / subbytes;
                    const int owner = tm.order[tm.island_off[h] + tm.my_pos];
                    gb_st16(tm.ws[owner] + a.off_b + (size_t)buf * a.len_b
                            + (size_t)tm.my_island * subbytes + (at - h * subbytes), r.u);
                } else {
                    for (int d = 0; d < tm.n_islands; ++d) {
                        const int isl = (tm.my_island + d) % tm.n_islands;
                        const int owner = tm.order[tm.island_off[isl] + tm.my_pos];
                        gb_st16(tm.ws[owner] + a.off_b + (size_t)buf * a.len_b
                                + (size_t)tm.my_island * sbytes + at, r.u);
                    }
                }
            }
        });
}

// Step C: add the island results in island order, AVG, one rounding, into region C.
template <typename T, int OP>
__device__ __forceinline__ bool bridge_reduce_ring(GbRing& R, const GbTeam& tm, const GbArgs& a,
                                                   int bi, int nb, size_t count, int buf) {
    typedef typename GbAcc<T>::type A;
    constexpr int V = Vec<T>::N;
    const size_t sbytes = a.stripe * sizeof(T);
    const char* parts = tm.ws[tm.rank] + a.off_b + (size_t)buf * a.len_b;
    char* result = tm.ws[tm.rank] + a.off_c + (size_t)buf * a.len_c;
    const int groups = tm.n_islands;
    if (a.role_b != 0) {
        // two-shot: this owner finishes sub-stripe `my_island` and sends it to every island
        const size_t sub = a.stripe / (size_t)groups, subbytes = sub * sizeof(T);
        const size_t lo = (size_t)tm.my_island * sub;
        const size_t mine = count > lo ? (count - lo < sub ? count - lo : sub) : 0;
        if (mine == 0) return true;
        return gb_ring_run(R, tm, bi, nb, parts, subbytes, groups, mine * sizeof(T), true,
            [&](const unsigned char* stage, unsigned pitch, size_t off, unsigned len) {
                const unsigned nv = len >> 4;
                for (unsigned v = threadIdx.x; v < nv; v += THREADS) {
                    A total[V];
                    for (int g = 0; g < groups; ++g) {
                        Vec<T> w;
                        w.u = *reinterpret_cast<const uint4*>(stage + (size_t)g * pitch + ((size_t)v << 4));
                        #pragma unroll
                        for (int j = 0; j < V; ++j)
                            total[j] = (g == 0) ? gb_up<T>(w.e[j])
                                                : GbFold<OP, A>::run(total[j], gb_up<T>(w.e[j]));
                    }
                    Vec<T> r;
                    #pragma unroll
                    for (int j = 0; j < V; ++j)
                        r.e[j] = gb_down<T>(a.divide > 0 ? gb_divide<A>(total[j], a.divide) : total[j]);
                    const size_t at = (size_t)tm.my_island * subbytes + off + ((size_t)v << 4);
                    for (int d = 0; d < groups; ++d) {
                        const int isl = (tm.my_island + d) % groups;
                        const int owner = tm.order[tm.island_off[isl] + tm.my_pos];
                        gb_st16(tm.ws[owner] + a.off_c + (size_t)buf * a.len_c + at, r.u);
                    }
                }
            });
    }
    return gb_ring_run(R, tm, bi, nb, parts, sbytes, groups, count * sizeof(T), true,
        [&](const unsigned char* stage, unsigned pitch, size_t off, unsigned len) {
            const unsigned nv = len >> 4;
            for (unsigned v = threadIdx.x; v < nv; v += THREADS) {
                A total[V];
                for (int g = 0; g < groups; ++g) {
                    Vec<T> w;
                    w.u = *reinterpret_cast<const uint4*>(stage + (size_t)g * pitch + ((size_t)v << 4));
                    #pragma unroll
                    for (int j = 0; j < V; ++j)
                        total[j] = (g == 0) ? gb_up<T>(w.e[j])
                                            : GbFold<OP, A>::run(total[j], gb_up<T>(w.e[j]));
                }
                Vec<T> r;
                #pragma unroll
                for (int j = 0; j < V; ++j)
                    r.e[j] = gb_down<T>(a.divide > 0 ? gb_divide<A>(total[j], a.divide) : total[j]);
                gb_st16(result + off + ((size_t)v << 4), r.u);
            }
        });
}

template <typename T, int OP>
__global__ void __launch_bounds__(THREADS)
allreduce_ring_phased_kernel(GbTeam tm, GbArgs a) {
    GbRing R = gb_ring_init();
    const T* in = static_cast<const T*>(a.in);
    T* out = static_cast<T*>(a.out);
    const bool owner = tm.my_pos < a.k;
    const bool bridged = tm.n_islands > 1;
    const size_t sbytes = a.stripe * sizeof(T);
    const long nchunks = (long)((a.n + a.chunk - 1) / a.chunk);
    const int depth = bridged ? 3 : 2;
    const int channels = a.role_a > 0 ? a.role_a : 1;
    const int per = (int)gridDim.x / channels;
    const int ch = (int)blockIdx.x / per;
    if (ch >= channels) return;
    const int bi = (int)blockIdx.x - ch * per;
    const GbLane L = gb_lane_blocks(ch * per, per, tm.ld_mode);
    const long mine = nchunks > ch ? (nchunks - ch + channels - 1) / channels : 0;
    if (mine == 0) return;
    const long iters = mine + depth;
    GbArgs b = a;                                        // this channel's regions
    b.off_a = a.off_a + (size_t)ch * 2 * a.len_a;
    b.off_b = a.off_b + (size_t)ch * 2 * a.len_b;
    b.off_c = a.off_c + (size_t)ch * 2 * a.len_c;
    for (long i = 0; i < iters; ++i) {
        if (i < mine) {                                  // A(i)
            const size_t c0 = (size_t)(ch + i * channels) * a.chunk;
            for (int dj = 0; dj < a.k; ++dj) {
                const int j = (tm.my_pos + dj) % a.k;
                const int own = tm.order[tm.island_off[tm.my_island] + j];
                char* dst = tm.ws[own] + b.off_a + (size_t)(i & 1) * a.len_a
                            + (size_t)tm.my_pos * sbytes;
                const size_t valid = stripe_valid(a, c0, j);
                if (valid && !gb_ring_copy(R, tm, L, bi, per, dst, in + c0 + (size_t)j * a.stripe,
                                           valid * sizeof(T), false))
                    return;
                zero_range(L, dst, valid * sizeof(T), round_up(valid, 256) * sizeof(T));
            }
        }
        if (owner && i >= 1 && i - 1 < mine) {           // B(i-1)
            const long c = ch + (i - 1) * channels;
            const size_t need = round_up(stripe_valid(a, (size_t)c * a.chunk, tm.my_pos), 256);
            const char* slots = tm.ws[tm.rank] + b.off_a + (size_t)((i - 1) & 1) * a.len_a;
            if (!island_reduce_ring<T, OP>(R, tm, b, bi, per, slots, need, (int)((i - 1) & 1)))
                return;
        }
        if (bridged && owner && i >= 2 && i - 2 < mine) {        // C(i-2)
            const long c = ch + (i - 2) * channels;
            const size_t need = round_up(stripe_valid(a, (size_t)c * a.chunk, tm.my_pos), 256);
            if (!bridge_reduce_ring<T, OP>(R, tm, b, bi, per, need, (int)((i - 2) & 1))) return;
        }
        if (i >= depth) {                                // D(i-depth)
            const long c = ch + (i - depth) * channels;
            const size_t c0 = (size_t)c * a.chunk;
            for (int dj = 0; dj < a.k; ++dj) {
                const int j = (tm.my_pos + dj) % a.k;
                const int own = tm.order[tm.island_off[tm.my_island] + j];
                const size_t valid = stripe_valid(a, c0, j);
                if (valid && !gb_ring_copy(R, tm, L, bi, per, out + c0 + (size_t)j * a.stripe,
                                           tm.ws[own] + b.off_c + (size_t)((i - depth) & 1) * a.len_c,
                                           valid * sizeof(T), true))
                    return;
            }
        }
        if (i + 1 < iters &&
            !gb_sync(tm, ch, (unsigned)per, (unsigned)(i < 7 ? i : 7), i == 0 && ch == 0))
            return;
    }
}

// ---- all-reduce through the switch (NVLS) --------------------------------------------------------
// One island, SUM / AVG of f32, bf16 or f16.  Every rank owns a buffer bound to one NVLink
// multicast object: a multimem.ld_reduce on the multicast address returns the sum of that
// address over all ranks, computed inside the NVSwitch, and a multimem.st writes all ranks'
// copies at once.  Per chunk: copy the input into the own buffer; barrier; reduce the own
// 1/world slice through the switch and write it back to everybody; barrier; copy the buffer
// to the output.  A GPU then receives and sends one chunk's worth of data per chunk instead of
// 2 (world - 1) / world: half the traffic of the two-shot exchange over peer memory.  Every
// element is reduced by exactly one rank, so all ranks end with identical bits; the order of
// the addends is the switch's.  Region: `sym` / `mc` + off_a, three buffers of len_a bytes used in
// turn by the chunks.
template <typename T> struct Multimem;
template <> struct Multimem<float> {
    static __device__ __forceinline__ uint4 load_sum(const char* mc) {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
        return v;
    }
};
template <> struct Multimem<__nv_bfloat16> {
    static __device__ __forceinline__ uint4 load_sum(const char* mc) {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
        return v;
    }
};
template <> struct Multimem<__half> {
    static __device__ __forceinline__ uint4 load_sum(const char* mc) {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
        return v;
    }
};
__device__ __forceinline__ void multimem_store(char* mc, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
                 :: "l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
allreduce_nvls_kernel(GbTeam tm, GbArgs a) {
    typedef typename GbAcc<T>::type A;
    constexpr int V = Vec<T>::N;
    const char* in = static_cast<const char*>(a.in);
    char* out = static_cast<char*>(a.out);
    const size_t total = a.n * sizeof(T);
    const size_t chunk = a.chunk * sizeof(T);              // a multiple of 16 * world
    const long nchunks = (long)((total + chunk - 1) / chunk);
    // Software pipeline over three buffers, one barrier per iteration: iteration i copies
    // chunk i into the own buffer, reduces chunk i - 1 through the switch and copies chunk
    // i - 2 out.  The first `a.k` blocks do the switch step (link-bound: few SMs saturate it),
    // the others the two local copies, so the steps of an iteration run side by side.
    const int reducers = a.k > 0 && a.k < (int)gridDim.x ? a.k : (int)gridDim.x;
    const bool split = reducers < (int)gridDim.x;
    const bool do_reduce = !split || (int)blockIdx.x < reducers;
    const bool do_copy = !split || (int)blockIdx.x >= reducers;
    const GbLane L = !split ? gb_lane_all(tm.ld_mode)
                   : do_reduce ? gb_lane_blocks(0, reducers, tm.ld_mode)
                               : gb_lane_blocks(reducers, (int)gridDim.x - reducers, tm.ld_mode);
    auto len_of = [&](long c) {
        const size_t c0 = (size_t)c * chunk;
        return total - c0 < chunk ? total - c0 : chunk;
    };
    for (long i = 0; i < nchunks + 2; ++i) {
        if (do_copy && i < nchunks) {                       // copy chunk i in
            const size_t len = len_of(i);
            char* mine = a.sym + a.off_a + (size_t)(i % 3) * a.len_a;
            gb_copy_bytes(L, mine, in + (size_t)i * chunk, len, false);
            zero_range(L, mine, len, round_up(len, 16 * (size_t)tm.world));
        }
        if (do_reduce && i >= 1 && i - 1 < nchunks) {       // reduce chunk i - 1 in the switch
            const long c = i - 1;
            const size_t padded = round_up(len_of(c), 16 * (size_t)tm.world);
            char* everyone = a.mc + a.off_a + (size_t)(c % 3) * a.len_a;
            const size_t slice = padded / (size_t)tm.world;    // a multiple of 16
            const size_t s0 = (size_t)tm.rank * slice;
            const size_t nvec = slice >> 4;
            for (size_t v = L.tid; v < nvec; v += L.nth) {
                Vec<T> r;
                r.u = Multimem<T>::load_sum(everyone + s0 + (v << 4));
                if (a.divide > 0) {
                    #pragma unroll
                    for (int j = 0; j < V; ++j)
                        r.e[j] = gb_down<T>(gb_divide<A>(gb_up<T>(r.e[j]), a.divide));
                }
                multimem_store(everyone + s0 + (v << 4), r.u);
            }
        }
        if (do_copy && i >= 2) {                            // copy chunk i - 2 out
            const long c = i - 2;
            gb_copy_bytes(L, out + (size_t)c * chunk,
                          a.sym + a.off_a + (size_t)(c % 3) * a.len_a, len_of(c), true);
        }
        if (i + 1 < nchunks + 2 && !gb_sync_all(tm, (unsigned)(i < 7 ? i : 7), i == 0)) return;
    }
}

// ---- all-gather ---------------------------------------------------------------------------------
// Region A: [2 parities][2 chunk buffers] of len_a bytes.  n and chunk are bytes.
__global__ void __launch_bounds__(THREADS)
allgather_kernel(GbTeam tm, GbArgs a) {
    GbRing R = gb_ring_init();
    const unsigned parity = gb_ld_volatile(&tm.ctrl->epoch) & 1u;
    const char* in = static_cast<const char*>(a.in);
    char* out = static_cast<char*>(a.out);
    const long nchunks = (long)((a.n + a.chunk - 1) / a.chunk);
    const GbLane L = gb_lane_all(tm.ld_mode);
    const int bi = (int)blockIdx.x, nb = (int)gridDim.x;
    for (long t = 0; t <= nchunks; ++t) {
        if (t < nchunks) {
            const size_t c0 = (size_t)t * a.chunk;
            const size_t len = a.n - c0 < a.chunk ? a.n - c0 : a.chunk;
            if (!gb_ring_copy(R, tm, L, bi, nb,
                              tm.ws[tm.rank] + a.off_a + (size_t)(parity * 2 + (t & 1)) * a.len_a,
                              in + c0, len, false))
                return;
        }
        if (t >= 1) {
            const long c = t - 1;
            const size_t c0 = (size_t)c * a.chunk;
            const size_t len = a.n - c0 < a.chunk ? a.n - c0 : a.chunk;
            for (int d = 0; d < tm.world; ++d) {
                const int peer = (tm.rank + d) % tm.world;
                if (!gb_ring_copy(R, tm, L, bi, nb, out + (size_t)peer * a.n + c0,
                                  tm.ws[peer] + a.off_a + (size_t)(parity * 2 + (c & 1)) * a.len_a,
                                  len, true))
                    return;
            }
        }
        if (t < nchunks && !gb_sync_all(tm, (unsigned)(t < 7 ? t : 7), t == 0)) return;
    }
}

// ---- reduce-scatter -------------------------------------------------------------------------------
// Region A: [2 parities][2 chunk buffers][world slots] ; len_a = world * chunk bytes.
// n: elements of one slice; chunk: elements per step.
// TO: the type of the output slice (T, or the other one of float / bf16: the cast that would
// otherwise be a separate pass over the result is the reduction's one rounding).
template <typename T, int OP, typename TO = T>
__global__ void __launch_bounds__(THREADS)
reduce_scatter_kernel(GbTeam tm, GbArgs a) {
    const unsigned parity = gb_ld_volatile(&tm.ctrl->epoch) & 1u;
    const T* in = static_cast<const T*>(a.in);
    TO* out = static_cast<TO*>(a.out);
    const size_t slot = a.chunk * sizeof(T);
    const long nchunks = (long)((a.n + a.chunk - 1) / a.chunk);
    // Roles: the blocks of role A store chunk t into its owners while the rest reduce chunk t-1.
    const bool split = a.role_a > 0;
    const bool do_a = !split || (int)blockIdx.x < a.role_a;
    const bool do_b = !split || (int)blockIdx.x >= a.role_a;
    const GbLane L = !split ? gb_lane_all(tm.ld_mode)
                   : do_a ? gb_lane_blocks(0, a.role_a, tm.ld_mode)
                          : gb_lane_blocks(a.role_a, (int)gridDim.x - a.role_a, tm.ld_mode);
    GbRing R = gb_ring_init();
    const int ring_bi = !split || do_a ? (int)blockIdx.x : (int)blockIdx.x - a.role_a;
    const int ring_nb = !split ? (int)gridDim.x : do_a ? a.role_a : (int)gridDim.x - a.role_a;
    for (long t = 0; t <= nchunks; ++t) {
        if (do_a && t < nchunks) {
            const size_t c0 = (size_t)t * a.chunk;
            const size_t len = a.n - c0 < a.chunk ? a.n - c0 : a.chunk;
            for (int d = 0; d < tm.world; ++d) {
                const int owner = (tm.rank + d) % tm.world;
                if (!gb_ring_copy(R, tm, L, ring_bi, ring_nb,
                                  tm.ws[owner] + a.off_a + (size_t)(parity * 2 + (t & 1)) * a.len_a
                                  + (size_t)tm.rank * slot,
                                  in + (size_t)owner * a.n + c0, len * sizeof(T), false))
                    return;
            }
        }
        if (do_b && t >= 1) {
            const long c = t - 1;
            const size_t c0 = (size_t)c * a.chunk;
            const size_t len = a.n - c0 < a.chunk ? a.n - c0 : a.chunk;
            reduce_slots<T, OP, TO>(L, tm.ws[tm.rank] + a.off_a + (size_t)(parity * 2 + (c & 1)) * a.len_a,
                                    slot, tm.order, tm.island_off, tm.n_islands, len, out + c0, a.divide);
        }
        if (t < nchunks && !gb_sync_all(tm, (unsigned)(t < 7 ? t : 7), t == 0)) return;
    }
}

// ---- broadcast --------------------------------------------------------------------------------------
// Region A: [2 parities][2 chunk buffers] of len_a = stripe bytes.  n, chunk, stripe are bytes
// (chunk = world * stripe).  `out` is the tensor on every rank (the data on the source).
__global__ void __launch_bounds__(THREADS)
broadcast_kernel(GbTeam tm, GbArgs a) {
    const unsigned parity = gb_ld_volatile(&tm.ctrl->epoch) & 1u;
    char* data = static_cast<char*>(a.out);
    const long nchunks = (long)((a.n + a.chunk - 1) / a.chunk);
    const GbLane L = gb_lane_all(tm.ld_mode);
    GbRing R = gb_ring_init();
    const int bi = (int)blockIdx.x, nb = (int)gridDim.x;
    for (long t = 0; t <= nchunks; ++t) {
        if (t < nchunks && tm.rank == a.root) {
            const size_t c0 = (size_t)t * a.chunk;
            for (int d = 0; d < tm.world; ++d) {
                const int j = (tm.rank + d) % tm.world;
                const size_t s0 = c0 + (size_t)j * a.stripe;
                if (s0 >= a.n) continue;
                const size_t len = a.n - s0 < a.stripe ? a.n - s0 : a.stripe;
                if (!gb_ring_copy(R, tm, L, bi, nb,
                                  tm.ws[j] + a.off_a + (size_t)(parity * 2 + (t & 1)) * a.len_a,
                                  data + s0, len, false))
                    return;
            }
        }
        if (t >= 1 && tm.rank != a.root) {
            const long c = t - 1;
            const size_t c0 = (size_t)c * a.chunk;
            for (int d = 0; d < tm.world; ++d) {
                const int j = (tm.rank + d) % tm.world;
                const size_t s0 = c0 + (size_t)j * a.stripe;
                if (s0 >= a.n) continue;
                const size_t len = a.n - s0 < a.stripe ? a.n - s0 : a.stripe;
                if (!gb_ring_copy(R, tm, L, bi, nb, data + s0,
                                  tm.ws[j] + a.off_a + (size_t)(parity * 2 + (c & 1)) * a.len_a,
                                  len, true))
                    return;
            }
        }
        if (t < nchunks && !gb_sync_all(tm, (unsigned)(t < 7 ? t : 7), t == 0)) return;
    }
}

__global__ void __launch_bounds__(THREADS)
barrier_kernel(GbTeam tm) {
    gb_sync_all(tm, 0, true);
}

// Link probe: what one kind of traffic achieves with a given grid, and what a barrier costs.
//   k = 0  store n bytes from the own workspace (region B) into the next rank's (region A)
//   k = 1  load n bytes from the next rank's workspace (region B) into the own (region A)
//   k = 2  local copy of n bytes (region B to region A)
//   k = 3  n barriers and nothing else
//   k = 4  the first half of the blocks store while the second half load (mixed traffic)
//   k = 5  like 4 plus a third group that copies locally
//   k = 6, 7, 8  like 0, 1, 2 but through the bulk-copy ring
// Each pass is repeated `divide` times inside the launch; one barrier at the start and the end.
__global__ void __launch_bounds__(THREADS)
probe_kernel(GbTeam tm, GbArgs a) {
    const GbLane L = gb_lane_all(tm.ld_mode);
    const int next = (tm.rank + 1) % tm.world;
    if (!gb_sync_all(tm, 0, true)) return;
    if (a.k == 3) {
        for (size_t i = 0; i < a.n; ++i)
            if (!gb_sync_all(tm, 1, false)) return;
        return;
    }
    if (a.k == 4 || a.k == 5) {
        const int groups = a.k == 4 ? 2 : 3;
        const int per = (int)gridDim.x / groups;
        const int g = (int)blockIdx.x / per;
        if (g < groups) {
            const GbLane G = gb_lane_blocks(g * per, per, tm.ld_mode);
            for (int rep = 0; rep < a.divide; ++rep) {
                if (g == 0)
                    gb_copy_bytes(G, tm.ws[next] + a.off_a, tm.ws[tm.rank] + a.off_b, a.n, false);
                else if (g == 1)
                    gb_copy_bytes(G, tm.ws[tm.rank] + a.off_c, tm.ws[next] + a.off_b, a.n, true);
                else
                    gb_copy_bytes(G, tm.ws[tm.rank] + a.off_a + a.len_a, tm.ws[tm.rank] + a.off_b,
                                  a.n, false);
            }
        }
        gb_sync_all(tm, 2, false);
        return;
    }
    if (a.k >= 6) {
        GbRing R = gb_ring_init();
        for (int rep = 0; rep < a.divide; ++rep) {
            bool ok;
            if (a.k == 6)
                ok = gb_ring_copy(R, tm, L, (int)blockIdx.x, (int)gridDim.x, tm.ws[next] + a.off_a,
                                  tm.ws[tm.rank] + a.off_b, a.n, false);
            else if (a.k == 7)
                ok = gb_ring_copy(R, tm, L, (int)blockIdx.x, (int)gridDim.x, tm.ws[tm.rank] + a.off_a,
                                  tm.ws[next] + a.off_b, a.n, true);
            else
                ok = gb_ring_copy(R, tm, L, (int)blockIdx.x, (int)gridDim.x, tm.ws[tm.rank] + a.off_a,
                                  tm.ws[tm.rank] + a.off_b, a.n, false);
            if (!ok) return;
        }
        gb_sync_all(tm, 2, false);
        return;
    }
    for (int rep = 0; rep < a.divide; ++rep) {
        if (a.k == 0)
            gb_copy_bytes(L, tm.ws[next] + a.off_a, tm.ws[tm.rank] + a.off_b, a.n, false);
        else if (a.k == 1)
            gb_copy_bytes(L, tm.ws[tm.rank] + a.off_a, tm.ws[next] + a.off_b, a.n, true);
        else
            gb_copy_bytes(L, tm.ws[tm.rank] + a.off_a, tm.ws[tm.rank] + a.off_b, a.n, false);
    }
    gb_sync_all(tm, 2, false);
}

// ---- dispatch -----------------------------------------------------------------------------------------
template <typename T, int OP>
cudaError_t launch_plain(int kind, const GbTeam& tm, const GbArgs& a, int grid, cudaStream_t s) {
    if (kind == 0) allreduce_oneshot_kernel<T, OP><<<grid, THREADS, 0, s>>>(tm, a);
    else if (kind == 1) allreduce_hier_kernel<T, OP, GB_RAW><<<grid, THREADS, 0, s>>>(tm, a);
    else if (kind == 2) {
        static cudaError_t opted = cudaFuncSetAttribute(
            reduce_scatter_kernel<T, OP>, cudaFuncAttributeMaxDynamicSharedMemorySize, GB_RING_SMEM);
        if (opted != cudaSuccess) return opted;
        reduce_scatter_kernel<T, OP><<<grid, THREADS, GB_RING_SMEM, s>>>(tm, a);
    }
    else if (kind == 3) {
        // the ring needs more dynamic shared memory than the default limit: opt in once
        static cudaError_t opted = cudaFuncSetAttribute(
            allreduce_ring_kernel<T, OP>, cudaFuncAttributeMaxDynamicSharedMemorySize, GB_RING_SMEM);
        if (opted != cudaSuccess) return opted;
        allreduce_ring_kernel<T, OP><<<grid, THREADS, GB_RING_SMEM, s>>>(tm, a);
    }
    else if (kind == 4) {
        static cudaError_t opted = cudaFuncSetAttribute(
            allreduce_ring_phased_kernel<T, OP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
            GB_RING_SMEM);
        if (opted != cudaSuccess) return opted;
        allreduce_ring_phased_kernel<T, OP><<<grid, THREADS, GB_RING_SMEM, s>>>(tm, a);
    }
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

template <typename T, typename TO>
cudaError_t launch_scatter_cast(const GbTeam& tm, const GbArgs& a, int grid, cudaStream_t s) {
    static cudaError_t opted = cudaFuncSetAttribute(
        reduce_scatter_kernel<T, GB_SUM, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, GB_RING_SMEM);
    if (opted != cudaSuccess) return opted;
    reduce_scatter_kernel<T, GB_SUM, TO><<<grid, THREADS, GB_RING_SMEM, s>>>(tm, a);
    return cudaGetLastError();
}

template <typename T>
cudaError_t launch_nvls(const GbTeam& tm, const GbArgs& a, int grid, cudaStream_t s) {
    allreduce_nvls_kernel<T><<<grid, THREADS, 0, s>>>(tm, a);
    return cudaGetLastError();
}

template <typename T>
cudaError_t launch_op(int kind, int op, const GbTeam& tm, const GbArgs& a, int grid, cudaStream_t s) {
    if (op == GB_SUM) return launch_plain<T, GB_SUM>(kind, tm, a, grid, s);
    if (kind == 2) return cudaErrorInvalidValue;            // reduce-scatter: SUM only
    if (op == GB_MAX) return launch_plain<T, GB_MAX>(kind, tm, a, grid, s);
    if (op == GB_MIN) return launch_plain<T, GB_MIN>(kind, tm, a, grid, s);
    return cudaErrorInvalidValue;
}

template <typename T>
cudaError_t launch_coded(int codec, const GbTeam& tm, const GbArgs& a, int grid, cudaStream_t s) {
    if (codec == GB_C_FP8_REF)
        allreduce_hier_kernel<T, GB_SUM, GB_C_FP8_REF><<<grid, THREADS, 0, s>>>(tm, a);
    else if (codec == GB_C_FP8_B200)
        allreduce_hier_kernel<T, GB_SUM, GB_C_FP8_B200><<<grid, THREADS, 0, s>>>(tm, a);
    else if (codec == GB_C_BF16 && sizeof(T) >= 4)
        allreduce_hier_kernel<T, GB_SUM, GB_C_BF16><<<grid, THREADS, 0, s>>>(tm, a);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace

// kind: 0 one-shot all-reduce, 1 hierarchical all-reduce, 2 reduce-scatter,
//       3 / 4 hierarchical all-reduce through the bulk-copy ring (queue / phased; no codec),
//       5 all-reduce through the switch (NVLS multimem),
//       6 reduce-scatter whose output has the other float type (dtype f32: bf16 out; bf16: f32 out).
// codec (kind 1, SUM, floating point only): GbCodec.  Returns a cudaError_t.
extern "C" int gb_launch_reduce(int kind, int dtype, int op, int codec, const GbTeam* team,
                                const GbArgs* args, int grid, cudaStream_t stream) {
    const GbTeam& tm = *team;
    const GbArgs& a = *args;
    if (codec != GB_RAW) {
        if (kind != 1 || op != GB_SUM) return cudaErrorInvalidValue;
        switch (dtype) {
            case GB_F32: return launch_coded<float>(codec, tm, a, grid, stream);
            case GB_F64: return launch_coded<double>(codec, tm, a, grid, stream);
            case GB_BF16: return launch_coded<__nv_bfloat16>(codec, tm, a, grid, stream);
            case GB_F16: return launch_coded<__half>(codec, tm, a, grid, stream);
        }
        return cudaErrorInvalidValue;
    }
    if (kind == 6) {                        // reduce-scatter that casts: float in -> bf16 out or back
        if (op != GB_SUM) return cudaErrorInvalidValue;
        if (dtype == GB_F32) return launch_scatter_cast<float, __nv_bfloat16>(tm, a, grid, stream);
        if (dtype == GB_BF16) return launch_scatter_cast<__nv_bfloat16, float>(tm, a, grid, stream);
        return cudaErrorInvalidValue;
    }
    if (kind == 5) {                        // through the switch: SUM of f32, bf16, f16 only
        if (op != GB_SUM || a.mc == nullptr || a.sym == nullptr) return cudaErrorInvalidValue;
        switch (dtype) {
            case GB_F32: return launch_nvls<float>(tm, a, grid, stream);
            case GB_BF16: return launch_nvls<__nv_bfloat16>(tm, a, grid, stream);
            case GB_F16: return launch_nvls<__half>(tm, a, grid, stream);
        }
        return cudaErrorInvalidValue;
    }
    switch (dtype) {
        case GB_F32: return launch_op<float>(kind, op, tm, a, grid, stream);
        case GB_BF16: return launch_op<__nv_bfloat16>(kind, op, tm, a, grid, stream);
        case GB_F16: return launch_op<__half>(kind, op, tm, a, grid, stream);
        case GB_F64: return launch_op<double>(kind, op, tm, a, grid, stream);
        case GB_I8: return launch_op<signed char>(kind, op, tm, a, grid, stream);
        case GB_U8: return launch_op<unsigned char>(kind, op, tm, a, grid, stream);
        case GB_I32: return launch_op<int>(kind, op, tm, a, grid, stream);
        case GB_I64: return launch_op<long long>(kind, op, tm, a, grid, stream);
    }
    return cudaErrorInvalidValue;
}

// kind: 0 all-gather, 1 broadcast, 2 barrier, 3 link probe.
extern "C" int gb_launch_copy(int kind, const GbTeam* team, const GbArgs* args, int grid,
                              cudaStream_t stream) {
    if (kind == 0) {
        static cudaError_t opted = cudaFuncSetAttribute(
            allgather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GB_RING_SMEM);
        if (opted != cudaSuccess) return opted;
        allgather_kernel<<<grid, THREADS, GB_RING_SMEM, stream>>>(*team, *args);
    }
    else if (kind == 1) {
        static cudaError_t opted = cudaFuncSetAttribute(
            broadcast_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GB_RING_SMEM);
        if (opted != cudaSuccess) return opted;
        broadcast_kernel<<<grid, THREADS, GB_RING_SMEM, stream>>>(*team, *args);
    }
    else if (kind == 2) barrier_kernel<<<1, THREADS, 0, stream>>>(*team);
    else if (kind == 3) {
        static cudaError_t opted = cudaFuncSetAttribute(
            probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GB_RING_SMEM);
        if (opted != cudaSuccess) return opted;
        probe_kernel<<<grid, THREADS, args->k >= 6 ? GB_RING_SMEM : 0, stream>>>(*team, *args);
    }
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

extern "C" size_t gb_sizeof_team() { return sizeof(GbTeam); }
extern "C" size_t gb_sizeof_args() { return sizeof(GbArgs); }
extern "C" size_t gb_sizeof_ctrl() { return sizeof(GbCtrl); }
extern "C" size_t gb_payload_bytes(int codec, int elem_size, size_t stripe) {
    if (codec == GB_RAW) return stripe * (size_t)elem_size;
    if (codec == GB_C_BF16) return stripe * 2;
    const size_t bs = codec == GB_C_FP8_B200 ? 128 : 256;
    return (stripe + 4 * (stripe / bs) + 15) / 16 * 16;
}

GB_BOUNDS_HOST(collectives)
