// Tile shape of the single-CTA tcgen05 GEMM kernels (gb_gemm.cu, gb_gemm_rs.cu): one block
// computes a 128 x 256 output tile in steps of 64 along the contraction, from a 4-stage operand
// ring in shared memory into one of two 256-column accumulators in tensor memory.
#pragma once
#include "gb_tc.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;                 // 16 KiB
constexpr int B_BYTES = BN * BK * 2;                 // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;                    // TMA warp, MMA warp, four epilogue warps
constexpr int TMEM_COLS = 512;                       // two accumulators of 256 columns

}  // namespace
