// Row-parallel GEMM (+bias) fused with reduce-scatter, for sm_100a.
//
// Capability: gemm-rs/reference.py:36-60 -- every rank holds input[M, K/ws] and
// weight[N, K/ws], the result is sum_r input_r * weight_r^T (+ bias) scattered along M so
// that rank r keeps rows [r*M/ws, (r+1)*M/ws).  The reference runs three serial stages
// (library GEMM, elementwise bias, library reduce-scatter).  Here ONE persistent kernel
//   * computes 128 x BN tiles (single CTAs) or 256 x BN tiles (CTA pairs, cta_group::2) with
//     tcgen05.mma (bf16 in, fp32 accumulators in tensor memory), operands staged by plain
//     TMA loads into 128B-swizzled shared memory through an mbarrier pipeline, two
//     accumulator buffers so the epilogue of a tile overlaps the main loop of the next;
//   * in the epilogue rounds each partial row to bf16 (the reference's rounding point) and
//     stores it into the *owning* rank's staging slot over NVLink (TMA stores), then bumps
//     that owner's arrival counters -- tiles are visited so that the rows a rank owns
//     itself come last;
//   * reduces the world_size partials of its own rows in fixed rank order in fp32, adds the
//     bias with its multiplicity, rounds once and writes out[M/ws, N] -- on dedicated reducer
//     warps that take each output unit as soon as its last partial has arrived, while the
//     tensor cores are still busy with other tiles.
// Small problems are cut along K into slices that travel as fp32 "virtual ranks".
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "status.h"

namespace b200 {

constexpr int kGemmRsBlockM = 128;
constexpr int kGemmRsBlockN = 256;  // widest tile; narrower instantiations exist for small problems
constexpr int kGemmRsBlockK = 64;

struct GemmRsArgs {
  const void* a;     // [M, K] bf16, row-major (this rank's K slice)
  const void* w;     // [N, K] bf16, row-major
  const void* bias;  // [N] bf16 or nullptr
  void* out;         // [M / world_size, N] bf16
  int M, N, K, world_size, rank;
  float bias_scale;  // multiplier of the bias when it is added once by the owning rank
  int bias_at_source;  // 1: every rank adds the bias to its own bf16 partial before the reduction, as the
                       // reference does (gemm-rs/reference.py:54-59), so the result holds world_size * bias
  uint64_t peer_base[kMaxWorldSize];
  uint64_t off_stage;     // staging buffer of the current parity: bf16 [world][M/ws][N]
  uint64_t off_counters;  // arrival counters of the current parity: uint32 [m_tiles][n_tiles]
  uint64_t epoch;
  uint64_t timeout_ns;
  StatusBlock* status;
  uint32_t* sync_counters;
  int max_ctas;  // 0 = one per SM
  int block_n;   // 0 = choose from the shape; else 64, 128 or 256
  int cta_pair;  // -1 = choose from the shape; 0 = single CTAs; 1 = CTA pairs (256-row tiles)
  int splits;    // 0 = choose from the shape; else the number of K slices per tile
  uint64_t* trace;  // optional device buffer [CTAs][8] of globaltimer stamps (start, pipeline ready, GEMM
                    // tiles done, exit, first own tile reached, its peers' rows arrived, last own tile
                    // stored); nullptr = no tracing
  int debug;        // measurement aids, results are wrong when set: 1 = stage locally, 2 = do not stage
  int fuse_own;     // 1 = a rank adds the peers' rows to its own tiles in their epilogue; 0 = own tiles are
                    // staged like the others and reduced by all CTAs after the GEMM tiles
  int tma_store;    // 0 = per-lane staging stores only; otherwise TMA stores where the shape allows
  int force_staged; // 1 = stage and reduce even on a single rank (exercises the staged path on one GPU)
  uint64_t nvls_local;  // NVLS mode (both non-zero): this parity's staging in this rank's own multicast-bound memory,
  uint64_t nvls_mc;     // bf16 [M][N], and the same offset seen through the multicast address
  int checked;      // 1 = range-check every staging store against `stage_capacity` (record and skip on violation)
  uint64_t stage_capacity;  // bytes of one parity's staging region
};

// How a problem will be run, and what ONE parity of its workspace needs.  A pure function of
// its arguments (and the SM count), so every rank derives the same plan.
struct GemmRsPlan {
  int block_n, cta_pair, splits;
  uint64_t stage_bytes;    // bf16 [world][M / world][N]; fp32 [world * splits][M / world][N] when K is cut
  uint64_t counter_bytes;  // uint32 [m_tiles][n_tiles][4]
};
GemmRsPlan gemm_rs_plan(int M, int N, int K, int world_size, int block_n, int cta_pair, int splits);

cudaError_t launch_gemm_rs(const GemmRsArgs& args, cudaStream_t stream);

}  // namespace b200
