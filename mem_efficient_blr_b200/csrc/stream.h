// Parameter block of the weight-streaming kernel used for small token counts (N <= 16).
//
// The kernel evaluates up to two "phases".  A phase is a grouped product
//     out[g][n][m] = sum_k W[g][m][k] * A[g][n][k]        g < G, m < M, n < N, k < K
// where W is a stack of weight blocks (16-bit, int8 or packed int4) and A the 16-bit activations.
// Between two phases the kernel crosses one grid-wide barrier (two when the BLAST coupling
// z_i = sum_j S_ij (.) y_j has to be applied in between).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace blr {

static constexpr int kStreamMaxTokens = 16;
static constexpr int kTileRows = 32;       // weight rows per tile (one TMA box)
static constexpr int kBatchTiles = 4;      // tiles consumed together (128 rows)
static constexpr int kTileBytes = 4096;    // 32 rows x 128 B   or   64 k-rows x 64 B
static constexpr int kConsumerWarps = 8;
static constexpr int kStreamThreads = (kConsumerWarps + 2) * 32;
static constexpr int kRedStride = 17;      // fp32 words per reduction-buffer row (16 tokens + pad)

struct alignas(64) PhaseDesc {
  CUtensorMap tmW;  // weights: K-major dims (K, M, G) box (128 B, 32, 1); M-major dims (M, K, G) box (32, 64, 1)
  CUtensorMap tmA;  // activations: dims (K, N, G) box (64, 8|16, 1)
  int G, M, K;
  int kmajor;       // 1: W[g][m][k] (k contiguous)   0: W[g][k][m] (m contiguous; 16-bit only)
  int wbits;        // 16, 8, 4
  int tiles_per_g;  // ceil(M / 32)
  int ntiles;       // G * tiles_per_g
  int nchunks;      // K-chunks per tile: 128 B of k per row (K-major) or 64 k-rows (M-major)
  int a_boxes;      // 64-wide activation boxes per chunk: 1 (16-bit), 2 (int8), 4 (int4)
  int out_f32;      // 1: out is fp32, 0: out has the activation dtype
  int round_out;    // 1: round to nearest integer and clamp to [-128,127] before storing
  int per;          // output offset = g*os_g + n*os_n + (m / per)*os_hi + (m % per)*os_lo
  long long os_g, os_n, os_hi, os_lo;
  void* out;
  const __half* scale;  // per-row dequantisation scale [G*M] or nullptr
};

struct alignas(64) StreamParams {
  PhaseDesc ph[2];
  int nphases;
  int N;
  int mix;        // 1: BLAST coupling between phase 0 and phase 1
  int b, R;       // coupling dimensions
  int round_z;    // 1: round/clamp z like round_out
  long long s_i, s_j, s_r;  // element strides of S for (out block, in block, rank)
  const void* S;
  float* y32;     // [b][N][R] fp32 scratch (phase 0 output when mix)
  void* z16;      // [b][N][R] 16-bit scratch (phase 1 activations when mix)
  unsigned* counters;  // [0],[1] grid barriers, [2] exit count, [3] status (0 ok)
  int stage_bytes;
  int nstages;
};

// Launches the kernel (cooperative launch, one CTA per SM).  is_bf16 selects the 16-bit type.
int launch_stream(const StreamParams& p, int is_bf16, cudaStream_t stream);

}  // namespace blr
