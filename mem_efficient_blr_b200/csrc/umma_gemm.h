// Grouped tensor-core GEMM for token counts above the streaming kernel's limit:
//     out[g][n][m] = sum_k W[g][m][k] * A[g][n][k]
// fp32 accumulation in TMEM, 16-bit output.  Two orientations of the tcgen05 tile:
//   tokens_as_rows = 1: 128 tokens are the MMA's 128 rows, up to 256 weight rows its columns; an epilogue
//                       thread then owns one token and writes runs of consecutive outputs (16-byte stores);
//   tokens_as_rows = 0: 128 weight rows are the MMA rows and up to 256 tokens its columns ("swap-AB"),
//                       which wastes nothing when there are fewer than 128 tokens.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace blr {

struct alignas(64) GemmParams {
  CUtensorMap tmW;  // K-major: dims (K, M, G) box (64, row-tile, 1); M-major: dims (M, K, G) box (64, 64, 1)
                    // quantised weights (w_bits 8 | 4, K-major): bytes, dims (K*w_bits/8, M, G) box (8*w_bits, row-tile, 1), no swizzle
  CUtensorMap tmA;  // dims (K, N, G) box (64, token-tile, 1)
  int G, M, K, N;
  int kmajor;          // weight layout
  int tokens_as_rows;  // orientation (see above)
  int bn;              // extent of the MMA's column operand: tokens (swap-AB) or weight rows; multiple of 16, <= 256
  int nstages;
  int is_bf16;
  int round_out;    // round to nearest integer, clamp to [-128, 127] before storing
  int per;          // output offset = g*os_g + n*os_n + (m / per)*os_hi + (m % per)*os_lo
  long long os_g, os_n, os_hi, os_lo;
  void* out;
  unsigned* status;  // optional: set to 1 when a device-side wait gave up
  // Optional additions in the epilogue, for outputs laid out [n][g * M + m] (per >= M, os_lo = 1): bias[g * M + m] and
  // residual[n * ldr + g * M + m], both of the 16-bit dtype.  extra_vec: both may be read in 16-byte pieces.
  const void* bias;
  const void* residual;
  long long ldr;
  int extra_vec;
  int act_out;  // applied after the bias, before the residual: 0 none, 1 GELU (erf), 2 GELU (tanh approximation)
  // Quantised weights: int8 or packed int4 (two per byte along k, even index in the low nibble, two's complement) with
  // fp16 scales [g][m][scales_per_row] (1: per weight row; K / 128: per 128 contraction indices).  Converter warps
  // widen every staged tile to the 16-bit dtype (q * scale, rounded once) in shared memory ahead of the MMA.
  int w_bits;  // 0 / 16: 16-bit weights
  int scales_per_row;
  const void* w_scale;
};

int launch_umma_gemm(const GemmParams& p, cudaStream_t stream);

// Picks orientation, tile extents and ring depth from N, M; fills tokens_as_rows / bn / nstages.
void umma_gemm_tiling(GemmParams& p);

// Rows of the weight tile and of the token tile implied by the tiling (for the TMA boxes).
inline int umma_w_tile_rows(const GemmParams& p) { return p.tokens_as_rows ? p.bn : 128; }
inline int umma_a_tile_rows(const GemmParams& p) { return p.tokens_as_rows ? 128 : p.bn; }

}  // namespace blr
