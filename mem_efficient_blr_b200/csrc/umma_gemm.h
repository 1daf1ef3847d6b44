// Grouped tensor-core GEMM for token counts above the streaming kernel's limit:
//     out[g][n][m] = sum_k W[g][m][k] * A[g][n][k]
// with the weights as the 128-row tcgen05 operand ("swap-AB": the tokens are the N dimension of the MMA,
// so a tile is 128 weight rows x up to 256 tokens), fp32 accumulation in TMEM, 16-bit output.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace blr {

struct alignas(64) GemmParams {
  CUtensorMap tmW;  // K-major: dims (K, M, G) box (64, 128, 1); M-major: dims (M, K, G) box (64, 64, 1)
  CUtensorMap tmA;  // dims (K, N, G) box (64, BN, 1)
  int G, M, K, N;
  int kmajor;       // weight layout
  int bn;           // tokens per tile (multiple of 16, <= 256)
  int nstages;
  int is_bf16;
  int round_out;    // round to nearest integer, clamp to [-128, 127] before storing
  int per;          // output offset = g*os_g + n*os_n + (m / per)*os_hi + (m % per)*os_lo
  long long os_g, os_n, os_hi, os_lo;
  void* out;
  unsigned* status;  // optional: set to 1 when a device-side wait gave up
};

int launch_umma_gemm(const GemmParams& p, cudaStream_t stream);

// Picks the token tile and ring depth for N tokens and fills bn / nstages.
void umma_gemm_tiling(GemmParams& p);

}  // namespace blr
