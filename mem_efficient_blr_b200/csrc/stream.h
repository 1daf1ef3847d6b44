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
static constexpr int kBatchRows = 128;      // weight rows consumed together: 16 per consumer warp
static constexpr int kSubBytes = kBatchRows * 128;  // weight bytes of one K-chunk of a full batch
static constexpr int kTileBytes = 4096;     // m-contiguous layout: one box = 64 k-rows x 32 m (64 B)
static constexpr int kConsumerWarps = 8;
static constexpr int kStreamThreads = (kConsumerWarps + 2) * 32;
static constexpr int kStreamTailBytes = 2 * 16 * 8 + 64 + 1024;  // barriers, abort flag, alignment slack

static constexpr int kScaleGroup = 128;  // the one supported width of a scale group

struct alignas(64) PhaseDesc {
  // weights, K-major: dims (K, M, G), tmW[h-1] has box (128 B, 16*h, 1) so that one load brings a whole
  // batch of h row groups; M-major: dims (M, K, G), only tmW[0] with box (32, 64, 1)
  CUtensorMap tmW[8];
  CUtensorMap tmA;  // activations: dims (K, N, G) box (64, 8|16, 1)
  int G, M, K;
  int kmajor;       // 1: W[g][m][k] (k contiguous)   0: W[g][k][m] (m contiguous; 16-bit only)
  int wbits;        // 16, 8, 4
  int unit_rows;    // rows per work unit: 16 (K-major) or 32 (M-major)
  int tiles_per_g;  // work units per block: ceil(M / unit_rows)
  int ntiles;       // G * tiles_per_g
  int nchunks;      // K-chunks per unit: 128 B of k per row (K-major) or 64 k-rows (M-major)
  int ks;           // K-chunks per ring stage (1, 2, 4 or 8)
  int sub_bytes;    // distance between the K-chunks of a stage: the weight bytes of one chunk of the largest batch
                    // a CTA gets in this phase (kSubBytes for a full batch of 128 rows)
  int nstage_chunks;  // ceil(nchunks / ks): ring stages per batch
  int a_boxes;      // 64-wide activation boxes per chunk: 1 (16-bit), 2 (int8), 4 (int4)
  int out_f32;      // 1: out is fp32, 0: out has the activation dtype
  int round_out;    // 1: round to nearest integer and clamp to [-128,127] before storing
  int per;          // output offset = g*os_g + n*os_n + (m / per)*os_hi + (m % per)*os_lo
  long long os_g, os_n, os_hi, os_lo;
  void* out;
  const __half* scale;  // dequantisation scales: [G*M] (one per row), [G*M][K/group] when group != 0, or nullptr
  int group;            // 0, or kScaleGroup: contraction indices per scale
};

struct alignas(64) StreamParams {
  PhaseDesc ph[2];
  int nphases;
  int N;
  int mix;        // 1: BLAST coupling between phase 0 and phase 1
  int b, R;       // coupling dimensions: in-blocks, rank
  int b_out;      // out-blocks present in S / z (== b unless the call holds a slice of the output blocks)
  int round_z;    // 1: round/clamp z like round_out
  long long s_i, s_j, s_r;  // element strides of S for (out block, in block, rank)
  const void* S;
  float* y32;     // [b][N][R] fp32 scratch (phase 0 output when mix)
  void* z16;      // [b][N][R] 16-bit scratch (phase 1 activations when mix)
  unsigned* counters;  // [0],[1] grid barriers, [2] exit count, [3] status (0 ok)
  int stage_bytes;
  int w_bytes;    // weight part of a stage: max over phases of ks * sub_bytes
  int nstages;
  int mix_bytes;  // shared memory for the coupling's copy of y (0 when mix == 0)
#ifdef BLR_TIMELINE
  unsigned long long* timeline;  // profiling builds: 16 time stamps per CTA
#endif
};

// Launches the kernel (cooperative launch, one CTA per SM).  is_bf16 selects the 16-bit type.
int launch_stream(const StreamParams& p, int is_bf16, cudaStream_t stream);
#ifdef BLR_TIMELINE
// Profiling builds: when set, every launch records %globaltimer stamps, 16 slots per CTA, at dev_ptr.
void set_stream_timeline(unsigned long long* dev_ptr);
#endif

}  // namespace blr
