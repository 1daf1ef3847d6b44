// BLAST for 1..16 tokens as two dependent launches with no exchange between CTAs:
//
//   front  one CTA per slice of 8 consecutive ranks r.  The slice is self-contained: y_j[r] = V_j[r,:] x_j for
//          every in-block j needs the 8 rows r of every V_j (b pieces of 8 contiguous rows) and the whole of x;
//          z_i[r] = sum_j S[i][j][r] y_j[r] for every out-block i follows inside the CTA.  z goes to global memory
//          as (out-block, token, rank), 16-bit.
//   back   one CTA per run of consecutive 16-row groups of one U_i.  It holds its rows over the whole contraction
//          in shared memory, reads z_i, and writes its outputs directly: no split of the contraction over CTAs, so
//          no reduction in global memory and a fixed summation order.
//
// Both kernels fetch their weights - all of them where they fit, else a ring's worth - BEFORE they wait for the
// kernel ahead of them in the stream (programmatic dependent launch): the weights of a layer stream from HBM while
// the previous kernel computes, and what is left on the dependent path after the wait is a read of the activations
// from L2, the products on shared-memory operands, and the stores.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "stream.h"

namespace blr {

static constexpr int kSplitRanks = 8;                       // ranks per front CTA
static constexpr int kSplitWarps = 16;                      // consumer warps per CTA (a power of two)
static constexpr int kSplitFrontThreads = kSplitWarps * 32;
static constexpr int kSplitBackThreads = (kSplitWarps + 1) * 32;
static constexpr int kSplitStageChunks = 8;                 // 128-byte K-chunks of a 16-row group per ring stage
static constexpr int kSplitChunkBytes = 16 * 128;
static constexpr int kSplitStageBytes = kSplitStageChunks * kSplitChunkBytes;
static constexpr int kSplitMaxBlocks = 32;

static constexpr int kSplitMaxProblems = 3;  // layers that share x and their shapes, run by one pair of launches

// Input transform applied while x is staged: none, or x := silu(x) * x_mul (the SwiGLU product in front of a
// down projection; models the reference's `down_proj(act_fn(gate_proj(h)) * up_proj(h))`).
static constexpr int kSplitActNone = 0, kSplitActSiluMul = 1;

struct SplitProblem {
  CUtensorMap tmV;  // dims (P | row bytes, R, b), box (128 B, 8, b), 128-byte swizzle
  CUtensorMap tmU;  // dims (R | row bytes, Q, b_out), box (128 B, 16, 1), 128-byte swizzle
  const void* S;           // coupling factors or nullptr (all ones)
  const __half* v_scale;   // (b, R) or (b, R, P / group) or nullptr
  const __half* u_scale;   // (b_out, Q) or (b_out, Q, R / group) or nullptr
  void* z;                 // (b_out, N, R) 16-bit, written by the front kernel, read by the back kernel
  void* out;               // (N, b_out * Q), row stride ldo
  const void* bias;        // (b_out * Q) 16-bit added to every row, or nullptr
  const void* residual;    // (N, b_out * Q) 16-bit added to the result (row stride ldr), or nullptr
  long long ldo, ldr;
};

struct alignas(64) SplitParams {
  SplitProblem pr[kSplitMaxProblems];  // blockIdx.y picks the problem; all share x, the shapes and the strides of S
  const void* x;
  const void* x_mul;       // second input of the input transform (same shape and row stride as x), or nullptr
  unsigned* status;        // set to 1 when a wait ran out
  void* xq;                // scratch for x converted to fixed point once per call (more than 2 tokens, quantised
  float* xq_scale;         // factors): b * N rows of the front kernel's row pitch, and their scales; nullptr otherwise
  long long ldx, s_i, s_j, s_r;
  int nprob, act;
  int N, b, bo, P, Q, R;
  int wbits, group;
  int round_y, round_z;
  int monarch, mon_per, mon_torch;  // Monarch: no coupling, z_l[k * per + jj] = y_k[m]; rows m in the torch order (jj * b + l) or grouped (l * per + jj)
  int out_interleaved;     // output feature of row s of out-block l: s * b + l instead of l * Q + s
  int z_shared;            // no coupling factors (S == nullptr, low rank as BLAST): z is the same for every out-block, kept once
  int nch0, nch1;          // 128-byte chunks per row of V / of U
  int cpb, gpc;            // back kernel: CTAs per out-block, 16-row groups per CTA
  int nstages;             // back kernel: ring stages
  unsigned magic_N, magic_rows;  // ceil(2^32 / d) for d = N, 8 gpc (0 for d = 1): division-free quotients
#ifdef BLR_TIMELINE
  unsigned long long* timeline;  // profiling builds: 16 stamps per CTA of this launch
#endif
};

// Bytes of one fixed-point activation row over K contraction indices (the front kernel's row pitch).
size_t split_fx_row_bytes(int K, int wbits);
size_t split_front_smem(const SplitParams& p);
size_t split_back_smem(const SplitParams& p);
// Enqueues both kernels.  is_bf16 selects the 16-bit type.
int launch_blast_split(const SplitParams& p, int is_bf16, cudaStream_t stream);

}  // namespace blr
