// BLAST for 1..16 tokens without grid barriers: the rank index r is cut into slices, one thread-block cluster
// per slice, one CTA of the cluster per block index.  CTA j computes y_j on the slice, the cluster exchanges y
// through distributed shared memory, CTA i couples z_i on the slice and multiplies it with the matching columns
// of U_i; the partial outputs of the slices are summed with fp32 reductions in global memory and the last CTA to
// finish a block converts it.  Nothing waits on another cluster.  The rows of U_i can be cut into parts (one
// cluster per slice and part; the parts of a slice repeat its first stage and coupling).  Monarch runs on the same
// kernel with the permutation between its stages as the exchange.
#pragma once
#include <cuda_runtime.h>

#include "stream.h"

namespace blr {

static constexpr int kClusterThreads = (kConsumerWarps + 1) * 32;
static constexpr int kClusterOut32Bytes = 2 << 20;   // fixed fp32 accumulation area at the start of a workspace
static constexpr int kXchPull = 0, kXchSubslice = 1, kXchMonarch = 2;  // exchange forms (template parameter)
static constexpr int kClusterMaxTokens = 16;          // tokens per call this kernel is used for
static constexpr int kClusterMaxSlice = 256;         // ranks per slice
static constexpr int kClusterHalfSmem = 115712;      // dynamic shared memory per CTA that lets two CTAs share an SM
static constexpr int kClusterMaxParts = 7;           // row parts of U_i (counters: parts * 16 words)

struct alignas(64) ClusterParams {
  PhaseDesc ph[2];     // ph[0]: V (G = b, M = R, K = P) with tmA = x; ph[1]: U (G = b, M = Q, K = R), tmA unused
  int N, b, R, Q;
  int rs;              // ranks per slice (multiple of the K extent of one chunk)
  int nslices;
  int qsplit, q_part;  // the rows of U_i are cut into qsplit parts of q_part rows (a multiple of 16), one cluster each;
                       // the clusters of one slice repeat its first phase and coupling
  int ks0, ks1;        // K-chunks per ring stage in the two phases
  int nchunks1;        // chunks of the second phase inside one slice
  int round_y, round_z;
  int subslice;        // 1: coupling by rank sub-slice (needs rs % (8 b) == 0): CTA c gathers ranks [c w, (c+1) w), w = rs / b,
                       // of every y_j, couples them for every out-block i and scatters z_i's piece to CTA i; the
                       // distributed-shared-memory traffic is 2 N rs values per CTA instead of b N rs
  // Monarch (monarch = 1): no coupling factors; the first phase of slice sl covers the mblk first-stage blocks
  // sl*mblk .. whose outputs feed the slice, cpb = b / mblk CTAs per block with rs rows each, and the exchange is
  // the permutation: z_l[t] = pre[k][q], k = sl*mblk + t / per, q = (t % per)*b + l (w1_grouped: l*per + t % per)
  int monarch, mblk, cpb, per, w1_grouped;
  long long out_blk, out_q;  // output feature of (block, row) = block * out_blk + row * out_q
  long long s_i, s_j, s_r;
  const void* S;       // coupling factors, or nullptr for all ones
  void* out;
  long long ldo;
  float* out32;        // [b*Q][8 or 16] fp32, zero between calls
  unsigned* counters;  // [qsplit][b] slices finished per (part, block), zero between calls
  unsigned* status;    // set to 1 when a wait ran out
  int stage_bytes, w_bytes, nstages;
#ifdef BLR_TIMELINE
  unsigned long long* timeline;  // profiling builds: 16 stamps per CTA
#endif
};

// Largest number of clusters of `b` CTAs that can be resident (0: this cluster shape cannot be launched).
// variant: 0 (BLAST, per-channel scales or none), kScaleGroup (BLAST with per-group scales), kClusterVariantMonarch
static constexpr int kClusterVariantMonarch = -1;
int cluster_capacity(int b, int is_bf16, int variant, int n_tokens, int smem_bytes);
size_t cluster_smem_bytes(const ClusterParams& p, int np);
int launch_blast_cluster(const ClusterParams& p, int is_bf16, cudaStream_t stream);

}  // namespace blr
