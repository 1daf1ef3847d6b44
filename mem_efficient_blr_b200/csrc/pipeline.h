// Tensor-core pipeline for token counts above the streaming kernel's limit (declared here, defined in
// pipeline.cu): grouped tcgen05 GEMMs with the weights as the 128-row operand, plus the BLAST coupling.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace blr {

// Quantised factors of a BLAST layer (bits 8 | 4 | 16 per factor; fp16 scales; group 0 | 128).
struct BlastQuant {
  int u_bits, v_bits, group;
  const void* u_scale;
  const void* v_scale;
};

int pipeline_blast(const void* x, int64_t ldx, int64_t N, int dtype, const void* U, int u_layout, const void* V,
                   int v_layout, const void* S, int64_t s_i, int64_t s_j, int64_t s_r, int b, int b_out, int P, int Q, int R,
                   int act_int8, void* out, int64_t ldo, void* y16, void* z16, void* e16, cudaStream_t stream,
                   const void* e_ready = nullptr, const BlastQuant* quant = nullptr, const void* bias = nullptr,
                   const void* residual = nullptr, int64_t ldr = 0, int out_act = 0);
// Expanded coupling factors of the prefill pipeline: size (0: shapes whose coupling does not use them) and construction.
size_t pipeline_coupling_bytes(int b, int b_out, int R);
int pipeline_expand_coupling(const void* S, int64_t s_i, int64_t s_j, int64_t s_r, int b, int b_out, int R, int dtype, void* E,
                             cudaStream_t stream);
int pipeline_monarch(const void* x, int64_t ldx, int64_t N, int dtype, const void* w1, int w1_layout, int grouped,
                     const void* w2, int w2_layout, int b, int P, int rank, int Qs, int interleaved, void* out,
                     int64_t ldo, void* z16, void* scratch, cudaStream_t stream);
int pipeline_low_rank(const void* x, int64_t ldx, int64_t N, int dtype, const void* V, int v_layout, const void* U,
                      int u_layout, int I, int R, int O, void* out, int64_t ldo, void* z16, void* parts, size_t parts_bytes,
                      cudaStream_t stream);
int pipeline_dense(const void* x, int64_t ldx, int64_t N, int dtype, const void* W, int w_layout, int I, int O,
                   void* out, int64_t ldo, cudaStream_t stream);

}  // namespace blr
