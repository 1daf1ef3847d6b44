// Tensor-core pipeline for more than 16 tokens: grouped tcgen05 GEMMs (umma_gemm.cu) chained through
// 16-bit intermediates, plus the BLAST coupling kernel between the two GEMMs.
#include "pipeline.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tmap.h"
#include "umma_gemm.h"

namespace blr {

static CUtensorMapDataType dt16(int dtype) {
  return dtype == BLR_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

struct OutSpec {
  void* out;
  long long os_g, os_n, os_hi, os_lo;
  int per;
  int round_out;
};

// One grouped GEMM: W (G blocks of M rows over K), A[g][n][k] with element strides (1, ld_n, ld_g).
static int run_gemm(int dtype, const void* W, int layout, int G, int M, int K, const void* A, int64_t N, int64_t ld_n,
                    int64_t ld_g, const OutSpec& o, cudaStream_t stream) {
  GemmParams p = {};
  p.G = G; p.M = M; p.K = K; p.N = (int)N;
  p.kmajor = layout == BLR_W_KMAJOR;
  p.is_bf16 = dtype == BLR_DTYPE_BF16;
  p.round_out = o.round_out;
  p.per = o.per; p.os_g = o.os_g; p.os_n = o.os_n; p.os_hi = o.os_hi; p.os_lo = o.os_lo; p.out = o.out;
  p.status = nullptr;
  BLR_REQUIRE(N < (1ll << 31), BLR_ERR_SHAPE, "too many tokens");
  umma_gemm_tiling(p);
  int rc;
  if (p.kmajor) {
    BLR_REQUIRE(K % 8 == 0, BLR_ERR_SHAPE, "contraction length %d must be a multiple of 8", K);
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)M, (uint64_t)G};
    const uint64_t str[2] = {(uint64_t)K * 2, (uint64_t)M * K * 2};
    const uint32_t box[3] = {64, 128, 1};
    rc = encode_tmap_3d(&p.tmW, dt16(dtype), W, dims, str, box, Swz::B128);
  } else {
    BLR_REQUIRE(M % 8 == 0, BLR_ERR_SHAPE, "block output width %d must be a multiple of 8", M);
    const uint64_t dims[3] = {(uint64_t)M, (uint64_t)K, (uint64_t)G};
    const uint64_t str[2] = {(uint64_t)M * 2, (uint64_t)M * K * 2};
    const uint32_t box[3] = {64, 64, 1};
    rc = encode_tmap_3d(&p.tmW, dt16(dtype), W, dims, str, box, Swz::B128);
  }
  if (rc) return rc;
  BLR_REQUIRE(ld_n % 8 == 0 && ld_g % 8 == 0, BLR_ERR_ALIGN, "activation strides (%lld, %lld elements) must be multiples of 8",
              (long long)ld_n, (long long)ld_g);
  const uint64_t adims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)G};
  const uint64_t astr[2] = {(uint64_t)ld_n * 2, (uint64_t)(G > 1 ? ld_g : ld_n * N) * 2};
  const uint32_t abox[3] = {64, (uint32_t)p.bn, 1};
  if ((rc = encode_tmap_3d(&p.tmA, dt16(dtype), A, adims, astr, abox, Swz::B128))) return rc;
  return launch_umma_gemm(p, stream);
}

// ------------------------------------------------------------------------------------------ BLAST coupling
// z[i][n][r] = sum_j S[i][j][r] * y[j][n][r], y and z 16-bit [b][N][R].
// A block owns 64 consecutive r and a range of tokens; its slice of S sits in shared memory as fp32-ready
// 16-bit [i][j][64].  Thread = (8-wide r vector, group of 4 out-blocks, token lane).
template <typename T>
__device__ __forceinline__ float2 up2(uint32_t w);
template <>
__device__ __forceinline__ float2 up2<__half>(uint32_t w) { return __half22float2(*reinterpret_cast<const __half2*>(&w)); }
template <>
__device__ __forceinline__ float2 up2<__nv_bfloat16>(uint32_t w) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w)); }
template <typename T>
__device__ __forceinline__ uint32_t pk2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pk2<__half>(float a, float b) { const __half2 v = __floats2half2_rn(a, b); return *reinterpret_cast<const uint32_t*>(&v); }
template <>
__device__ __forceinline__ uint32_t pk2<__nv_bfloat16>(float a, float b) { const __nv_bfloat162 v = __floats2bfloat162_rn(a, b); return *reinterpret_cast<const uint32_t*>(&v); }
template <typename T>
__device__ __forceinline__ float ld1(const T* p);
template <>
__device__ __forceinline__ float ld1<__half>(const __half* p) { return __half2float(*p); }
template <>
__device__ __forceinline__ float ld1<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__global__ void __launch_bounds__(256) blast_couple_kernel(const T* __restrict__ y, const T* __restrict__ S, long long s_i,
                                                          long long s_j, long long s_r, T* __restrict__ z, int b, int N, int R,
                                                          int tokens_per_block, int round_z) {
  extern __shared__ __align__(16) uint8_t sm[];
  T* sS = reinterpret_cast<T*>(sm);  // [b][b][64]
  const int r0 = blockIdx.x * 64, n_begin = blockIdx.y * tokens_per_block;
  const int n_end = min(N, n_begin + tokens_per_block);
  const int rw = min(64, R - r0);
  for (int e = threadIdx.x; e < b * b * 64; e += blockDim.x) {
    const int rr = e & 63, ij = e >> 6, i = ij / b, j = ij - i * b;
    sS[e] = rr < rw ? S[i * s_i + j * s_j + (long long)(r0 + rr) * s_r] : T(0.f);
  }
  __syncthreads();
  const int IG = (b + 3) / 4;
  const int vec = threadIdx.x & 7, ig = (threadIdx.x >> 3) % IG, nl = threadIdx.x / (8 * IG);
  const int n_par = blockDim.x / (8 * IG);
  if (nl >= n_par || vec * 8 >= rw) return;
  const long long plane = (long long)N * R;
  for (int n = n_begin + nl; n < n_end; n += n_par) {
    float acc[4][8];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[a][k] = 0.f;
    const T* yp = y + (long long)n * R + r0 + vec * 8;
    for (int j = 0; j < b; ++j) {
      const uint4 yv = *reinterpret_cast<const uint4*>(yp + j * plane);
      const float2 y0 = up2<T>(yv.x), y1 = up2<T>(yv.y), y2 = up2<T>(yv.z), y3 = up2<T>(yv.w);
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const int i = ig * 4 + a;
        if (i < b) {
          const uint4 sv = *reinterpret_cast<const uint4*>(sS + ((i * b + j) << 6) + vec * 8);
          const float2 s0 = up2<T>(sv.x), s1 = up2<T>(sv.y), s2 = up2<T>(sv.z), s3 = up2<T>(sv.w);
          acc[a][0] = fmaf(s0.x, y0.x, acc[a][0]); acc[a][1] = fmaf(s0.y, y0.y, acc[a][1]);
          acc[a][2] = fmaf(s1.x, y1.x, acc[a][2]); acc[a][3] = fmaf(s1.y, y1.y, acc[a][3]);
          acc[a][4] = fmaf(s2.x, y2.x, acc[a][4]); acc[a][5] = fmaf(s2.y, y2.y, acc[a][5]);
          acc[a][6] = fmaf(s3.x, y3.x, acc[a][6]); acc[a][7] = fmaf(s3.y, y3.y, acc[a][7]);
        }
      }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int i = ig * 4 + a;
      if (i < b) {
        if (round_z) {
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[a][k] = fminf(fmaxf(rintf(acc[a][k]), -128.f), 127.f);
        }
        uint4 o;
        o.x = pk2<T>(acc[a][0], acc[a][1]); o.y = pk2<T>(acc[a][2], acc[a][3]);
        o.z = pk2<T>(acc[a][4], acc[a][5]); o.w = pk2<T>(acc[a][6], acc[a][7]);
        *reinterpret_cast<uint4*>(z + i * plane + (long long)n * R + r0 + vec * 8) = o;
      }
    }
  }
}

// Any block count / any strides: one thread per output element.
template <typename T>
__global__ void blast_couple_generic_kernel(const T* __restrict__ y, const T* __restrict__ S, long long s_i, long long s_j,
                                            long long s_r, T* __restrict__ z, int b, long long NR, int R, int round_z) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= NR) return;
  const int r = (int)(e % R);
  for (int i = 0; i < b; ++i) {
    float s = 0.f;
    for (int j = 0; j < b; ++j) s = fmaf(ld1<T>(S + i * s_i + j * s_j + (long long)r * s_r), ld1<T>(y + j * NR + e), s);
    if (round_z) s = fminf(fmaxf(rintf(s), -128.f), 127.f);
    z[i * NR + e] = T(s);
  }
}

template <typename T>
static int run_couple(const void* y, const void* S, int64_t s_i, int64_t s_j, int64_t s_r, void* z, int b, int64_t N, int R,
                      int round_z, cudaStream_t stream) {
  if (b <= 16 && R % 8 == 0) {
    const size_t smem = (size_t)b * b * 64 * sizeof(T);
    // at most 16 * 16 * 64 * 2 = 32 KB: within the default dynamic shared-memory limit
    const int rblocks = (R + 63) / 64;
    int tokens_per_block = 128;
    // enough blocks to fill the machine without shrinking the per-block reuse of S too far
    while (tokens_per_block > 32 && (long long)rblocks * ((N + tokens_per_block - 1) / tokens_per_block) < 296) tokens_per_block /= 2;
    dim3 grid(rblocks, (unsigned)((N + tokens_per_block - 1) / tokens_per_block));
    BLR_REQUIRE(grid.y <= 65535, BLR_ERR_SHAPE, "too many tokens for the coupling kernel");
    blast_couple_kernel<T><<<grid, 256, smem, stream>>>(static_cast<const T*>(y), static_cast<const T*>(S), s_i, s_j, s_r,
                                                         static_cast<T*>(z), b, (int)N, R, tokens_per_block, round_z);
  } else {
    const long long NR = (long long)N * R;
    blast_couple_generic_kernel<T><<<(unsigned)((NR + 255) / 256), 256, 0, stream>>>(
        static_cast<const T*>(y), static_cast<const T*>(S), s_i, s_j, s_r, static_cast<T*>(z), b, NR, R, round_z);
  }
  BLR_CUDA_OK(cudaGetLastError());
  return BLR_OK;
}

// ------------------------------------------------------------------------------------------ operators
int pipeline_blast(const void* x, int64_t ldx, int64_t N, int dtype, const void* U, int u_layout, const void* V,
                   int v_layout, const void* S, int64_t s_i, int64_t s_j, int64_t s_r, int b, int P, int Q, int R,
                   int act_int8, void* out, int64_t ldo, void* y16, void* z16, cudaStream_t stream) {
  const long long plane = (long long)N * R;
  // y[j][n][r] = sum_p V[j][r][p] x[n][j*P + p]
  int rc = run_gemm(dtype, V, v_layout, b, R, P, x, N, ldx, P, OutSpec{y16, plane, R, 0, 1, R, act_int8}, stream);
  if (rc) return rc;
  rc = dtype == BLR_DTYPE_BF16 ? run_couple<__nv_bfloat16>(y16, S, s_i, s_j, s_r, z16, b, N, R, act_int8, stream)
                               : run_couple<__half>(y16, S, s_i, s_j, s_r, z16, b, N, R, act_int8, stream);
  if (rc) return rc;
  // out[n][i*Q + q] = sum_r U[i][q][r] z[i][n][r]
  return run_gemm(dtype, U, u_layout, b, Q, R, z16, N, R, plane, OutSpec{out, Q, ldo, 0, 1, Q, 0}, stream);
}

int pipeline_monarch(const void* x, int64_t ldx, int64_t N, int dtype, const void* w1, int w1_layout, int grouped,
                     const void* w2, int w2_layout, int b, int P, int rank, int Qs, int interleaved, void* out,
                     int64_t ldo, void* z16, cudaStream_t stream) {
  const int per = rank / b;
  const long long plane = (long long)N * rank;
  const OutSpec o1 = grouped ? OutSpec{z16, per, rank, plane, 1, per, 0} : OutSpec{z16, per, rank, 1, plane, b, 0};
  int rc = run_gemm(dtype, w1, w1_layout, b, rank, P, x, N, ldx, P, o1, stream);
  if (rc) return rc;
  const OutSpec o2 = interleaved ? OutSpec{out, 1, ldo, 0, b, Qs, 0} : OutSpec{out, Qs, ldo, 0, 1, Qs, 0};
  return run_gemm(dtype, w2, w2_layout, b, Qs, rank, z16, N, rank, plane, o2, stream);
}

int pipeline_low_rank(const void* x, int64_t ldx, int64_t N, int dtype, const void* V, int v_layout, const void* U,
                      int u_layout, int I, int R, int O, void* out, int64_t ldo, void* z16, cudaStream_t stream) {
  int rc = run_gemm(dtype, V, v_layout, 1, R, I, x, N, ldx, 0, OutSpec{z16, 0, R, 0, 1, R, 0}, stream);
  if (rc) return rc;
  return run_gemm(dtype, U, u_layout, 1, O, R, z16, N, R, 0, OutSpec{out, 0, ldo, 0, 1, O, 0}, stream);
}

int pipeline_dense(const void* x, int64_t ldx, int64_t N, int dtype, const void* W, int w_layout, int I, int O, void* out,
                   int64_t ldo, cudaStream_t stream) {
  return run_gemm(dtype, W, w_layout, 1, O, I, x, N, ldx, 0, OutSpec{out, 0, ldo, 0, 1, O, 0}, stream);
}

}  // namespace blr
