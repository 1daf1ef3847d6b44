// fp32 verification path (the `_fp32` entry points) and the symmetric weight quantiser.
// These kernels favour exact, easily audited arithmetic over speed: a shared-memory tiled fp32
// grouped GEMM with explicit strides, the BLAST coupling, and a one-block-per-row quantiser.
#include "../../include/blr_b200.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tmap.h"

namespace blr {

struct OutMap {
  long long os_g, os_n, os_hi, os_lo;
  int per;
};

// out[g][n][m] = sum_k A[g][n][k] * W[g][m][k]; A strides (a_g, a_n, 1); W strides (w_g, w_m, w_k).
__global__ void gemm_f32_kernel(const float* __restrict__ A, long long a_g, long long a_n, const float* __restrict__ W,
                                long long w_g, long long w_m, long long w_k, float* __restrict__ out, OutMap om, int N,
                                int M, int K) {
  __shared__ float sa[32][33];
  __shared__ float sw[32][33];
  const int g = blockIdx.z, n0 = blockIdx.y * 32, m0 = blockIdx.x * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 8
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < K; k0 += 32) {
    for (int r = ty; r < 32; r += 8) {
      const int n = n0 + r, m = m0 + r, k = k0 + tx;
      sa[r][tx] = (n < N && k < K) ? A[g * a_g + n * a_n + k] : 0.f;
      sw[r][tx] = (m < M && k < K) ? W[g * w_g + m * w_m + k * w_k] : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < 32; ++k) {
      const float wv = sw[tx][k];
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[r] = fmaf(sa[ty + 8 * r][k], wv, acc[r]);
    }
    __syncthreads();
  }
  const int m = m0 + tx;
  if (m < M) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int n = n0 + ty + 8 * r;
      if (n < N) out[g * om.os_g + n * om.os_n + (m / om.per) * om.os_hi + (m % om.per) * om.os_lo] = acc[r];
    }
  }
}

static int gemm_f32(const float* A, long long a_g, long long a_n, const float* W, int layout, int G, int M, int K,
                    float* out, OutMap om, int64_t N, cudaStream_t stream) {
  const long long w_g = (long long)M * K;
  const long long w_m = layout == BLR_W_KMAJOR ? K : 1;
  const long long w_k = layout == BLR_W_KMAJOR ? 1 : M;
  dim3 grid((M + 31) / 32, (unsigned)((N + 31) / 32), G), block(32, 8);
  BLR_REQUIRE(grid.y <= 65535 && grid.z <= 65535, BLR_ERR_SHAPE, "problem too large for the fp32 verification kernel");
  gemm_f32_kernel<<<grid, block, 0, stream>>>(A, a_g, a_n, W, w_g, w_m, w_k, out, om, (int)N, M, K);
  BLR_CUDA_OK(cudaGetLastError());
  return BLR_OK;
}

// z[i][n][r] = sum_j S[i][j][r] * y[j][n][r]
__global__ void mix_f32_kernel(const float* __restrict__ S, long long s_i, long long s_j, long long s_r,
                               const float* __restrict__ y, float* __restrict__ z, int b, long long NR, int R) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= NR) return;
  const int r = (int)(e % R);
  for (int i = 0; i < b; ++i) {
    float s = 0.f;
    for (int j = 0; j < b; ++j) s = fmaf(S[i * s_i + j * s_j + r * s_r], y[j * NR + e], s);
    z[i * NR + e] = s;
  }
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// One block per row: scale = max|w| / qmax (rounded to fp16), q = clamp(rint(w / scale)).
template <typename T>
__global__ void quantize_kernel(const T* __restrict__ w, long long K, int bits, int8_t* __restrict__ q8,
                                uint8_t* __restrict__ q4, __half* __restrict__ scale) {
  __shared__ float red[32];
  __shared__ float s_scale;
  const long long row = blockIdx.x;
  const T* wr = w + row * K;
  float amax = 0.f;
  for (long long k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(to_f32(wr[k])));
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) m = fmaxf(m, red[i]);
    const float qmax = bits == 8 ? 127.f : 7.f;
    const __half hs = __float2half_rn(__fdiv_rn(m, qmax));
    scale[row] = hs;
    s_scale = __half2float(hs);
  }
  __syncthreads();
  const float sc = s_scale, qmax = bits == 8 ? 127.f : 7.f;
  if (bits == 8) {
    for (long long k = threadIdx.x; k < K; k += blockDim.x) {
      const float v = sc > 0.f ? fminf(fmaxf(rintf(__fdiv_rn(to_f32(wr[k]), sc)), -qmax), qmax) : 0.f;
      q8[row * K + k] = (int8_t)v;
    }
  } else {
    for (long long k2 = threadIdx.x; k2 < K / 2; k2 += blockDim.x) {
      const float a = sc > 0.f ? fminf(fmaxf(rintf(__fdiv_rn(to_f32(wr[2 * k2]), sc)), -qmax), qmax) : 0.f;
      const float c = sc > 0.f ? fminf(fmaxf(rintf(__fdiv_rn(to_f32(wr[2 * k2 + 1]), sc)), -qmax), qmax) : 0.f;
      q4[row * (K / 2) + k2] = (uint8_t)(((int)a & 0xF) | (((int)c & 0xF) << 4));
    }
  }
}

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Inverse of the quantiser: 16 consecutive weights per thread, w = q * scale rounded to the 16-bit type.
// `group` consecutive weights share a scale (the row length for per-channel scales); it is a multiple of 16.
template <typename T>
__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t* __restrict__ q, const __half* __restrict__ scale,
                                                         long long total, long long group, int bits, T* __restrict__ out) {
  const long long e0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 16;
  if (e0 >= total) return;
  const float sc = __half2float(scale[e0 / group]);
  float v[16];
  if (bits == 8) {
    const uint4 w = *reinterpret_cast<const uint4*>(q + e0);
    const int8_t* b = reinterpret_cast<const int8_t*>(&w);
#pragma unroll
    for (int k = 0; k < 16; ++k) v[k] = (float)b[k] * sc;
  } else {
    const uint2 w = *reinterpret_cast<const uint2*>(q + e0 / 2);
    const uint8_t* b = reinterpret_cast<const uint8_t*>(&w);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int lo = b[k] & 0xF, hi = b[k] >> 4;
      v[2 * k] = (float)(lo > 7 ? lo - 16 : lo) * sc;
      v[2 * k + 1] = (float)(hi > 7 ? hi - 16 : hi) * sc;
    }
  }
  __align__(16) T o[16];
#pragma unroll
  for (int k = 0; k < 16; ++k) o[k] = from_f32<T>(v[k]);
  reinterpret_cast<uint4*>(out + e0)[0] = reinterpret_cast<const uint4*>(o)[0];
  reinterpret_cast<uint4*>(out + e0)[1] = reinterpret_cast<const uint4*>(o)[1];
}

}  // namespace blr

using namespace blr;

extern "C" {

int blr_blast_f32(const float* x, int64_t ldx, int64_t N, const float* U, int u_layout, const float* V, int v_layout,
                  const float* S, int64_t s_i, int64_t s_j, int64_t s_r, int b, int P, int Q, int R, float* out,
                  int64_t ldo, float* z, float* y, void* stream) {
  BLR_REQUIRE(x && U && V && S && out && z && y, BLR_ERR_ARG, "null pointer");
  BLR_REQUIRE(N >= 1 && b >= 2 && P > 0 && Q > 0 && R > 0, BLR_ERR_SHAPE, "bad dimensions (the reference asserts b != 1)");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long NR = (long long)N * R;
  int rc = gemm_f32(x, P, ldx, V, v_layout, b, R, P, y, OutMap{NR, R, 0, 1, R}, N, st);
  if (rc) return rc;
  mix_f32_kernel<<<(unsigned)((NR + 255) / 256), 256, 0, st>>>(S, s_i, s_j, s_r, y, z, b, NR, R);
  BLR_CUDA_OK(cudaGetLastError());
  return gemm_f32(z, NR, R, U, u_layout, b, Q, R, out, OutMap{Q, ldo, 0, 1, Q}, N, st);
}

int blr_monarch_f32(const float* x, int64_t ldx, int64_t N, const float* w1, int w1_layout, int w1_cols,
                    const float* w2, int w2_layout, int b, int P, int rank, int Qs, int out_order, float* out,
                    int64_t ldo, float* out1, void* stream) {
  BLR_REQUIRE(x && w1 && w2 && out && out1, BLR_ERR_ARG, "null pointer");
  BLR_REQUIRE(N >= 1 && b >= 1 && P > 0 && rank > 0 && Qs > 0 && rank % b == 0, BLR_ERR_SHAPE, "bad dimensions");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int per = rank / b;
  const long long plane = (long long)N * rank;
  const OutMap m1 = w1_cols == BLR_MONARCH_COLS_GROUPED ? OutMap{per, rank, plane, 1, per} : OutMap{per, rank, 1, plane, b};
  int rc = gemm_f32(x, P, ldx, w1, w1_layout, b, rank, P, out1, m1, N, st);
  if (rc) return rc;
  const OutMap m2 = out_order == BLR_OUT_INTERLEAVED ? OutMap{1, ldo, 0, b, Qs} : OutMap{Qs, ldo, 0, 1, Qs};
  return gemm_f32(out1, plane, rank, w2, w2_layout, b, Qs, rank, out, m2, N, st);
}

int blr_low_rank_f32(const float* x, int64_t ldx, int64_t N, const float* V, int v_layout, const float* U,
                     int u_layout, int I, int R, int O, float* out, int64_t ldo, float* z, void* stream) {
  BLR_REQUIRE(x && V && U && out && z, BLR_ERR_ARG, "null pointer");
  BLR_REQUIRE(N >= 1 && I > 0 && R > 0 && O > 0, BLR_ERR_SHAPE, "bad dimensions");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = gemm_f32(x, 0, ldx, V, v_layout, 1, R, I, z, OutMap{0, R, 0, 1, R}, N, st);
  if (rc) return rc;
  return gemm_f32(z, 0, R, U, u_layout, 1, O, R, out, OutMap{0, ldo, 0, 1, O}, N, st);
}

int blr_dense_f32(const float* x, int64_t ldx, int64_t N, const float* W, int w_layout, int I, int O, float* out,
                  int64_t ldo, void* stream) {
  BLR_REQUIRE(x && W && out, BLR_ERR_ARG, "null pointer");
  BLR_REQUIRE(N >= 1 && I > 0 && O > 0, BLR_ERR_SHAPE, "bad dimensions");
  return gemm_f32(x, 0, ldx, W, w_layout, 1, O, I, out, OutMap{0, ldo, 0, 1, O}, N, static_cast<cudaStream_t>(stream));
}

int blr_quantize_sym(const void* w, int dtype, int64_t rows, int64_t K, int bits, void* q, void* scale, void* stream) {
  BLR_REQUIRE(w && q && scale, BLR_ERR_ARG, "null pointer");
  BLR_REQUIRE(bits == 8 || bits == 4, BLR_ERR_ARG, "bits must be 8 or 4");
  BLR_REQUIRE(rows >= 1 && K >= 1 && (bits == 8 || K % 2 == 0), BLR_ERR_SHAPE, "bad dimensions");
  BLR_REQUIRE(rows < (1ll << 31), BLR_ERR_SHAPE, "too many rows");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == BLR_DTYPE_BF16)
    quantize_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(w), K, bits,
                                                                  static_cast<int8_t*>(q), static_cast<uint8_t*>(q),
                                                                  static_cast<__half*>(scale));
  else if (dtype == BLR_DTYPE_F16)
    quantize_kernel<__half><<<(unsigned)rows, 256, 0, st>>>(static_cast<const __half*>(w), K, bits,
                                                           static_cast<int8_t*>(q), static_cast<uint8_t*>(q),
                                                           static_cast<__half*>(scale));
  else
    BLR_REQUIRE(false, BLR_ERR_ARG, "unknown dtype %d", dtype);
  BLR_CUDA_OK(cudaGetLastError());
  return BLR_OK;
}

int blr_dequantize_sym(const void* q, const void* scale, int64_t rows, int64_t K, int bits, int64_t group, int dtype,
                       void* w, void* stream) {
  BLR_REQUIRE(q && scale && w, BLR_ERR_ARG, "null pointer");
  BLR_REQUIRE(bits == 8 || bits == 4, BLR_ERR_ARG, "bits must be 8 or 4");
  const int64_t g = group == 0 ? K : group;
  BLR_REQUIRE(rows >= 1 && K >= 16 && K % 16 == 0 && g % 16 == 0 && K % g == 0, BLR_ERR_SHAPE,
              "row length %lld and scale group %lld must be multiples of 16, the group a divisor of the row", (long long)K,
              (long long)g);
  BLR_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0, BLR_ERR_ALIGN,
              "q and w must be 16-byte aligned");
  const long long total = rows * K;
  const long long blocks = (total / 16 + 255) / 256;
  BLR_REQUIRE(blocks < (1ll << 31), BLR_ERR_SHAPE, "too many weights");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == BLR_DTYPE_BF16)
    dequantize_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const uint8_t*>(q), static_cast<const __half*>(scale),
                                                                      total, g, bits, static_cast<__nv_bfloat16*>(w));
  else if (dtype == BLR_DTYPE_F16)
    dequantize_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const uint8_t*>(q), static_cast<const __half*>(scale), total,
                                                               g, bits, static_cast<__half*>(w));
  else
    BLR_REQUIRE(false, BLR_ERR_ARG, "unknown dtype %d", dtype);
  BLR_CUDA_OK(cudaGetLastError());
  return BLR_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------- load / store probe
// Streams up to three operand arrays once (16-byte loads, nothing kept) and writes the output, the way the reference's
// load-store probes do: they measure what a kernel with this memory traffic and no arithmetic would take.
namespace blr {
template <typename T>
__global__ void __launch_bounds__(256) load_store_probe_kernel(const uint4* a, long long na, const uint4* b, long long nb,
                                                               const uint4* c, long long nc, T* out, long long N, long long O,
                                                               long long ldo, int tile, unsigned* sink) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  unsigned acc = 0;
  const uint4* src[3] = {a, b, c};
  const long long cnt[3] = {na, nb, nc};
#pragma unroll
  for (int s = 0; s < 3; ++s)
    for (long long i = tid; i < cnt[s]; i += nth) {
      uint4 v;
      asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src[s] + i));
      acc ^= v.x ^ v.y ^ v.z ^ v.w;
    }
  if (acc == 0x9E3779B9u && sink) *sink = acc;  // keeps the loads alive; practically never taken
  for (long long e = tid; e < N * O; e += nth) {
    const long long n = e / O, o = e - n * O;
    out[n * ldo + o] = static_cast<T>(tile > 0 ? (float)(o / tile) : 0.f);
  }
}
}  // namespace blr

extern "C" int blr_load_store_probe(const void* a, size_t a_bytes, const void* b, size_t b_bytes, const void* c, size_t c_bytes,
                                    int out_kind, void* out, int64_t n_tokens, int64_t out_features, int64_t ldo, int tile,
                                    void* stream) {
  using namespace blr;
  BLR_REQUIRE(out != nullptr && n_tokens >= 0 && out_features > 0 && ldo >= out_features, BLR_ERR_ARG, "bad output arguments");
  BLR_REQUIRE(out_kind >= 0 && out_kind <= 2, BLR_ERR_ARG, "out_kind must be 0 (f16), 1 (bf16) or 2 (f32)");
  const void* ptrs[3] = {a, b, c};
  const size_t bytes[3] = {a_bytes, b_bytes, c_bytes};
  for (int i = 0; i < 3; ++i)
    BLR_REQUIRE(bytes[i] == 0 || (ptrs[i] != nullptr && (reinterpret_cast<uintptr_t>(ptrs[i]) & 15) == 0 && bytes[i] % 16 == 0),
                BLR_ERR_ALIGN, "operand %d must be 16-byte aligned and a multiple of 16 bytes long", i);
  if (n_tokens == 0) return BLR_OK;
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)di.sm_count * 8;
#define BLR_PROBE(T)                                                                                                     \
  load_store_probe_kernel<T><<<grid, 256, 0, st>>>(static_cast<const uint4*>(a), (long long)(a_bytes / 16),              \
                                                   static_cast<const uint4*>(b), (long long)(b_bytes / 16),              \
                                                   static_cast<const uint4*>(c), (long long)(c_bytes / 16),              \
                                                   static_cast<T*>(out), (long long)n_tokens, (long long)out_features,    \
                                                   (long long)ldo, tile, nullptr)
  if (out_kind == 0) BLR_PROBE(__half);
  else if (out_kind == 1) BLR_PROBE(__nv_bfloat16);
  else BLR_PROBE(float);
#undef BLR_PROBE
  BLR_CUDA_OK(cudaGetLastError());
  return BLR_OK;
}
