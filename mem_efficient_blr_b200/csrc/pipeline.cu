// Tensor-core pipeline for more than 16 tokens: grouped tcgen05 GEMMs (umma_gemm.cu) chained through
// 16-bit intermediates; the BLAST coupling between the two GEMMs is itself a grouped GEMM (see
// expand_coupling_kernel).
#include "pipeline.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tmap.h"
#include "umma_gemm.h"

namespace blr {

static CUtensorMapDataType dt16(int dtype) {
  return dtype == BLR_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

static constexpr int kCoupleTileMaxTokens = 256;  // above: coupling as a grouped GEMM over expanded factors

// Launch with programmatic stream serialisation: the kernel may start while its predecessor drains; it calls
// griddepcontrol.launch_dependents at its start and griddepcontrol.wait before it touches what the predecessor wrote.
template <typename K, typename... A>
static int launch_pdl(K kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st, A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  BLR_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, args...));
  return BLR_OK;
}

struct OutSpec {
  void* out;
  long long os_g, os_n, os_hi, os_lo;
  int per;
  int round_out;
  // added to the result where the output is laid out [n][g * M + m]: bias[g * M + m], residual[n * ldr + g * M + m]
  const void* bias = nullptr;
  const void* residual = nullptr;
  long long ldr = 0;
  int act = 0;  // after the bias, before the residual: 1 GELU, 2 GELU (tanh)
};

// Quantised weights of one GEMM: bits 8 | 4 (16: none), fp16 scales per weight row (group = 0) or per `group`
// contraction indices.
struct QuantSpec {
  int bits = 16;
  const void* scale = nullptr;
  int group = 0;
};

// One grouped GEMM: W (G blocks of M rows over K), A[g][n][k] with element strides (1, ld_n, ld_g).
static int run_gemm(int dtype, const void* W, int layout, int G, int M, int K, const void* A, int64_t N, int64_t ld_n,
                    int64_t ld_g, const OutSpec& o, cudaStream_t stream, const QuantSpec& q = QuantSpec(), int64_t w_row = 0,
                    int64_t w_grp = 0) {
  // w_row / w_grp (elements, 16-bit K-major weights only; 0 = packed): the distance between consecutive rows of a
  // block and between blocks when the blocks are column slices of a wider matrix
  GemmParams p = {};
  p.G = G; p.M = M; p.K = K; p.N = (int)N;
  p.kmajor = layout == BLR_W_KMAJOR;
  p.is_bf16 = dtype == BLR_DTYPE_BF16;
  p.round_out = o.round_out;
  p.per = o.per; p.os_g = o.os_g; p.os_n = o.os_n; p.os_hi = o.os_hi; p.os_lo = o.os_lo; p.out = o.out;
  p.bias = o.bias; p.residual = o.residual; p.ldr = o.ldr; p.act_out = o.act;
  p.extra_vec = M % 8 == 0 && (reinterpret_cast<uintptr_t>(o.bias) & 15) == 0 && (reinterpret_cast<uintptr_t>(o.residual) & 15) == 0 &&
                o.ldr % 8 == 0;
  p.status = nullptr;
  BLR_REQUIRE(N < (1ll << 31), BLR_ERR_SHAPE, "too many tokens");
  const bool quant = q.bits == 8 || q.bits == 4;
  if (quant) {
    p.w_bits = q.bits;
    p.w_scale = q.scale;
    p.scales_per_row = q.group == 0 ? 1 : K / q.group;
  }
  umma_gemm_tiling(p);
  int rc;
  if (quant) {
    // the stored bytes travel as they are: rows of K * bits / 8 bytes
    const uint64_t row = (uint64_t)K * q.bits / 8;
    BLR_REQUIRE(p.kmajor && row % 16 == 0, BLR_ERR_UNSUPPORTED,
                "quantised factors above 16 tokens: contraction-contiguous rows of a multiple of 16 bytes (K = %d, %d bits)", K, q.bits);
    BLR_REQUIRE(q.group == 0 || q.group == 128, BLR_ERR_UNSUPPORTED, "scale groups of 128 contraction indices");
    const uint64_t dims[3] = {row, (uint64_t)M, (uint64_t)G};
    const uint64_t str[2] = {row, (uint64_t)M * row};
    const uint32_t box[3] = {(uint32_t)(8 * q.bits), (uint32_t)umma_w_tile_rows(p), 1};
    rc = encode_tmap_3d(&p.tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, W, dims, str, box, Swz::None);
  } else if (p.kmajor) {
    BLR_REQUIRE(K % 8 == 0, BLR_ERR_SHAPE, "contraction length %d must be a multiple of 8", K);
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)M, (uint64_t)G};
    const uint64_t str[2] = {(uint64_t)(w_row ? w_row : K) * 2, (uint64_t)(w_grp ? w_grp : (int64_t)M * K) * 2};
    const uint32_t box[3] = {64, (uint32_t)umma_w_tile_rows(p), 1};
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
  const uint32_t abox[3] = {64, (uint32_t)umma_a_tile_rows(p), 1};
  if ((rc = encode_tmap_3d(&p.tmA, dt16(dtype), A, adims, astr, abox, Swz::B128))) return rc;
  return launch_umma_gemm(p, stream);
}

// ------------------------------------------------------------------------------------------ BLAST coupling
template <typename T>
__device__ __forceinline__ float ld1(const T* p);
template <>
__device__ __forceinline__ float ld1<__half>(const __half* p) { return __half2float(*p); }
template <>
__device__ __forceinline__ float ld1<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// Expanded coupling factors: for every group of GS consecutive r (GS = 16, or 8 when R is not a multiple of
// 16), the (GS*b x GS*b) matrix
//     E[g][(i, r')][(j, r'')] = S[i][j][GS*g + r'] if r' == r'' else 0
// so that z[i][n][GS*g + r'] = sum_{(j, r'')} E[g][(i, r')][(j, r'')] * y[j][n][GS*g + r''] is one grouped GEMM with
// K = GS*b on the tensor cores.  All but 1/GS of the products are with zeros; the coupling stays bound by the
// y / z traffic.  GS = 16 makes every contiguous piece of y' and z a full 32-byte sector.
template <typename T, int GS>
__global__ void expand_coupling_kernel(const T* __restrict__ S, long long s_i, long long s_j, long long s_r,
                                       T* __restrict__ E, int b, int b_out, int R) {
  // one thread per (row (g, i, r'), in-block j): a vector of GS values with a single non-zero at position r';
  // consecutive threads write consecutive vectors of a row
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const long long total = (long long)(R / GS) * GS * b_out * b;
  const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (id >= total) {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // every thread waits: the grid must not complete before its predecessor
    return;
  }
  const int j = (int)(id % b);
  const long long row_id = id / b;
  const int h = GS * b_out, row = (int)(row_id % h), g = (int)(row_id / h), i = row / GS, r1 = row % GS;
  alignas(16) T v[GS];
#pragma unroll
  for (int k = 0; k < GS; ++k) v[k] = T(0.f);
  v[r1] = S[i * s_i + j * s_j + (long long)(GS * g + r1) * s_r];
  // the factors do not depend on the previous kernel; E may still be read by it (the coupling GEMM of the previous
  // call on this workspace), so the stores wait for its completion
  asm volatile("griddepcontrol.wait;" ::: "memory");
  T* dst = E + id * GS;
#pragma unroll
  for (int k = 0; k < GS / 8; ++k) *reinterpret_cast<uint4*>(dst + 8 * k) = *reinterpret_cast<const uint4*>(v + 8 * k);
}

// Any block count / any strides: one thread per output element.
template <typename T>
__global__ void blast_couple_generic_kernel(const T* __restrict__ y, const T* __restrict__ S, long long s_i, long long s_j,
                                            long long s_r, T* __restrict__ z, int b, int b_out, long long NR, int R, int round_z) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= NR) return;
  const int r = (int)(e % R);
  for (int i = 0; i < b_out; ++i) {
    float s = 0.f;
    for (int j = 0; j < b; ++j) s = fmaf(ld1<T>(S + i * s_i + j * s_j + (long long)r * s_r), ld1<T>(y + j * NR + e), s);
    if (round_z) s = fminf(fmaxf(rintf(s), -128.f), 127.f);
    z[i * NR + e] = T(s);
  }
}

template <typename T>
static int run_couple_generic(const void* y, const void* S, int64_t s_i, int64_t s_j, int64_t s_r, void* z, int b, int b_out,
                              int64_t N, int R, int round_z, cudaStream_t stream) {
  const long long NR = (long long)N * R;
  blast_couple_generic_kernel<T><<<(unsigned)((NR + 255) / 256), 256, 0, stream>>>(
      static_cast<const T*>(y), static_cast<const T*>(S), s_i, s_j, s_r, static_cast<T*>(z), b, b_out, NR, R, round_z);
  BLR_CUDA_OK(cudaGetLastError());
  return BLR_OK;
}

// Coupling on the CUDA cores for a few hundred tokens, where building and multiplying the expanded factors costs more
// than the coupling itself: a block takes 64 consecutive ranks, stages S[i][j][64 ranks] for all pairs of blocks in
// shared memory once, and walks its share of the tokens; a thread owns 8 ranks of one token, holds the b vectors
// y_j in registers and produces the b_out vectors z_i.  y, z: [block][token][R], S with unit rank stride.
// With few tokens the out-blocks are shared out over grid.y as well (i_per per block), so that the grid still fills
// the GPU: every such block re-reads the y vectors (from L2) but stages and applies only its own rows of S.
template <typename T, int B>
__global__ void __launch_bounds__(256) blast_couple_tile_kernel(const T* __restrict__ y, const T* __restrict__ S, long long s_i,
                                                                long long s_j, T* __restrict__ z, int b_out, long long N, int R,
                                                                int round_z, int tok_groups, int i_per) {
  extern __shared__ __align__(16) unsigned char couple_smem[];
  T* sS = reinterpret_cast<T*>(couple_smem);  // [i_per][B][64]
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int rt = blockIdx.x / tok_groups, tg = blockIdx.x - rt * tok_groups, r0 = rt * 64;
  const int i_lo = blockIdx.y * i_per, i_n = min(i_per, b_out - i_lo);
  for (int e = threadIdx.x; e < i_n * B * 8; e += 256) {
    const int ij = e >> 3, v = e & 7, il = ij / B, j = ij - il * B, i = i_lo + il;
    uint4 w = make_uint4(0, 0, 0, 0);
    if (r0 + v * 8 < R) w = __ldg(reinterpret_cast<const uint4*>(S + i * s_i + j * s_j + r0 + v * 8));
    reinterpret_cast<uint4*>(sS)[e] = w;
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");  // y comes from the previous kernel; z may still be read by an earlier one
  __syncthreads();
  const int v = threadIdx.x & 7, nl = threadIdx.x >> 3;  // 8 rank vectors x 32 tokens per pass
  const long long plane = N * R;
  if (r0 + v * 8 >= R) return;
  for (long long n = (long long)tg * 32 + nl; n < N; n += (long long)tok_groups * 32) {
    float yv[B][8];
#pragma unroll
    for (int j = 0; j < B; ++j) {
      const uint4 w = *reinterpret_cast<const uint4*>(y + j * plane + n * R + r0 + v * 8);
      const T* h = reinterpret_cast<const T*>(&w);
#pragma unroll
      for (int k = 0; k < 8; ++k) yv[j][k] = (float)h[k];
    }
    for (int il = 0; il < i_n; ++il) {
      const int i = i_lo + il;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < B; ++j) {
        const uint4 w = reinterpret_cast<const uint4*>(sS)[(il * B + j) * 8 + v];
        const T* h = reinterpret_cast<const T*>(&w);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = fmaf((float)h[k], yv[j][k], acc[k]);
      }
      alignas(16) T o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = T(round_z ? fminf(fmaxf(rintf(acc[k]), -128.f), 127.f) : acc[k]);
      *reinterpret_cast<uint4*>(z + i * plane + n * R + r0 + v * 8) = *reinterpret_cast<const uint4*>(o);
    }
  }
}

template <typename T>
static int run_couple_tile(const void* y, const void* S, int64_t s_i, int64_t s_j, void* z, int b, int b_out, int64_t N, int R,
                           int round_z, cudaStream_t stream) {
  const void* kern = nullptr;
  switch (b) {
    case 2: kern = (const void*)blast_couple_tile_kernel<T, 2>; break;
    case 3: kern = (const void*)blast_couple_tile_kernel<T, 3>; break;
    case 4: kern = (const void*)blast_couple_tile_kernel<T, 4>; break;
    case 6: kern = (const void*)blast_couple_tile_kernel<T, 6>; break;
    case 8: kern = (const void*)blast_couple_tile_kernel<T, 8>; break;
    case 9: kern = (const void*)blast_couple_tile_kernel<T, 9>; break;
    case 12: kern = (const void*)blast_couple_tile_kernel<T, 12>; break;
    case 16: kern = (const void*)blast_couple_tile_kernel<T, 16>; break;
    default: return 1;  // no instantiation for this block count
  }
  // One wave: as many blocks as are resident at once.  (With 16 blocks a thread holds 128 values of y in registers and
  // one block fits an SM; twice as many blocks as fit ran as two waves, 12.5 instead of about 8 us at 128 tokens.)
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != BLR_OK) return rc;
  static int resident[64][17] = {};  // blocks per SM of this instance, per device (0: not asked yet)
  int dev = 0;
  BLR_CUDA_OK(cudaGetDevice(&dev));
  int& per_sm = resident[dev & 63][b];
  if (per_sm == 0) {
    int n = 1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, 256, (size_t)2 * b * 64 * sizeof(T)) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = 1;
    }
    per_sm = n > 2 ? 2 : n;
  }
  const int r_tiles = (R + 63) / 64;
  int tok_groups = (int)((N + 31) / 32);
  const int want = (per_sm * di.sm_count) / r_tiles > 0 ? (per_sm * di.sm_count) / r_tiles : 1;
  if (tok_groups > want) tok_groups = want;
  // too few blocks for the GPU: share the out-blocks out as well (at least two per block)
  int i_groups = want / tok_groups;
  if (i_groups > b_out / 2) i_groups = b_out / 2;
  if (i_groups < 1) i_groups = 1;
  int i_per = (b_out + i_groups - 1) / i_groups;
  i_groups = (b_out + i_per - 1) / i_per;
  const size_t smem = (size_t)i_per * b * 64 * sizeof(T);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(r_tiles * tok_groups), (unsigned)i_groups);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  const T* yp = static_cast<const T*>(y);
  const T* Sp = static_cast<const T*>(S);
  T* zp = static_cast<T*>(z);
  long long si = s_i, sj = s_j, n = N;
  void* args[] = {&yp, &Sp, &si, &sj, &zp, &b_out, &n, &R, &round_z, &tok_groups, &i_per};
  if (smem > 48 * 1024) BLR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  BLR_CUDA_OK(cudaLaunchKernelExC(&cfg, kern, args));
  return BLR_OK;
}

template <typename T>
static int run_expand(const void* S, int64_t s_i, int64_t s_j, int64_t s_r, void* E, int b, int b_out, int R, int gs,
                      cudaStream_t stream) {
  const long long total = (long long)(R / gs) * gs * b_out * b;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  const T* Sp = static_cast<const T*>(S);
  T* Ep = static_cast<T*>(E);
  void* args[] = {&Sp, &s_i, &s_j, &s_r, &Ep, &b, &b_out, &R};
  if (gs == 16) BLR_CUDA_OK(cudaLaunchKernelExC(&cfg, (const void*)expand_coupling_kernel<T, 16>, args));
  else BLR_CUDA_OK(cudaLaunchKernelExC(&cfg, (const void*)expand_coupling_kernel<T, 8>, args));
  return BLR_OK;
}

// ------------------------------------------------------------------------------------------ operators
int pipeline_blast(const void* x, int64_t ldx, int64_t N, int dtype, const void* U, int u_layout, const void* V,
                   int v_layout, const void* S, int64_t s_i, int64_t s_j, int64_t s_r, int b, int b_out, int P, int Q, int R,
                   int act_int8, void* out, int64_t ldo, void* y16, void* z16, void* e16, cudaStream_t stream, const void* e_ready,
                   const BlastQuant* quant, const void* bias, const void* residual, int64_t ldr, int out_act) {
  QuantSpec qu, qv;  // quantised U / V: widened tile by tile inside the GEMMs that read them
  if (quant != nullptr) {
    qu.bits = quant->u_bits, qu.scale = quant->u_scale, qu.group = quant->group;
    qv.bits = quant->v_bits, qv.scale = quant->v_scale, qv.group = quant->group;
  }
  const long long plane = (long long)N * R;
  const bool bf = dtype == BLR_DTYPE_BF16;
  int rc;
  // Up to a few hundred tokens the coupling is cheaper on the CUDA cores (one kernel, factors staged in shared
  // memory) than as a GEMM over expanded factors (two kernels, 16x the products).
  const bool s_vec = s_r == 1 && (s_i & 7) == 0 && (s_j & 7) == 0 && (reinterpret_cast<uintptr_t>(S) & 15) == 0;
  if (N <= kCoupleTileMaxTokens && R % 8 == 0 && s_vec && b <= 16) {
    rc = run_gemm(dtype, V, v_layout, b, R, P, x, N, ldx, P, OutSpec{y16, plane, R, 0, 1, R, act_int8}, stream, qv);
    if (rc) return rc;
    rc = bf ? run_couple_tile<__nv_bfloat16>(y16, S, s_i, s_j, z16, b, b_out, N, R, act_int8, stream)
            : run_couple_tile<__half>(y16, S, s_i, s_j, z16, b, b_out, N, R, act_int8, stream);
    if (rc < 0) return rc;
    if (rc == 0) return run_gemm(dtype, U, u_layout, b_out, Q, R, z16, N, R, plane, OutSpec{out, Q, ldo, 0, 1, Q, 0, bias, residual, ldr, out_act}, stream, qu);
    // rc == 1: no instantiation for this block count; y16 is overwritten below in the layout that path wants
  }
  if (b <= 16 && R % 8 == 0) {
    // y'[n][r/GS][j][r%GS] = sum_p V[j][r][p] x[n][j*P + p]: the (j, r%GS) index is contiguous, ready to be the
    // K dimension of the coupling GEMM
    const int gs = R % 16 == 0 ? 16 : 8, w = gs * b;
    rc = run_gemm(dtype, V, v_layout, b, R, P, x, N, ldx, P, OutSpec{y16, gs, (long long)R * b, w, 1, gs, act_int8}, stream, qv);
    if (rc) return rc;
    if (e_ready != nullptr) {
      e16 = const_cast<void*>(e_ready);  // expanded once by the caller (pipeline_expand_coupling), valid while S is unchanged
    } else {
      rc = bf ? run_expand<__nv_bfloat16>(S, s_i, s_j, s_r, e16, b, b_out, R, gs, stream)
              : run_expand<__half>(S, s_i, s_j, s_r, e16, b, b_out, R, gs, stream);
      if (rc) return rc;
    }
    // z[i][n][GS*g + r'] = sum_k E[g][(i, r')][k] y'[n][g][k]
    rc = run_gemm(dtype, e16, BLR_W_KMAJOR, R / gs, gs * b_out, w, y16, N, (int64_t)R * b, w, OutSpec{z16, gs, R, plane, 1, gs, act_int8}, stream);
    if (rc) return rc;
  } else {
    // y[j][n][r] = sum_p V[j][r][p] x[n][j*P + p]
    rc = run_gemm(dtype, V, v_layout, b, R, P, x, N, ldx, P, OutSpec{y16, plane, R, 0, 1, R, act_int8}, stream, qv);
    if (rc) return rc;
    rc = bf ? run_couple_generic<__nv_bfloat16>(y16, S, s_i, s_j, s_r, z16, b, b_out, N, R, act_int8, stream)
            : run_couple_generic<__half>(y16, S, s_i, s_j, s_r, z16, b, b_out, N, R, act_int8, stream);
    if (rc) return rc;
  }
  // out[n][i*Q + q] = sum_r U[i][q][r] z[i][n][r]
  return run_gemm(dtype, U, u_layout, b_out, Q, R, z16, N, R, plane, OutSpec{out, Q, ldo, 0, 1, Q, 0, bias, residual, ldr, out_act}, stream, qu);
}

size_t pipeline_coupling_bytes(int b, int b_out, int R) {
  if (b > 16 || R % 8 != 0) return 0;  // (the coupling of such shapes does not run as a GEMM over expanded factors)
  const int gs = R % 16 == 0 ? 16 : 8;
  return (size_t)R * gs * b_out * b * 2;
}

int pipeline_expand_coupling(const void* S, int64_t s_i, int64_t s_j, int64_t s_r, int b, int b_out, int R, int dtype, void* E,
                             cudaStream_t stream) {
  const int gs = R % 16 == 0 ? 16 : 8;
  return dtype == BLR_DTYPE_BF16 ? run_expand<__nv_bfloat16>(S, s_i, s_j, s_r, E, b, b_out, R, gs, stream)
                                 : run_expand<__half>(S, s_i, s_j, s_r, E, b, b_out, R, gs, stream);
}

// Transposes small matrices: in[a][c] (A x C, contiguous) -> out[c * out_c + a], kRowsPerCta matrices per CTA.
// Matrix (g, r), r < rows, is read at g * in_g + r * A * C and written at g * out_g + r * out_r.
// A GEMM that would scatter 2-byte stores across planes (Monarch's middle permutation on the torch layout) or across
// 32-byte sectors (Monarch's interleaved output) writes its natural layout instead, and this pass re-orders it:
// 16-byte global loads, element-wise through shared memory (pitch C + 2: the transposed reads touch all banks),
// 16-byte global stores where eight consecutive outputs are contiguous and aligned.
static constexpr int kRowsPerCta = 4;

__global__ void __launch_bounds__(256) transpose_rows_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out,
                                                             int A, int C, long long rows, long long in_g, long long out_g,
                                                             long long out_r, long long out_c, int vec_out) {
  extern __shared__ uint16_t tile[];  // [kRowsPerCta][A][C + 2]
  const long long chunks = (rows + kRowsPerCta - 1) / kRowsPerCta;
  const long long g = blockIdx.x / chunks, r0 = (blockIdx.x - g * chunks) * kRowsPerCta;
  const int nr = (int)(rows - r0 < kRowsPerCta ? rows - r0 : kRowsPerCta);
  const int pitch = C + 2, mat = A * C, total = nr * mat, step = blockDim.x * 8;
  const uint16_t* src = in + g * in_g + r0 * mat;
  {  // linear read of nr contiguous matrices, eight elements per thread and step (mat is a multiple of 8)
    for (int e = threadIdx.x * 8; e < total; e += step) {
      const uint4 v = *reinterpret_cast<const uint4*>(src + e);
      const uint16_t* h = reinterpret_cast<const uint16_t*>(&v);
      const int r = e / mat, em = e - r * mat;
      int a = em / C, c = em - a * C;
      uint16_t* t = tile + r * A * pitch;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        t[a * pitch + c] = h[k];
        if (++c == C) { c = 0; ++a; }
      }
    }
  }
  __syncthreads();
  for (int r = 0; r < nr; ++r) {
    const uint16_t* t = tile + r * A * pitch;
    uint16_t* dst = out + g * out_g + (r0 + r) * out_r;
    if (vec_out) {  // A % 8 == 0 and every run of A outputs starts 16-byte aligned
      for (int e = threadIdx.x * 8; e < mat; e += step) {
        const int c = e / A, a = e - c * A;
        uint4 v;
        uint16_t* h = reinterpret_cast<uint16_t*>(&v);
#pragma unroll
        for (int k = 0; k < 8; ++k) h[k] = t[(a + k) * pitch + c];
        *reinterpret_cast<uint4*>(dst + c * out_c + a) = v;
      }
    } else {
      for (int e = threadIdx.x; e < mat; e += blockDim.x) {
        const int c = e / A, a = e - c * A;
        dst[c * out_c + a] = t[a * pitch + c];
      }
    }
  }
}

// The same re-ordering when one side of the matrices is small (D = 2, 4, 8 or 16: Monarch's block count): an 8 x D
// piece is transposed in registers, 16-byte loads and stores on both sides, no shared memory and no division per element.
//   GATHER:  in[d][c] (D rows of C)  -> out[c * D + d]        a thread takes 8 consecutive c of all D rows and writes
//            8 * D consecutive outputs (the interleaved output features of a token)
//   !GATHER: in[a][d] (A rows of D)  -> out[d * out_c + a]    a thread takes 8 consecutive a (8 * D contiguous inputs)
//            and writes 8 of them to each of the D destinations (the middle permutation on the torch layout)
// Matrix (g, r) at in + g * in_g + r * A * C, written at out + g * out_g + r * out_r; `items` threads per matrix.
template <int D, bool GATHER>
__global__ void __launch_bounds__(256) reorder_small_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int L,
                                                            long long rows, long long in_g, long long out_g, long long out_r,
                                                            long long out_c, int items, long long total) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // (every thread: the grid completes after its predecessor)
  const long long id = (long long)blockIdx.x * 256 + threadIdx.x;
  if (id >= total) return;
  const long long m = id / items;  // matrix (g, r)
  const int it = (int)(id - m * items);
  const long long g = m / rows, r = m - g * rows;
  const uint16_t* src = in + g * in_g + r * (long long)L * D;
  uint16_t* dst = out + g * out_g + r * out_r;
  alignas(16) uint16_t v[D][8];  // GATHER: [d][c];  !GATHER: the 8 * D inputs in order, i.e. [a][d] flattened
  alignas(16) uint16_t w[D][8];
  if constexpr (GATHER) {
#pragma unroll
    for (int d = 0; d < D; ++d) *reinterpret_cast<uint4*>(v[d]) = *reinterpret_cast<const uint4*>(src + (long long)d * L + it * 8);
    uint16_t* wf = &w[0][0];  // outputs (c, d) in order
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
      for (int d = 0; d < D; ++d) wf[c * D + d] = v[d][c];
#pragma unroll
    for (int k = 0; k < D; ++k) *reinterpret_cast<uint4*>(dst + ((long long)it * 8) * D + k * 8) = *reinterpret_cast<const uint4*>(w[k]);
  } else {
#pragma unroll
    for (int k = 0; k < D; ++k) *reinterpret_cast<uint4*>(v[k]) = *reinterpret_cast<const uint4*>(src + ((long long)it * 8) * D + k * 8);
    const uint16_t* vf = &v[0][0];  // inputs (a, d) in order
#pragma unroll
    for (int d = 0; d < D; ++d)
#pragma unroll
      for (int a = 0; a < 8; ++a) w[d][a] = vf[a * D + d];
#pragma unroll
    for (int d = 0; d < D; ++d) *reinterpret_cast<uint4*>(dst + d * out_c + it * 8) = *reinterpret_cast<const uint4*>(w[d]);
  }
}

template <int D>
static int reorder_small(bool gather, const uint16_t* in, uint16_t* out, int L, long long groups, long long rows, long long in_g,
                         long long out_g, long long out_r, long long out_c, cudaStream_t stream) {
  const int items = L / 8;
  const long long total = groups * rows * items;
  BLR_REQUIRE((total + 255) / 256 < (1ll << 31), BLR_ERR_SHAPE, "too many rows to re-order");
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (gather) return launch_pdl(reorder_small_kernel<D, true>, dim3(blocks), dim3(256), 0, stream, in, out, L, rows, in_g, out_g, out_r, out_c, items, total);
  return launch_pdl(reorder_small_kernel<D, false>, dim3(blocks), dim3(256), 0, stream, in, out, L, rows, in_g, out_g, out_r, out_c, items, total);
}

static int transpose_rows(const void* in, void* out, int A, int C, long long groups, long long rows, long long in_g,
                          long long out_g, long long out_r, long long out_c, cudaStream_t stream) {
  {
    // one small side: the register version (everything it touches in 16-byte pieces must be aligned)
    const bool al = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 && in_g % 8 == 0 && out_g % 8 == 0 &&
                    out_r % 8 == 0;
    const bool gather = al && (A == 2 || A == 4 || A == 8 || A == 16) && C % 8 == 0 && out_c == A;
    const bool scatter = al && !gather && (C == 2 || C == 4 || C == 8 || C == 16) && A % 8 == 0 && out_c % 8 == 0;
    if (gather || scatter) {
      const uint16_t* ip = static_cast<const uint16_t*>(in);
      uint16_t* op = static_cast<uint16_t*>(out);
      const int D = gather ? A : C, L = gather ? C : A;
      switch (D) {
        case 2: return reorder_small<2>(gather, ip, op, L, groups, rows, in_g, out_g, out_r, out_c, stream);
        case 4: return reorder_small<4>(gather, ip, op, L, groups, rows, in_g, out_g, out_r, out_c, stream);
        case 8: return reorder_small<8>(gather, ip, op, L, groups, rows, in_g, out_g, out_r, out_c, stream);
        default: return reorder_small<16>(gather, ip, op, L, groups, rows, in_g, out_g, out_r, out_c, stream);
      }
    }
  }
  const size_t smem = (size_t)kRowsPerCta * A * (C + 2) * 2;
  BLR_REQUIRE((A * C) % 8 == 0, BLR_ERR_SHAPE, "re-ordering needs matrices of a multiple of 8 elements, got %d x %d", A, C);
  const long long chunks = (rows + kRowsPerCta - 1) / kRowsPerCta;
  BLR_REQUIRE(groups * chunks < (1ll << 31), BLR_ERR_SHAPE, "too many rows to re-order");
  static bool configured[64] = {};
  int dev = 0;
  BLR_CUDA_OK(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    BLR_CUDA_OK(cudaFuncSetAttribute(transpose_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    configured[dev & 63] = true;
  }
  const int vec_out = A % 8 == 0 && out_c % 8 == 0 && out_g % 8 == 0 && out_r % 8 == 0 &&
                      (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  transpose_rows_kernel<<<(unsigned)(groups * chunks), 256, smem, stream>>>(static_cast<const uint16_t*>(in),
                                                                             static_cast<uint16_t*>(out), A, C, rows, in_g,
                                                                             out_g, out_r, out_c, vec_out);
  BLR_CUDA_OK(cudaGetLastError());
  return BLR_OK;
}

// Shared memory the re-ordering pass needs for A x C matrices.
static size_t transpose_smem(int A, int C) { return (size_t)kRowsPerCta * A * (C + 2) * 2; }

// scratch: at least 4 * b * N * rank bytes (the fp32-sized region of a workspace), z16: 2 * b * N * rank bytes.
int pipeline_monarch(const void* x, int64_t ldx, int64_t N, int dtype, const void* w1, int w1_layout, int grouped,
                     const void* w2, int w2_layout, int b, int P, int rank, int Qs, int interleaved, void* out,
                     int64_t ldo, void* z16, void* scratch, cudaStream_t stream) {
  const int per = rank / b;
  const long long plane = (long long)N * rank;
  int rc;
  if (grouped) {
    // columns already grouped by destination block: column l*per + jj of block k goes to Z[l][n][k*per + jj]
    rc = run_gemm(dtype, w1, w1_layout, b, rank, P, x, N, ldx, P, OutSpec{z16, per, rank, plane, 1, per, 0}, stream);
    if (rc) return rc;
  } else if (rank % 8 == 0 && transpose_smem(per, b) <= 160 * 1024) {
    // torch layout: column jj*b + l of block k goes to Z[l][n][k*per + jj].  Written directly that is one 2-byte
    // store per plane; instead the GEMM writes pre[k][n][q] and a pass transposes every (k, n) row (per x b).
    rc = run_gemm(dtype, w1, w1_layout, b, rank, P, x, N, ldx, P, OutSpec{scratch, plane, rank, 0, 1, rank, 0}, stream);
    if (rc) return rc;
    rc = transpose_rows(scratch, z16, per, b, b, N, plane, per, rank, plane, stream);
    if (rc) return rc;
  } else {
    rc = run_gemm(dtype, w1, w1_layout, b, rank, P, x, N, ldx, P, OutSpec{z16, per, rank, 1, plane, b, 0}, stream);
    if (rc) return rc;
  }
  if (!interleaved) return run_gemm(dtype, w2, w2_layout, b, Qs, rank, z16, N, rank, plane, OutSpec{out, Qs, ldo, 0, 1, Qs, 0}, stream);
  // interleaved output, feature s*b + l: written directly, neighbouring outputs of a block are b elements apart
  // (one sector per 2-byte store).  When the scratch region can hold the block-major result, write that and
  // transpose every token's (b x Qs) row.
  if (Qs <= 2 * rank && (b * Qs) % 8 == 0 && transpose_smem(b, Qs) <= 160 * 1024) {
    rc = run_gemm(dtype, w2, w2_layout, b, Qs, rank, z16, N, rank, plane,
                  OutSpec{scratch, Qs, (long long)b * Qs, 0, 1, Qs, 0}, stream);
    if (rc) return rc;
    return transpose_rows(scratch, out, b, Qs, 1, N, 0, 0, ldo, b, stream);
  }
  return run_gemm(dtype, w2, w2_layout, b, Qs, rank, z16, N, rank, plane, OutSpec{out, 1, ldo, 0, b, Qs, 0}, stream);
}

// z[e] = sum over the planes of parts[plane][e] (fp32 sums of 16-bit values), 8 elements per thread.
template <typename T>
__global__ void __launch_bounds__(256) sum_planes_kernel(const T* __restrict__ parts, int nparts, long long plane, T* __restrict__ z) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const long long e = ((long long)blockIdx.x * 256 + threadIdx.x) * 8;
  if (e >= plane) return;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int g = 0; g < nparts; ++g) {
    const uint4 v = *reinterpret_cast<const uint4*>(parts + (long long)g * plane + e);
    const T* h = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] += (float)h[k];
  }
  alignas(16) T o[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) o[k] = T(acc[k]);
  *reinterpret_cast<uint4*>(z + e) = *reinterpret_cast<const uint4*>(o);
}

// parts: room for the first stage's partial results (parts_bytes; may be null).  With few tokens the first GEMM has
// few tiles (R / 128 or so) over a long contraction, i.e. a handful of CTAs that each stream megabytes: the
// contraction is then cut into up to 16 slices that run as the groups of one grouped GEMM (the slices of V are column
// ranges of its rows, or packed row ranges when the output index is contiguous) and a small kernel adds the slices.
int pipeline_low_rank(const void* x, int64_t ldx, int64_t N, int dtype, const void* V, int v_layout, const void* U,
                      int u_layout, int I, int R, int O, void* out, int64_t ldo, void* z16, void* parts, size_t parts_bytes,
                      cudaStream_t stream) {
  int rc;
  int split = 1;
  const long long tiles = (long long)((R + 127) / 128) * ((N + 127) / 128);
  if (parts != nullptr && tiles < 74 && ((long long)N * R) % 8 == 0) {
    for (int sp = 16; sp >= 2; sp >>= 1) {
      if (I % (sp * 8) != 0 || I / sp < 256 || tiles * sp > 2 * 148 || (size_t)sp * N * R * 2 > parts_bytes) continue;
      split = sp;
      break;
    }
  }
  if (split > 1) {
    const int Ks = I / split;
    const bool vk = v_layout == BLR_W_KMAJOR;
    rc = run_gemm(dtype, V, v_layout, split, R, Ks, x, N, ldx, Ks, OutSpec{parts, (long long)N * R, R, 0, 1, R, 0}, stream, QuantSpec(),
                  vk ? I : 0, vk ? Ks : 0);
    if (rc) return rc;
    const long long plane = (long long)N * R;
    const unsigned blocks = (unsigned)((plane / 8 + 255) / 256);
    if (dtype == BLR_DTYPE_BF16)
      rc = launch_pdl(sum_planes_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(parts), split, plane,
                      static_cast<__nv_bfloat16*>(z16));
    else
      rc = launch_pdl(sum_planes_kernel<__half>, dim3(blocks), dim3(256), 0, stream, static_cast<const __half*>(parts), split, plane,
                      static_cast<__half*>(z16));
    if (rc) return rc;
  } else {
    rc = run_gemm(dtype, V, v_layout, 1, R, I, x, N, ldx, 0, OutSpec{z16, 0, R, 0, 1, R, 0}, stream);
    if (rc) return rc;
  }
  return run_gemm(dtype, U, u_layout, 1, O, R, z16, N, R, 0, OutSpec{out, 0, ldo, 0, 1, O, 0}, stream);
}

int pipeline_dense(const void* x, int64_t ldx, int64_t N, int dtype, const void* W, int w_layout, int I, int O, void* out,
                   int64_t ldo, cudaStream_t stream) {
  return run_gemm(dtype, W, w_layout, 1, O, I, x, N, ldx, 0, OutSpec{out, 0, ldo, 0, 1, O, 0}, stream);
}

}  // namespace blr
