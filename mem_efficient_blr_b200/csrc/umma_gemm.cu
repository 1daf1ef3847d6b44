// tcgen05 / TMEM grouped GEMM (sm_100a).  Persistent, one CTA per SM, warp-specialised:
//   warp 0   TMA producer: weight tile (128 rows x 64 k, 16 KB) + token tile (bn tokens x 64 k) per stage
//   warp 1   MMA issuer: one elected thread issues tcgen05.mma (M = 128, N = bn, K = 16) from shared-memory
//            descriptors, accumulators double-buffered in TMEM (2 x bn columns)
//   warps 2-5 epilogue: tcgen05.ld the accumulator (one weight row per thread, tokens along the columns),
//            convert and scatter to the output mapping
// All waits are bounded; a time-out sets *status and the kernel drains and frees its TMEM.
#include "ptx.cuh"
#include "tmap.h"
#include "umma_gemm.h"

namespace blr {

static constexpr int kGemmThreads = 192;
static constexpr int kBM = 128;
static constexpr int kBK = 64;
static constexpr int kWTileBytes = kBM * kBK * 2;
static constexpr int kMaxStages = 8;

template <bool BF16>
__device__ __forceinline__ void gemm_store(void* base, long long off, float v) {
  if constexpr (BF16) reinterpret_cast<__nv_bfloat16*>(base)[off] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(base)[off] = __float2half_rn(v);
}

template <bool BF16>
__global__ void __launch_bounds__(kGemmThreads, 1) blr_umma_gemm_kernel(const __grid_constant__ GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t a_tile_bytes = (uint32_t)p.bn * kBK * 2;
  const uint32_t stage_bytes = kWTileBytes + a_tile_bytes;
  const uint32_t NST = p.nstages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)NST * stage_bytes);
  // full[8], empty[8], tmem_full[2], tmem_empty[2]
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kMaxStages);
  const uint32_t tfull0 = smem_u32(bars + 2 * kMaxStages), tempty0 = smem_u32(bars + 2 * kMaxStages + 2);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + kBM - 1) / kBM, n_tiles = (p.N + p.bn - 1) / p.bn;
  const int tiles = p.G * m_tiles * n_tiles;
  const int kblocks = (p.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (uint32_t s = 0; s < NST; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull0 + 8 * b, 1);
      mbar_init(tempty0 + 8 * b, 4);  // one arrival per epilogue warp
    }
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&p.tmW);
      tma_prefetch_desc(&p.tmA);
      uint32_t s = 0, parity = 0;
      bool first = true, ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int nt = tile % n_tiles, gm = tile / n_tiles, mt = gm % m_tiles, g = gm / m_tiles;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!first && !mbar_wait(empty0 + 8 * s, parity ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t dst = smem_base + s * stage_bytes, bar = full0 + 8 * s;
          mbar_arrive_expect_tx(bar, stage_bytes);
          if (p.kmajor) {
            tma_load_3d(dst, &p.tmW, kb * kBK, mt * kBM, g, bar);
          } else {
            tma_load_3d(dst, &p.tmW, mt * kBM, kb * kBK, g, bar);
            tma_load_3d(dst + kWTileBytes / 2, &p.tmW, mt * kBM + 64, kb * kBK, g, bar);
          }
          tma_load_3d(dst + kWTileBytes, &p.tmA, kb * kBK, nt * p.bn, g, bar);
          if (++s == NST) { s = 0; parity ^= 1u; first = false; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(BF16, !p.kmajor, kBM, (uint32_t)p.bn);
      uint32_t s = 0, parity = 0;
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++it) {
        const uint32_t buf = it & 1u, use = it >> 1;
        // wait until the epilogue has drained this accumulator buffer (first use of each buffer is free)
        if (use > 0 && !mbar_wait(tempty0 + 8 * buf, (use - 1) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * (uint32_t)p.bn;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full0 + 8 * s, parity, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sW = smem_base + s * stage_bytes, sA = sW + kWTileBytes;
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            uint64_t adesc;
            if (p.kmajor) adesc = umma_smem_desc(sW + kk * 32, 16, 1024);
            else adesc = umma_smem_desc(sW + kk * 2048, kWTileBytes / 2, 1024);
            const uint64_t bdesc = umma_smem_desc(sA + kk * 32, 16, 1024);
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * s);  // frees the stage once these MMAs have read it
          if (++s == NST) { s = 0; parity ^= 1u; }
        }
        if (ok) umma_commit(tfull0 + 8 * buf);  // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------ epilogue: warp w reads TMEM lanes 32*(w%4)..+31
    const int q = warp & 3;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
      const int nt = tile % n_tiles, gm = tile / n_tiles, mt = gm % m_tiles, g = gm / m_tiles;
      const uint32_t buf = it & 1u, use = it >> 1;
      if (ok && !mbar_wait(tfull0 + 8 * buf, use & 1u, abort_flag)) ok = false;
      if (!ok) continue;
      tc_fence_after();
      const int m = mt * kBM + q * 32 + lane;
      const bool m_ok = m < p.M;
      const long long base = m_ok ? (long long)g * p.os_g + (long long)(m / p.per) * p.os_hi + (long long)(m % p.per) * p.os_lo : 0;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * (uint32_t)p.bn;
      const int n0 = nt * p.bn;
      for (int c = 0; c < p.bn; c += 16) {
        if (n0 + c >= p.N) break;  // whole chunk past the last token (warp-uniform)
        uint32_t r[16];
        tmem_ld16(taddr + c, r);
        tmem_ld_wait();
        if (m_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int n = n0 + c + j;
            if (n < p.N) {
              float v = __uint_as_float(r[j]);
              if (p.round_out) v = fminf(fmaxf(rintf(v), -128.f), 127.f);
              gemm_store<BF16>(p.out, base + (long long)n * p.os_n, v);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * buf);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1u);
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);  // let loads in flight land before the CTA's memory is released
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

void umma_gemm_tiling(GemmParams& p) {
  int bn = 256;
  if (p.N <= 256) bn = (p.N + 15) / 16 * 16;
  if (bn < 16) bn = 16;
  p.bn = bn;
  const int stage = kWTileBytes + bn * kBK * 2;
  int nst = (232448 - 1024 - 512) / stage;
  p.nstages = nst > kMaxStages ? kMaxStages : nst;
}

int launch_umma_gemm(const GemmParams& p, cudaStream_t stream) {
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != BLR_OK) return rc;
  const size_t smem = (size_t)p.nstages * (kWTileBytes + p.bn * kBK * 2) + 512 + 1024;
  BLR_REQUIRE((int)smem <= di.max_smem_optin, BLR_ERR_UNSUPPORTED, "needs %zu bytes of shared memory, device offers %d",
              smem, di.max_smem_optin);
  BLR_REQUIRE(p.bn % 16 == 0 && p.bn >= 16 && p.bn <= 256 && p.nstages >= 2, BLR_ERR_ARG, "bad tile configuration");
  int dev;
  BLR_CUDA_OK(cudaGetDevice(&dev));
  const int m_tiles = (p.M + kBM - 1) / kBM, n_tiles = (p.N + p.bn - 1) / p.bn;
  const long long tiles = (long long)p.G * m_tiles * n_tiles;
  const int grid = (int)(tiles < di.sm_count ? tiles : di.sm_count);
  if (p.is_bf16) {
    static bool configured[64] = {};
    if (!configured[dev & 63]) {
      BLR_CUDA_OK(cudaFuncSetAttribute(blr_umma_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem_optin));
      configured[dev & 63] = true;
    }
    blr_umma_gemm_kernel<true><<<grid, kGemmThreads, smem, stream>>>(p);
  } else {
    static bool configured[64] = {};
    if (!configured[dev & 63]) {
      BLR_CUDA_OK(cudaFuncSetAttribute(blr_umma_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem_optin));
      configured[dev & 63] = true;
    }
    blr_umma_gemm_kernel<false><<<grid, kGemmThreads, smem, stream>>>(p);
  }
  BLR_CUDA_OK(cudaGetLastError());
  return BLR_OK;
}

}  // namespace blr
