// Weight-streaming kernel for decode-size token counts (N <= 16) on sm_100a.
//
// One persistent CTA per SM.  Two single-thread producers feed a ring of shared-memory stages with
// TMA tile loads: one streams weight tiles (it never waits for anything but a free stage, so HBM
// stays busy across the grid barriers), the other streams the matching activation boxes (it waits
// at the grid barrier before it touches activations written by other CTAs).  Eight consumer
// warps take K-chunks round-robin, turn the stage into mma.sync m16n8k16 products with the
// weights as the 16-row operand and the tokens as the 8-column operand (int8 / int4 weights are
// widened in registers right before the MMA), and combine their partial sums through a small
// fp32 shared-memory buffer before the epilogue writes the phase output.
#include "ptx.cuh"
#include "stream.h"
#include "tmap.h"

namespace blr {

struct Batch {
  int g, mt0, nt;
};

__device__ __forceinline__ bool next_batch(const PhaseDesc& ph, int& t, int t_hi, Batch& b) {
  if (t >= t_hi) return false;
  b.g = t / ph.tiles_per_g;
  b.mt0 = t - b.g * ph.tiles_per_g;
  const int end = min(t_hi, (b.g + 1) * ph.tiles_per_g);
  b.nt = min(kBatchTiles, end - t);
  t += b.nt;
  return true;
}
__device__ __forceinline__ void tile_range(const PhaseDesc& ph, int& lo, int& hi) {
  lo = (int)(((long long)ph.ntiles * blockIdx.x) / gridDim.x);
  hi = (int)(((long long)ph.ntiles * (blockIdx.x + 1)) / gridDim.x);
}

// Byte offset of 16-byte chunk `c16` in row `row` of a 128-byte-swizzled box (rows of 128 B).
__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t c16) { return row * 128u + ((c16 ^ (row & 7u)) << 4); }
// Same for a 64-byte-swizzled box (rows of 64 B).
__device__ __forceinline__ uint32_t sw64(uint32_t row, uint32_t c16) { return row * 64u + ((c16 ^ ((row >> 1) & 3u)) << 4); }

template <int NT>
struct Acc {
  float v[kBatchTiles][2][NT][4];
};

// ------------------------------------------------------------------ stage consumers
// 16-bit weights, k contiguous: tile = 32 rows x 64 k.
template <bool BF16, int NT>
__device__ __forceinline__ void consume_k16(uint32_t sW, uint32_t sA, int nt_b, Acc<NT>& acc, int lane) {
  const uint32_t jm = lane >> 3, l7 = lane & 7;
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    uint32_t bf[NT][2];
    {
      const uint32_t nrow = (jm >> 1) * 8 + l7, c16 = ks * 2 + (jm & 1);
      if constexpr (NT == 2) {
        ldsm_x4(sA + sw128(nrow, c16), bf[0][0], bf[0][1], bf[1][0], bf[1][1]);
      } else {
        ldsm_x2(sA + sw128(l7, ks * 2 + (jm & 1)), bf[0][0], bf[0][1]);
      }
    }
#pragma unroll
    for (int t = 0; t < kBatchTiles; ++t) {
      if (t < nt_b) {
#pragma unroll
        for (int rg = 0; rg < 2; ++rg) {
          const uint32_t row = rg * 16 + l7 + (jm & 1) * 8, c16 = ks * 2 + (jm >> 1);
          uint32_t a0, a1, a2, a3;
          ldsm_x4(sW + t * kTileBytes + sw128(row, c16), a0, a1, a2, a3);
#pragma unroll
          for (int n = 0; n < NT; ++n) mma_16816<BF16>(acc.v[t][rg][n], a0, a1, a2, a3, bf[n][0], bf[n][1]);
        }
      }
    }
  }
}

// 16-bit weights, m contiguous: tile = 64 k-rows x 32 m (64-byte swizzle); fragments via ldmatrix.trans.
template <bool BF16, int NT>
__device__ __forceinline__ void consume_m16(uint32_t sW, uint32_t sA, int nt_b, Acc<NT>& acc, int lane) {
  const uint32_t jm = lane >> 3, l7 = lane & 7;
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    uint32_t bf[NT][2];
    {
      const uint32_t nrow = (jm >> 1) * 8 + l7, c16 = ks * 2 + (jm & 1);
      if constexpr (NT == 2) {
        ldsm_x4(sA + sw128(nrow, c16), bf[0][0], bf[0][1], bf[1][0], bf[1][1]);
      } else {
        ldsm_x2(sA + sw128(l7, ks * 2 + (jm & 1)), bf[0][0], bf[0][1]);
      }
    }
#pragma unroll
    for (int t = 0; t < kBatchTiles; ++t) {
      if (t < nt_b) {
#pragma unroll
        for (int rg = 0; rg < 2; ++rg) {
          const uint32_t krow = ks * 16 + l7 + (jm >> 1) * 8, c16 = rg * 2 + (jm & 1);
          uint32_t a0, a1, a2, a3;
          ldsm_x4_t(sW + t * kTileBytes + sw64(krow, c16), a0, a1, a2, a3);
#pragma unroll
          for (int n = 0; n < NT; ++n) mma_16816<BF16>(acc.v[t][rg][n], a0, a1, a2, a3, bf[n][0], bf[n][1]);
        }
      }
    }
  }
}

// int8 weights, k contiguous: tile = 32 rows x 128 k.  A thread's ldmatrix word holds k = 4t..4t+3 of a
// 16-wide window, so the matching activation fragment is the 8 contiguous bytes at the same k.
template <bool BF16, int NT>
__device__ __forceinline__ void consume_k8(uint32_t sW, uint32_t sA, int nt_b, Acc<NT>& acc, int lane) {
  const uint32_t jm = lane >> 3, l7 = lane & 7, g = lane >> 2, tq = lane & 3;
  constexpr uint32_t kABox = NT * 8 * 128;
#pragma unroll
  for (int win = 0; win < 4; ++win) {  // 32-byte windows of the 128-byte row
    uint32_t bf[2][NT][2];             // [half window][n-tile][b0,b1]
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const uint32_t nrow = n * 8 + g;
        const uint32_t c16 = (win & 1) * 4 + h * 2 + (tq >> 1);
        lds64(sA + (win >> 1) * kABox + sw128(nrow, c16) + (tq & 1) * 8, bf[h][n][0], bf[h][n][1]);
      }
#pragma unroll
    for (int t = 0; t < kBatchTiles; ++t) {
      if (t < nt_b) {
#pragma unroll
        for (int rg = 0; rg < 2; ++rg) {
          const uint32_t row = rg * 16 + l7 + (jm & 1) * 8, c16 = win * 2 + (jm >> 1);
          uint32_t r0, r1, r2, r3;
          ldsm_x4(sW + t * kTileBytes + sw128(row, c16), r0, r1, r2, r3);
          r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
          {
            const uint32_t a0 = cvt_u8pair<BF16>(r0, false), a1 = cvt_u8pair<BF16>(r1, false);
            const uint32_t a2 = cvt_u8pair<BF16>(r0, true), a3 = cvt_u8pair<BF16>(r1, true);
#pragma unroll
            for (int n = 0; n < NT; ++n) mma_16816<BF16>(acc.v[t][rg][n], a0, a1, a2, a3, bf[0][n][0], bf[0][n][1]);
          }
          {
            const uint32_t a0 = cvt_u8pair<BF16>(r2, false), a1 = cvt_u8pair<BF16>(r3, false);
            const uint32_t a2 = cvt_u8pair<BF16>(r2, true), a3 = cvt_u8pair<BF16>(r3, true);
#pragma unroll
            for (int n = 0; n < NT; ++n) mma_16816<BF16>(acc.v[t][rg][n], a0, a1, a2, a3, bf[1][n][0], bf[1][n][1]);
          }
        }
      }
    }
  }
}

// Packed int4 weights, k contiguous: tile = 32 rows x 256 k (128 bytes per row).  A thread's ldmatrix word
// holds k = 8t..8t+7 of a 32-wide window as nibbles; nibbles (e, e+4) convert together, so the
// activation pairs are permuted to (k_e, k_{e+4}) with prmt.
template <bool BF16, int NT>
__device__ __forceinline__ void consume_k4(uint32_t sW, uint32_t sA, int nt_b, Acc<NT>& acc, int lane) {
  const uint32_t jm = lane >> 3, l7 = lane & 7, g = lane >> 2, tq = lane & 3;
  constexpr uint32_t kABox = NT * 8 * 128;
#pragma unroll
  for (int win = 0; win < 4; ++win) {  // 32-byte windows = 64 k = one activation box
    uint32_t bf[2][NT][4];             // [half][n-tile][(k0,k4),(k1,k5),(k2,k6),(k3,k7)]
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const uint32_t nrow = n * 8 + g;
        uint32_t q0, q1, q2, q3;
        lds128(sA + win * kABox + sw128(nrow, h * 4 + tq), q0, q1, q2, q3);
        bf[h][n][0] = prmt(q0, q2, 0x5410u);
        bf[h][n][1] = prmt(q0, q2, 0x7632u);
        bf[h][n][2] = prmt(q1, q3, 0x5410u);
        bf[h][n][3] = prmt(q1, q3, 0x7632u);
      }
#pragma unroll
    for (int t = 0; t < kBatchTiles; ++t) {
      if (t < nt_b) {
#pragma unroll
        for (int rg = 0; rg < 2; ++rg) {
          const uint32_t row = rg * 16 + l7 + (jm & 1) * 8, c16 = win * 2 + (jm >> 1);
          uint32_t r[4];
          ldsm_x4(sW + t * kTileBytes + sw128(row, c16), r[0], r[1], r[2], r[3]);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t lo = r[h * 2] ^ 0x88888888u, hi = r[h * 2 + 1] ^ 0x88888888u;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const uint32_t a0 = cvt_u4pair<BF16>(lo, 2 * e), a1 = cvt_u4pair<BF16>(hi, 2 * e);
              const uint32_t a2 = cvt_u4pair<BF16>(lo, 2 * e + 1), a3 = cvt_u4pair<BF16>(hi, 2 * e + 1);
#pragma unroll
              for (int n = 0; n < NT; ++n)
                mma_16816<BF16>(acc.v[t][rg][n], a0, a1, a2, a3, bf[h][n][2 * e], bf[h][n][2 * e + 1]);
            }
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------ helpers
template <bool BF16>
__device__ __forceinline__ void store16(void* base, long long off, float v) {
  if constexpr (BF16) reinterpret_cast<__nv_bfloat16*>(base)[off] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(base)[off] = __float2half_rn(v);
}
template <bool BF16>
__device__ __forceinline__ float load16(const void* base, long long off) {
  if constexpr (BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[off]);
  else return __half2float(reinterpret_cast<const __half*>(base)[off]);
}
__device__ __forceinline__ float round_clamp_i8(float v) { return fminf(fmaxf(rintf(v), -128.f), 127.f); }
__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory"); }

// ------------------------------------------------------------------ kernel
template <bool BF16, int NT>
__global__ void __launch_bounds__(kStreamThreads, 1) blr_stream_kernel(const __grid_constant__ StreamParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // Carve: [stages][reduction buffers][barriers]
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const int NST = p.nstages;
  float* red = reinterpret_cast<float*>(smem + (size_t)NST * p.stage_bytes);   // [2][128][kRedStride]
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + 2 * 128 * kRedStride);      // full[NST], empty[NST]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * 16);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kABoxBytes = NT * 8 * 128;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < NST; ++s) {
      mbar_init(full0 + 8 * s, 2);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init_fence();
  }
  for (int i = threadIdx.x; i < 2 * 128 * kRedStride; i += blockDim.x) red[i] = 0.f;
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------------------------ weight producer
    if (lane == 0) {
      tma_prefetch_desc(&p.ph[0].tmW);
      if (p.nphases > 1) tma_prefetch_desc(&p.ph[1].tmW);
      uint32_t it = 0;
      bool ok = true;
      for (int phs = 0; phs < p.nphases && ok; ++phs) {
        const PhaseDesc& ph = p.ph[phs];
        int t, t_hi;
        tile_range(ph, t, t_hi);
        Batch b;
        while (ok && next_batch(ph, t, t_hi, b)) {
          for (int c = 0; c < ph.nchunks; ++c, ++it) {
            const uint32_t s = it % NST, use = it / NST;
            if (use > 0 && !mbar_wait(empty0 + 8 * s, (use - 1) & 1, abort_flag)) { ok = false; break; }
            const uint32_t dst = smem_base + s * p.stage_bytes, bar = full0 + 8 * s;
            mbar_arrive_expect_tx(bar, b.nt * kTileBytes);
            for (int tt = 0; tt < b.nt; ++tt) {
              const int m0 = (b.mt0 + tt) * kTileRows;
              if (ph.kmajor) tma_load_3d(dst + tt * kTileBytes, &ph.tmW, c * (ph.wbits == 16 ? 64 : 128), m0, b.g, bar);
              else tma_load_3d(dst + tt * kTileBytes, &ph.tmW, m0, c * 64, b.g, bar);
            }
          }
        }
      }
    }
  } else if (warp == kConsumerWarps + 1) {
    // ------------------------------------------------ activation producer
    if (lane == 0) {
      tma_prefetch_desc(&p.ph[0].tmA);
      if (p.nphases > 1) tma_prefetch_desc(&p.ph[1].tmA);
      uint32_t it = 0;
      bool ok = true;
      for (int phs = 0; phs < p.nphases && ok; ++phs) {
        const PhaseDesc& ph = p.ph[phs];
        int t, t_hi;
        tile_range(ph, t, t_hi);
        if (phs == 1) {
          // activations of the second phase are produced by the whole grid
          if (t < t_hi) {
            ok = wait_counter(p.counters + (p.mix ? 1 : 0), gridDim.x, abort_flag);
            fence_proxy_async();
          }
        }
        Batch b;
        while (ok && next_batch(ph, t, t_hi, b)) {
          for (int c = 0; c < ph.nchunks; ++c, ++it) {
            const uint32_t s = it % NST, use = it / NST;
            if (use > 0 && !mbar_wait(empty0 + 8 * s, (use - 1) & 1, abort_flag)) { ok = false; break; }
            const uint32_t dst = smem_base + s * p.stage_bytes + kBatchTiles * kTileBytes, bar = full0 + 8 * s;
            mbar_arrive_expect_tx(bar, ph.a_boxes * kABoxBytes);
            for (int bx = 0; bx < ph.a_boxes; ++bx)
              tma_load_3d(dst + bx * kABoxBytes, &ph.tmA, (c * ph.a_boxes + bx) * 64, 0, b.g, bar);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------ consumers
    const int ctid = threadIdx.x;  // 0..255
    uint32_t it = 0;
    int redbuf = 0;
    bool ok = true;
    for (int phs = 0; phs < p.nphases; ++phs) {
      const PhaseDesc& ph = p.ph[phs];
      int t, t_hi;
      tile_range(ph, t, t_hi);
      Batch b;
      while (next_batch(ph, t, t_hi, b)) {
        Acc<NT> acc;
#pragma unroll
        for (int a = 0; a < kBatchTiles; ++a)
#pragma unroll
          for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
              for (int e = 0; e < 4; ++e) acc.v[a][r][n][e] = 0.f;
        bool worked = false;
        // chunk c has global index it + c; this warp owns indices congruent to `warp` mod 8
        int c = (int)((warp + kConsumerWarps - (it % kConsumerWarps)) % kConsumerWarps);
        for (; c < ph.nchunks && ok; c += kConsumerWarps) {
          const uint32_t gi = it + c, s = gi % NST, use = gi / NST;
          if (!mbar_wait(full0 + 8 * s, use & 1, abort_flag)) { ok = false; break; }
          const uint32_t sW = smem_base + s * p.stage_bytes, sA = sW + kBatchTiles * kTileBytes;
          if (ph.wbits == 16) {
            if (ph.kmajor) consume_k16<BF16, NT>(sW, sA, b.nt, acc, lane);
            else consume_m16<BF16, NT>(sW, sA, b.nt, acc, lane);
          } else if (ph.wbits == 8) {
            consume_k8<BF16, NT>(sW, sA, b.nt, acc, lane);
          } else {
            consume_k4<BF16, NT>(sW, sA, b.nt, acc, lane);
          }
          worked = true;
          __syncwarp();
          if (lane == 0) mbar_arrive(empty0 + 8 * s);
        }
        it += ph.nchunks;
        // ---- combine the warps' partial sums
        float* rb = red + redbuf * 128 * kRedStride;
        if (worked) {
          const int g = lane >> 2, tq = lane & 3;
#pragma unroll
          for (int a = 0; a < kBatchTiles; ++a) {
            if (a < b.nt) {
#pragma unroll
              for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                  float* q = rb + (a * 32 + r * 16 + g) * kRedStride + n * 8 + tq * 2;
                  atomicAdd(q, acc.v[a][r][n][0]);
                  atomicAdd(q + 1, acc.v[a][r][n][1]);
                  atomicAdd(q + 8 * kRedStride, acc.v[a][r][n][2]);
                  atomicAdd(q + 8 * kRedStride + 1, acc.v[a][r][n][3]);
                }
            }
          }
        }
        consumer_bar();
        // ---- epilogue: scale, convert, scatter
        {
          const int m_base = b.mt0 * kTileRows;
          const int rows = min(b.nt * kTileRows, ph.M - m_base);
          const int total = rows * p.N;
          for (int e = ctid; e < total; e += kConsumerWarps * 32) {
            const int n = e / rows, m = e - n * rows;
            float* q = rb + m * kRedStride + n;
            float v = *q;
            *q = 0.f;
            const int mg = m_base + m;
            if (ph.scale) v *= __half2float(ph.scale[(long long)b.g * ph.M + mg]);
            if (ph.round_out) v = round_clamp_i8(v);
            const long long off = b.g * ph.os_g + n * ph.os_n + (mg / ph.per) * ph.os_hi + (mg % ph.per) * ph.os_lo;
            if (ph.out_f32) reinterpret_cast<float*>(ph.out)[off] = v;
            else store16<BF16>(ph.out, off, v);
          }
          // Padding entries (rows past the block end, token columns past N) only ever receive products
          // with zero-filled operands; clear them anyway so a non-finite operand cannot leak into a later batch.
          const int cols = NT * 8, clr = b.nt * kTileRows * cols;
          for (int e = ctid; e < clr; e += kConsumerWarps * 32) {
            const int m = e / cols, n = e - m * cols;
            if (m >= rows || n >= p.N) rb[m * kRedStride + n] = 0.f;
          }
        }
        redbuf ^= 1;
      }
      // ---- end of phase: publish, then (BLAST) apply the coupling
      if (phs + 1 < p.nphases) {
        __threadfence();
        fence_proxy_async();
        consumer_bar();
        if (ctid == 0) red_release_gpu_add(p.counters + 0, 1u);
        if (p.mix) {
          if (ctid == 0) {
            if (!wait_counter(p.counters + 0, gridDim.x, abort_flag)) ok = false;
          }
          consumer_bar();
          if (!*abort_flag) {
            // z[i][n][r] = sum_j S[i][j][r] * y[j][n][r]; points (n, r) are split evenly over the grid.
            const int NR = p.N * p.R;
            const int lo = (int)(((long long)NR * blockIdx.x) / gridDim.x);
            const int hi = (int)(((long long)NR * (blockIdx.x + 1)) / gridDim.x);
            const int npts = hi - lo, bb = p.b;
            const long long plane = (long long)p.N * p.R;
            const bool i_fast = (p.s_r != 1);  // S stored with the block indices innermost
            for (int e = ctid; e < npts * bb; e += kConsumerWarps * 32) {
              int i, pt;
              if (i_fast) { i = e % bb; pt = e / bb; }
              else { pt = e % npts; i = e / npts; }
              const int nr = lo + pt, r = nr % p.R;
              float s = 0.f;
              for (int j = 0; j < bb; ++j)
                s = fmaf(load16<BF16>(p.S, i * p.s_i + j * p.s_j + r * p.s_r), __ldcg(p.y32 + j * plane + nr), s);
              if (p.round_z) s = round_clamp_i8(s);
              store16<BF16>(p.z16, i * plane + nr, s);
            }
          }
          __threadfence();
          fence_proxy_async();
          consumer_bar();
          if (ctid == 0) red_release_gpu_add(p.counters + 1, 1u);
        }
      }
    }
    // ---- leave: last CTA out re-arms the counters for the next launch on this workspace
    consumer_bar();
    if (ctid == 0 && p.counters != nullptr) {
      if (*abort_flag) {
        atomicExch(p.counters + 3, 1u);
      } else {
        __threadfence();
        const unsigned prev = atomicAdd(p.counters + 2, 1u);
        if (prev == gridDim.x - 1) {
          p.counters[0] = 0u;
          p.counters[1] = 0u;
          p.counters[2] = 0u;
          __threadfence();
        }
      }
    }
  }
  __syncthreads();
  if (*abort_flag) {
    // let tile loads that may still be in flight land before the shared memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
}

// ------------------------------------------------------------------ host launcher
template <bool BF16, int NT>
static int launch_impl(const StreamParams& p, cudaStream_t stream) {
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != BLR_OK) return rc;
  BLR_REQUIRE(di.coop, BLR_ERR_UNSUPPORTED, "device does not support cooperative launch");
  const size_t smem = (size_t)p.nstages * p.stage_bytes + 2 * 128 * kRedStride * sizeof(float) + 2 * 16 * 8 + 64 + 1024;
  BLR_REQUIRE((int)smem <= di.max_smem_optin, BLR_ERR_UNSUPPORTED, "needs %zu bytes of shared memory, device offers %d",
              smem, di.max_smem_optin);
  auto kern = blr_stream_kernel<BF16, NT>;
  int dev;
  BLR_CUDA_OK(cudaGetDevice(&dev));
  static bool configured[64] = {};  // one flag per device for this template instance
  if (!configured[dev & 63]) {
    BLR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem_optin));
    configured[dev & 63] = true;
  }
  void* args[] = {const_cast<StreamParams*>(&p)};
  BLR_CUDA_OK(cudaLaunchCooperativeKernel((const void*)kern, dim3(di.sm_count), dim3(kStreamThreads), args, smem, stream));
  return BLR_OK;
}

int launch_stream(const StreamParams& p, int is_bf16, cudaStream_t stream) {
  BLR_REQUIRE(p.N >= 1 && p.N <= kStreamMaxTokens, BLR_ERR_ARG, "stream kernel handles 1..%d tokens, got %d",
              kStreamMaxTokens, p.N);
  if (p.N <= 8) return is_bf16 ? launch_impl<true, 1>(p, stream) : launch_impl<false, 1>(p, stream);
  return is_bf16 ? launch_impl<true, 2>(p, stream) : launch_impl<false, 2>(p, stream);
}

}  // namespace blr
