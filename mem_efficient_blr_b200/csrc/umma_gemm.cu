// tcgen05 / TMEM grouped GEMM (sm_100a).  Persistent, one CTA per SM, warp-specialised:
//   warp 0    TMA producer: per stage one 128-row tile (16 KB) of the MMA's row operand and one tile of up to
//             256 rows of its column operand, both 64 k wide, 128-byte swizzled
//   warp 1    MMA issuer: one elected thread issues tcgen05.mma (M = 128, N = bn, K = 16) from shared-memory
//             descriptors; accumulators are double-buffered in TMEM (2 x bn columns of fp32)
//   warps 2-9 epilogue: tcgen05.ld the accumulator (one MMA row per thread, two warps per 32 rows taking
//             alternate 64-column chunks, loads of the next chunk in flight), convert, store
// Which operand the tokens are is a template parameter (see umma_gemm.h).
// Quantised weights (WQ = 8 | 4) add
//   warps 10-17 converter: the producer stages the stored bytes of the weight tile next to the operand tiles; these
//             warps widen them (q * scale, rounded once to the 16-bit dtype) into the swizzled weight tile of the
//             stage and release it to the MMA issuer, so the quantised factors are the only copy in global memory
// All waits are bounded; a time-out sets *status and the kernel drains and frees its TMEM.
#include <stdlib.h>

#include "ptx.cuh"
#include "tmap.h"
#include "umma_gemm.h"

namespace blr {

static constexpr int kGemmThreads = 320;
static constexpr int kBM = 128;  // rows of the MMA (TMEM lanes)
static constexpr int kBK = 64;
static constexpr int kRowTileBytes = kBM * kBK * 2;
static constexpr int kMaxStages = 8;
static constexpr int kConvWarps = 8;  // converter warps of the quantised-weight variants

// Bytes k0 and k0 + 1 of `w` hold u = q + OFF: returns (q * s) for both as two values of the 16-bit dtype, the
// product rounded once (q and the fp16 scale are exact in either arithmetic: the result equals rn(float(q) * float(s))).
template <bool BF16, int OFF, int K0>
__device__ __forceinline__ uint32_t widen2(uint32_t w, float sf, __half2 sh) {
  if constexpr (BF16) {
    // 0x4B0000uu = 2^23 + u as a float
    const float a = __uint_as_float(prmt(w, 0x4B000000u, 0x7650u | K0)) - (8388608.f + OFF);
    const float b = __uint_as_float(prmt(w, 0x4B000000u, 0x7650u | (K0 + 1))) - (8388608.f + OFF);
    const __nv_bfloat162 v = __floats2bfloat162_rn(a * sf, b * sf);
    return *reinterpret_cast<const uint32_t*>(&v);
  } else {
    // 0x64uu = 1024 + u as a half
    const uint32_t m = prmt(w, 0x64646464u, K0 == 0 ? 0x4140u : 0x4342u);
    const __half2 off = __floats2half2_rn(1024.f + OFF, 1024.f + OFF);
    const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&m), off), sh);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}

// 16 consecutive quantised weights at `raw` (shared memory) -> 32 bytes of the 16-bit dtype in o[0..7]
template <bool BF16, int WQ>
__device__ __forceinline__ void widen16(uint32_t raw, __half scale, uint32_t (&o)[8]) {
  uint32_t bw[4];
  constexpr int OFF = WQ == 8 ? 128 : 8;
  if constexpr (WQ == 8) {
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(bw[0]), "=r"(bw[1]), "=r"(bw[2]), "=r"(bw[3]) : "r"(raw));
#pragma unroll
    for (int i = 0; i < 4; ++i) bw[i] ^= 0x80808080u;
  } else {
    uint32_t w[2];
    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(raw));
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint32_t lo = (w[i] & 0x0F0F0F0Fu) ^ 0x08080808u, hi = ((w[i] >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
      bw[2 * i] = prmt(lo, hi, 0x5140u);      // weights 0..3 of the word: (low, high) nibbles of bytes 0, 1
      bw[2 * i + 1] = prmt(lo, hi, 0x7362u);  // weights 4..7
    }
  }
  const float sf = __half2float(scale);
  const __half2 sh = __half2half2(scale);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = widen2<BF16, OFF, 0>(bw[i], sf, sh);
    o[2 * i + 1] = widen2<BF16, OFF, 2>(bw[i], sf, sh);
  }
}

template <bool BF16>
__device__ __forceinline__ void gemm_store(void* base, long long off, float v) {
  if constexpr (BF16) reinterpret_cast<__nv_bfloat16*>(base)[off] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(base)[off] = __float2half_rn(v);
}
template <bool BF16>
__device__ __forceinline__ uint32_t gemm_pack(float a, float b) {
  if constexpr (BF16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  } else {
    const __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}
template <bool RND>
__device__ __forceinline__ float gemm_round(float v) {
  if constexpr (RND) return fminf(fmaxf(rintf(v), -128.f), 127.f);
  else return v;
}

template <bool BF16>
__device__ __forceinline__ float2 gemm_unpack(uint32_t w) {
  if constexpr (BF16) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  else return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <bool BF16>
__device__ __forceinline__ float gemm_load(const uint16_t* p) {
  if constexpr (BF16) return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p));
  else return __half2float(*reinterpret_cast<const __half*>(p));
}

__device__ __forceinline__ float gemm_act(float v, int act) {
  if (act == 1) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
  if (act == 2) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * fmaf(0.044715f * v, v * v, v)));
    return 0.5f * v * (1.f + t);
  }
  return v;
}

// Epilogue of one tile when tokens are the MMA rows: this thread's token, its columns = consecutive weight rows.
struct EpiRow {
  int act;
  const uint16_t* bias;  // at the group's first feature, or null
  const uint16_t* res;   // the token's residual row at the group's first feature, or null
  int extra_vec;
  void* out;
  long long nbase, os_hi, os_lo;  // element offset of the token; strides of (m / per) and (m % per)
  int per, M, m0, cend;           // first weight row of the tile, columns of the tile that exist
  bool n_ok;                      // token exists
};

// MODE 2: 32-byte stores (16 consecutive outputs contiguous and aligned, no ragged tile edge), 1: 16-byte stores,
// 0: element stores.  The mode is a template parameter so that a chunk executes only its own variant.
template <bool BF16, bool RND, int MODE, bool EX>
__device__ __forceinline__ void epilogue_store32(const EpiRow& e, int c0, uint32_t (&rr)[2][16]) {
  int hi = (e.m0 + c0) / e.per, lo = (e.m0 + c0) - hi * e.per;  // (m / per, m % per), kept incrementally
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int c = c0 + 16 * u;
    if (c >= e.cend) break;
    uint32_t(&r)[16] = rr[u];
    tmem_regs_ready(r);
    if constexpr (EX) {
      // bias and residual of features m0 + c .. + 15 (16-byte pieces where the host found them aligned)
      const int m = e.m0 + c;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        const uint16_t* src = part == 0 ? e.bias : e.res;
        if (part == 1 && e.act != 0) {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(gemm_act(__uint_as_float(r[j]), e.act));
        }
        if (src == nullptr || (part == 1 && !e.n_ok)) continue;
        if (e.extra_vec && m + 16 <= e.M) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint4 v = *reinterpret_cast<const uint4*>(src + m + 8 * h);
            const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 f = gemm_unpack<BF16>(ws[k]);
              r[8 * h + 2 * k] = __float_as_uint(__uint_as_float(r[8 * h + 2 * k]) + f.x);
              r[8 * h + 2 * k + 1] = __float_as_uint(__uint_as_float(r[8 * h + 2 * k + 1]) + f.y);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (m + j < e.M) r[j] = __float_as_uint(__uint_as_float(r[j]) + gemm_load<BF16>(src + m + j));
        }
      }
    }
    if constexpr (MODE > 0) {
      uint32_t w[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        w[k] = gemm_pack<BF16>(gemm_round<RND>(__uint_as_float(r[2 * k])), gemm_round<RND>(__uint_as_float(r[2 * k + 1])));
      uint16_t* o16 = reinterpret_cast<uint16_t*>(e.out);
      if constexpr (MODE == 2) {
        // one full 32-byte sector per thread
        uint16_t* dst = o16 + e.nbase + (long long)hi * e.os_hi + lo;
        if (e.n_ok)
          asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                       "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
        lo += 16;
        if (lo >= e.per) { lo -= e.per; ++hi; }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (e.n_ok && e.m0 + c + 8 * h < e.M)
            *reinterpret_cast<uint4*>(o16 + e.nbase + (long long)hi * e.os_hi + lo) = make_uint4(w[4 * h], w[4 * h + 1], w[4 * h + 2], w[4 * h + 3]);
          lo += 8;
          if (lo >= e.per) { lo -= e.per; ++hi; }
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (e.n_ok && e.m0 + c + j < e.M)
          gemm_store<BF16>(e.out, e.nbase + (long long)hi * e.os_hi + (long long)lo * e.os_lo, gemm_round<RND>(__uint_as_float(r[j])));
        if (++lo == e.per) { lo = 0; ++hi; }
      }
    }
  }
}

__device__ __forceinline__ void epilogue_load32(uint32_t taddr, uint32_t (&rr)[2][16]) {
#pragma unroll
  for (int u = 0; u < 2; ++u) tmem_ld16(taddr + 16 * u, rr[u]);
}

// Columns c_first, c_first + 64, ... of the tile, 32 per round; the loads of the next round are in flight while
// this one is converted and stored.  (A round always loads 32 columns: the allocation has room behind the last
// tile column.)
template <bool BF16, bool RND, int MODE, bool EX>
__device__ __forceinline__ void epilogue_rows(const EpiRow& e, uint32_t taddr, int c_first) {
  uint32_t ra[2][16], rb[2][16];
  int c0 = c_first;
  if (c0 < e.cend) epilogue_load32(taddr + c0, ra);
  while (c0 < e.cend) {
    tmem_ld_wait();
    if (c0 + 64 < e.cend) epilogue_load32(taddr + c0 + 64, rb);
    epilogue_store32<BF16, RND, MODE, EX>(e, c0, ra);
    c0 += 64;
    if (c0 >= e.cend) break;
    tmem_ld_wait();
    if (c0 + 64 < e.cend) epilogue_load32(taddr + c0 + 64, ra);
    epilogue_store32<BF16, RND, MODE, EX>(e, c0, rb);
    c0 += 64;
  }
}

// TR = tokens are the MMA rows (weights its columns); !TR = weights are the rows ("swap-AB").
// MODE = store width of the TR epilogue (see epilogue_store32), RND = round the outputs to int8 steps; both are
// chosen by the host from the parameters, so that the epilogue holds exactly one variant.
// WQ = 0: 16-bit weights; 8 | 4: quantised weights widened by converter warps (K-major only).
// EX: the epilogue adds a bias and / or a residual (an instance of its own: the additions cost registers).
template <bool BF16, bool TR, int MODE, bool RND, int WQ, bool EX>
__global__ void __launch_bounds__(kGemmThreads + (WQ ? 32 * kConvWarps : 0), 1)
    blr_umma_gemm_kernel(const __grid_constant__ GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t col_tile_bytes = (uint32_t)p.bn * kBK * 2;
  const uint32_t tiles_bytes = kRowTileBytes + col_tile_bytes;  // the two operand tiles of a stage
  // quantised weights: the stored bytes of the weight tile follow them (8 * WQ bytes per row)
  const uint32_t raw_bytes = WQ ? (uint32_t)(TR ? p.bn : kBM) * (8u * WQ) : 0u;
  const uint32_t stage_bytes = tiles_bytes + raw_bytes;
  const uint32_t NST = p.nstages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)NST * stage_bytes);
  // full[8], empty[8], tmem_full[2], tmem_empty[2], (slot, abort flag), raw_full[8]
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kMaxStages);
  const uint32_t tfull0 = smem_u32(bars + 2 * kMaxStages), tempty0 = smem_u32(bars + 2 * kMaxStages + 2);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t rfull0 = smem_u32(bars + 2 * kMaxStages + 5);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // m_tiles: tiles along the weight rows; n_tiles: tiles along the tokens
  const int m_tiles = TR ? (p.M + p.bn - 1) / p.bn : (p.M + kBM - 1) / kBM;
  const int n_tiles = TR ? (p.N + kBM - 1) / kBM : (p.N + p.bn - 1) / p.bn;
  const int tiles = p.G * m_tiles * n_tiles;
  const int kblocks = (p.K + kBK - 1) / kBK;
  const int w_rows = TR ? p.bn : kBM;    // weight rows per tile
  const int a_rows = TR ? kBM : p.bn;    // tokens per tile
  // byte offsets of the two operands inside a stage
  const uint32_t w_off = TR ? kRowTileBytes : 0u, a_off = TR ? 0u : kRowTileBytes;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (uint32_t s = 0; s < NST; ++s) {
      mbar_init(full0 + 8 * s, WQ ? 1 + kConvWarps : 1);  // the producer's arrival (+ one per converter warp)
      mbar_init(empty0 + 8 * s, 1);
      if constexpr (WQ != 0) mbar_init(rfull0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull0 + 8 * b, 1);
      mbar_init(tempty0 + 8 * b, 8);  // one arrival per epilogue warp
    }
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch: everything above overlaps the tail of the previous kernel in the stream; its
  // results (this kernel's activations) and the buffers it may still be reading (this kernel's output) are
  // touched only after it has completed.  Every thread waits, so this grid completes after its predecessor.
  asm volatile("griddepcontrol.wait;" ::: "memory");

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
          if constexpr (WQ != 0) {
            // stored bytes to the converter warps; only the token tile completes `bar` by bytes
            mbar_arrive_expect_tx(rfull0 + 8 * s, raw_bytes);
            tma_load_3d(dst + tiles_bytes, &p.tmW, kb * (8 * WQ), mt * w_rows, g, rfull0 + 8 * s);
            mbar_arrive_expect_tx(bar, TR ? (uint32_t)kRowTileBytes : col_tile_bytes);
          } else if (p.kmajor) {
            mbar_arrive_expect_tx(bar, stage_bytes);
            tma_load_3d(dst + w_off, &p.tmW, kb * kBK, mt * w_rows, g, bar);
          } else {
            mbar_arrive_expect_tx(bar, stage_bytes);
            // output index contiguous: 64-wide column blocks of 64 k-rows, 8 KB each
            for (int blk = 0; blk < w_rows / 64; ++blk)
              tma_load_3d(dst + w_off + blk * 8192, &p.tmW, mt * w_rows + blk * 64, kb * kBK, g, bar);
          }
          tma_load_3d(dst + a_off, &p.tmA, kb * kBK, nt * a_rows, g, bar);
          if (++s == NST) { s = 0; parity ^= 1u; first = false; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = TR ? umma_idesc(BF16, false, !p.kmajor, kBM, (uint32_t)p.bn)
                                : umma_idesc(BF16, !p.kmajor, false, kBM, (uint32_t)p.bn);
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
          const uint32_t st = smem_base + s * stage_bytes, sW = st + w_off, sA = st + a_off;
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            // weights: K-major tile advances 32 B per k16 inside the swizzle atom; M-major tile advances 16 k-rows
            const uint64_t wdesc = p.kmajor ? umma_smem_desc(sW + kk * 32, 16, 1024) : umma_smem_desc(sW + kk * 2048, 8192, 1024);
            const uint64_t adesc = umma_smem_desc(sA + kk * 32, 16, 1024);
            if constexpr (TR) umma_f16(d_tmem, adesc, wdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
            else umma_f16(d_tmem, wdesc, adesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * s);  // frees the stage once these MMAs have read it
          if (++s == NST) { s = 0; parity ^= 1u; }
        }
        if (ok) umma_commit(tfull0 + 8 * buf);  // accumulator complete
      }
    }
  } else if (WQ != 0 && warp >= kGemmThreads / 32) {
    // ------------------------------------------------ converter: thread = (row of a band of rows, 16 weights of the
    // 64-wide k block); a warp reads 8 rows of stored bytes contiguously and writes their 16-byte pieces to the
    // places the 128-byte swizzle gives them (piece c of row r at c ^ (r & 7)): no bank conflicts either way
    if constexpr (WQ != 0) {
      const int ct = (int)threadIdx.x - kGemmThreads, j = ct & 3, r_in = ct >> 2;
      const __half* sc = static_cast<const __half*>(p.w_scale);
      constexpr int kBand = 8 * kConvWarps, kMaxBands = 256 / kBand;  // rows per pass of all converter threads
      const int bands = w_rows / kBand;
      const bool grouped = p.scales_per_row > 1;
      __half scale[kMaxBands];
      uint32_t s = 0, parity = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int gm = tile / n_tiles, mt = gm % m_tiles, g = gm / m_tiles;
        const int row0 = mt * w_rows;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (kb == 0 || (grouped && (kb & 1) == 0)) {
#pragma unroll
            for (int i = 0; i < kMaxBands; ++i) {
              const int m = row0 + r_in + kBand * i;
              scale[i] = i < bands && m < p.M ? sc[((long long)g * p.M + m) * p.scales_per_row + (grouped ? kb >> 1 : 0)]
                                              : __float2half(0.f);
            }
          }
          if (!mbar_wait(rfull0 + 8 * s, parity, abort_flag)) { ok = false; break; }
          const uint32_t st = smem_base + s * stage_bytes, raw = st + tiles_bytes, dstW = st + w_off;
#pragma unroll
          for (int i = 0; i < kMaxBands; ++i) {
            if (i < bands) {
              const int row = r_in + kBand * i;
              uint32_t o[8];
              widen16<BF16, WQ>(raw + row * (8 * WQ) + j * (2 * WQ), scale[i], o);
              const uint32_t d = dstW + row * 128, x = (uint32_t)(row & 7);
              asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(d + (((2 * j) ^ x) << 4)), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
              asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(d + (((2 * j + 1) ^ x) << 4)), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
            }
          }
          fence_proxy_async_smem();  // the MMA reads the tile through the async proxy
          __syncwarp();
          if (lane == 0) mbar_arrive(full0 + 8 * s);
          if (++s == NST) { s = 0; parity ^= 1u; }
        }
      }
    }
  } else {
    // ------------------------------------------------ epilogue: warp w reads TMEM lanes 32*(w%4)..+31; the two
    // warps of a lane quarter take alternate column chunks of the accumulator
    const int q = warp & 3, half = (warp - 2) >> 2;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
      const int nt = tile % n_tiles, gm = tile / n_tiles, mt = gm % m_tiles, g = gm / m_tiles;
      const uint32_t buf = it & 1u, use = it >> 1;
      if (ok && !mbar_wait(tfull0 + 8 * buf, use & 1u, abort_flag)) ok = false;
      if (!ok) continue;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * (uint32_t)p.bn;
      const long long gbase = (long long)g * p.os_g;
      if constexpr (TR) {
        EpiRow e;
        e.out = p.out;
        const int n = nt * kBM + q * 32 + lane;
        e.n_ok = n < p.N;
        e.extra_vec = p.extra_vec;
        e.act = p.act_out;
        e.bias = p.bias ? static_cast<const uint16_t*>(p.bias) + (long long)g * p.M : nullptr;
        e.res = p.residual && e.n_ok ? static_cast<const uint16_t*>(p.residual) + (long long)n * p.ldr + (long long)g * p.M : nullptr;
        e.nbase = gbase + (long long)n * p.os_n;
        e.os_hi = p.os_hi, e.os_lo = p.os_lo, e.per = p.per, e.M = p.M, e.m0 = mt * p.bn;
        e.cend = min(p.bn, p.M - e.m0);
        epilogue_rows<BF16, RND, MODE, EX>(e, taddr, 32 * half);
      } else {
        // thread = weight row, columns = tokens
        const int m = mt * kBM + q * 32 + lane;
        const bool m_ok = m < p.M;
        const long long base = m_ok ? gbase + (long long)(m / p.per) * p.os_hi + (long long)(m % p.per) * p.os_lo : 0;
        const int n0 = nt * p.bn;
        float bias_m = 0.f;
        const uint16_t* res_m = nullptr;
        if constexpr (EX) {
          if (p.bias && m_ok) bias_m = gemm_load<BF16>(static_cast<const uint16_t*>(p.bias) + (long long)g * p.M + m);
          if (p.residual && m_ok) res_m = static_cast<const uint16_t*>(p.residual) + (long long)g * p.M + m;
        }
        for (int c = 16 * half; c < p.bn; c += 32) {
          if (n0 + c >= p.N) break;  // whole chunk past the last token (warp-uniform)
          uint32_t r[16];
          tmem_ld16(taddr + c, r);
          tmem_ld_wait();
          tmem_regs_ready(r);
          if (m_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int n = n0 + c + j;
              if (n < p.N) {
                float v = __uint_as_float(r[j]);
                if constexpr (EX) {
                  v = gemm_act(v + bias_m, p.act_out);
                  if (res_m != nullptr) v += gemm_load<BF16>(res_m + (long long)n * p.ldr);
                }
                gemm_store<BF16>(p.out, base + (long long)n * p.os_n, gemm_round<RND>(v));
              }
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

static bool gemm_quantised(const GemmParams& p) { return p.w_bits == 8 || p.w_bits == 4; }
static int gemm_stage_bytes(const GemmParams& p) {
  const int w_rows = p.tokens_as_rows ? p.bn : kBM;
  return kRowTileBytes + p.bn * kBK * 2 + (gemm_quantised(p) ? w_rows * 8 * p.w_bits : 0);
}

void umma_gemm_tiling(GemmParams& p) {
  if (p.N > 64) {
    // tokens as MMA rows; weight rows as columns, 256 at a time when the block is tall enough
    p.tokens_as_rows = 1;
    int bn = 256;
    if (p.M <= 192) bn = (p.M + 63) / 64 * 64;  // multiples of 64 keep the M-major boxes whole
    // few token tiles: narrower weight tiles until there is about one tile per SM (a 128 x 256 tile of a short
    // contraction is over in a microsecond; half of the SMs idle costs more than the smaller MMA shape)
    const long long n_tiles = (p.N + kBM - 1) / kBM;
    // (long contractions keep the wide tile: there the loads per flop decide, and they grow as the tile narrows)
    while (p.K <= 512 && bn % 128 == 0 && (long long)p.G * ((p.M + bn - 1) / bn) * n_tiles < 132) bn /= 2;  // 256 -> 128 -> 64
    // long contraction: narrower only while the tiles still fit one wave (then a narrower tile is a shorter wave)
    while (p.K > 512 && bn % 128 == 0 && (long long)p.G * ((p.M + bn / 2 - 1) / (bn / 2)) * n_tiles <= 148) bn /= 2;
    p.bn = bn;
  } else {
    p.tokens_as_rows = 0;
    p.bn = (p.N + 15) / 16 * 16;
  }
  const int stage = gemm_stage_bytes(p);
  int nst = (232448 - 1024 - 512) / stage;
  p.nstages = nst > kMaxStages ? kMaxStages : nst;
}

template <bool BF16, bool TR, int MODE, bool RND, int WQ = 0, bool EX = false>
static int launch_variant(const GemmParams& p, int grid, size_t smem, int dev, int max_smem, cudaStream_t stream) {
  static bool configured[64] = {};
  if (!configured[dev & 63]) {
    BLR_CUDA_OK(cudaFuncSetAttribute(blr_umma_gemm_kernel<BF16, TR, MODE, RND, WQ, EX>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
    configured[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kGemmThreads + (WQ ? 32 * kConvWarps : 0));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  void* args[] = {const_cast<GemmParams*>(&p)};
  BLR_CUDA_OK(cudaLaunchKernelExC(&cfg, (const void*)blr_umma_gemm_kernel<BF16, TR, MODE, RND, WQ, EX>, args));
  return BLR_OK;
}

// No rounding variant with quantised weights or with additions in the epilogue (the rounded intermediates exist for
// 16-bit factors only, and they are never a layer's final result).
template <bool BF16, int WQ, bool EX>
static int launch_plain(const GemmParams& p, int mode, int grid, size_t smem, int dev, int max_smem, cudaStream_t stream) {
  if (!p.tokens_as_rows) return launch_variant<BF16, false, 0, false, WQ, EX>(p, grid, smem, dev, max_smem, stream);
  if (mode == 2) return launch_variant<BF16, true, 2, false, WQ, EX>(p, grid, smem, dev, max_smem, stream);
  if (mode == 1) return launch_variant<BF16, true, 1, false, WQ, EX>(p, grid, smem, dev, max_smem, stream);
  return launch_variant<BF16, true, 0, false, WQ, EX>(p, grid, smem, dev, max_smem, stream);
}
template <bool BF16, int WQ>
static int launch_quantised(const GemmParams& p, int mode, int grid, size_t smem, int dev, int max_smem, cudaStream_t stream) {
  return (p.bias || p.residual || p.act_out) ? launch_plain<BF16, WQ, true>(p, mode, grid, smem, dev, max_smem, stream)
                                : launch_plain<BF16, WQ, false>(p, mode, grid, smem, dev, max_smem, stream);
}

template <bool BF16>
static int launch_dtype(const GemmParams& p, int mode, int grid, size_t smem, int dev, int max_smem, cudaStream_t stream) {
  if (p.w_bits == 8) return launch_quantised<BF16, 8>(p, mode, grid, smem, dev, max_smem, stream);
  if (p.w_bits == 4) return launch_quantised<BF16, 4>(p, mode, grid, smem, dev, max_smem, stream);
  if (p.bias || p.residual || p.act_out) {
    BLR_REQUIRE(!p.round_out, BLR_ERR_ARG, "bias and residual are not combined with rounded outputs");
    return launch_plain<BF16, 0, true>(p, mode, grid, smem, dev, max_smem, stream);
  }
  if (!p.tokens_as_rows) {
    return p.round_out ? launch_variant<BF16, false, 0, true>(p, grid, smem, dev, max_smem, stream)
                       : launch_variant<BF16, false, 0, false>(p, grid, smem, dev, max_smem, stream);
  }
  if (p.round_out) {
    if (mode == 2) return launch_variant<BF16, true, 2, true>(p, grid, smem, dev, max_smem, stream);
    if (mode == 1) return launch_variant<BF16, true, 1, true>(p, grid, smem, dev, max_smem, stream);
    return launch_variant<BF16, true, 0, true>(p, grid, smem, dev, max_smem, stream);
  }
  if (mode == 2) return launch_variant<BF16, true, 2, false>(p, grid, smem, dev, max_smem, stream);
  if (mode == 1) return launch_variant<BF16, true, 1, false>(p, grid, smem, dev, max_smem, stream);
  return launch_variant<BF16, true, 0, false>(p, grid, smem, dev, max_smem, stream);
}

int launch_umma_gemm(const GemmParams& p_in, cudaStream_t stream) {
  GemmParams p = p_in;
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != BLR_OK) return rc;
  const size_t smem = (size_t)p.nstages * gemm_stage_bytes(p) + 512 + 1024;
  if (gemm_quantised(p)) {
    BLR_REQUIRE(p.kmajor && !p.round_out && p.w_scale != nullptr && p.scales_per_row >= 1, BLR_ERR_ARG,
                "quantised weights are contraction-contiguous, scaled and not combined with rounded outputs");
    BLR_REQUIRE((p.tokens_as_rows ? p.bn : kBM) % (8 * kConvWarps) == 0, BLR_ERR_ARG, "bad tile configuration for quantised weights");
    BLR_REQUIRE(p.scales_per_row == 1 || p.scales_per_row * 128 == p.K, BLR_ERR_SHAPE,
                "scales per weight row: one, or one per 128 contraction indices");
  }
  BLR_REQUIRE((int)smem <= di.max_smem_optin, BLR_ERR_UNSUPPORTED, "needs %zu bytes of shared memory, device offers %d",
              smem, di.max_smem_optin);
  BLR_REQUIRE(p.bn % 16 == 0 && p.bn >= 16 && p.bn <= 256 && p.nstages >= 2, BLR_ERR_ARG, "bad tile configuration");
  BLR_REQUIRE(p.kmajor || !p.tokens_as_rows || p.bn % 64 == 0, BLR_ERR_ARG, "bad tile configuration for this weight layout");
  int dev;
  BLR_CUDA_OK(cudaGetDevice(&dev));
  const int m_tiles = p.tokens_as_rows ? (p.M + p.bn - 1) / p.bn : (p.M + kBM - 1) / kBM;
  const int n_tiles = p.tokens_as_rows ? (p.N + kBM - 1) / kBM : (p.N + p.bn - 1) / p.bn;
  const long long tiles = (long long)p.G * m_tiles * n_tiles;
  const int grid = (int)(tiles < di.sm_count ? tiles : di.sm_count);
  // store width of the epilogue when tokens are the MMA rows: 16-byte stores need 8 consecutive outputs contiguous
  // and aligned in memory; 32-byte stores 16 of them, 32-byte aligned, and no ragged tile edge
  const bool vec_out = p.os_lo == 1 && (p.per & 7) == 0 && (p.M & 7) == 0 && (p.os_g & 7) == 0 && (p.os_n & 7) == 0 &&
                       (p.os_hi & 7) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
  const bool wide_out = vec_out && (p.per & 15) == 0 && (p.M & 15) == 0 && (p.os_g & 15) == 0 && (p.os_n & 15) == 0 &&
                        (p.os_hi & 15) == 0 && (p.bn & 15) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 31) == 0;
  const int mode = wide_out ? 2 : vec_out ? 1 : 0;
  return p.is_bf16 ? launch_dtype<true>(p, mode, grid, smem, dev, di.max_smem_optin, stream)
                   : launch_dtype<false>(p, mode, grid, smem, dev, di.max_smem_optin, stream);
}

}  // namespace blr
