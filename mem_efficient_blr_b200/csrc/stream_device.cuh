// Device helpers shared by the weight-streaming kernels: ring position bookkeeping, swizzled shared-memory
// addressing, and the stage consumers that turn one K-chunk of a 16-row weight group into mma.sync products
// (16-bit weights in either layout, int8 and packed int4 widened in registers).
#pragma once
#include "ptx.cuh"
#include "stream.h"

namespace blr {

struct RingPos {
  uint32_t s = 0, use_parity = 0;
  bool first_pass = true;
  __device__ __forceinline__ void advance(uint32_t nst) {
    if (++s == nst) {
      s = 0;
      use_parity ^= 1u;
      first_pass = false;
    }
  }
};

// Byte offset of 16-byte chunk `c16` in row `row` of a 128-byte-swizzled box (rows of 128 B).
__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t c16) { return row * 128u + ((c16 ^ (row & 7u)) << 4); }
// Same for a 64-byte-swizzled box (rows of 64 B).
__device__ __forceinline__ uint32_t sw64(uint32_t row, uint32_t c16) { return row * 64u + ((c16 ^ ((row >> 1) & 3u)) << 4); }

// ------------------------------------------------------------------ stage consumers (one 16-row group per warp)
// Activation fragments of one k16 step from a [tokens][64 k] box.
template <int NT>
__device__ __forceinline__ void load_bfrag(uint32_t sA, int ks, int lane, uint32_t (&bf)[NT][2]) {
  const uint32_t jm = lane >> 3, l7 = lane & 7;
  if constexpr (NT == 2) {
    ldsm_x4(sA + sw128((jm >> 1) * 8 + l7, ks * 2 + (jm & 1)), bf[0][0], bf[0][1], bf[1][0], bf[1][1]);
  } else {
    ldsm_x2(sA + sw128(l7, ks * 2 + (jm & 1)), bf[0][0], bf[0][1]);
  }
}

// 16-bit weights, k contiguous: the stage is one box of rows x 64 k; row0 is this warp's first row.
template <bool BF16, int NT>
__device__ __forceinline__ void consume_k16(uint32_t sWt, uint32_t sA, int row0, float (&acc)[4][NT][4], int lane) {
  const uint32_t jm = lane >> 3, l7 = lane & 7;
  const uint32_t row = row0 + l7 + (jm & 1) * 8;
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    uint32_t bf[NT][2];
    load_bfrag<NT>(sA, ks, lane, bf);
    uint32_t a0, a1, a2, a3;
    ldsm_x4(sWt + sw128(row, ks * 2 + (jm >> 1)), a0, a1, a2, a3);
#pragma unroll
    for (int n = 0; n < NT; ++n) mma_16816<BF16>(acc[ks][n], a0, a1, a2, a3, bf[n][0], bf[n][1]);
  }
}

// 16-bit weights, m contiguous: tile = 64 k-rows x 32 m (64-byte swizzle); fragments via ldmatrix.trans.
template <bool BF16, int NT>
__device__ __forceinline__ void consume_m16(uint32_t sWt, uint32_t sA, int rg, float (&acc)[4][NT][4], int lane) {
  const uint32_t jm = lane >> 3, l7 = lane & 7;
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    uint32_t bf[NT][2];
    load_bfrag<NT>(sA, ks, lane, bf);
    const uint32_t krow = ks * 16 + l7 + (jm >> 1) * 8, c16 = rg * 2 + (jm & 1);
    uint32_t a0, a1, a2, a3;
    ldsm_x4_t(sWt + sw64(krow, c16), a0, a1, a2, a3);
#pragma unroll
    for (int n = 0; n < NT; ++n) mma_16816<BF16>(acc[ks][n], a0, a1, a2, a3, bf[n][0], bf[n][1]);
  }
}

// int8 weights, k contiguous: box of rows x 128 k.  A thread's ldmatrix word holds k = 4t..4t+3 of a
// 16-wide window, so the matching activation fragment is the 8 contiguous bytes at the same k.
// kABox: distance between the two activation boxes of the chunk (a box of NT * 8 token rows by default).
template <bool BF16, int NT>
__device__ __forceinline__ void consume_k8(uint32_t sWt, uint32_t sA, int row0, float (&acc)[4][NT][4], int lane,
                                           const uint32_t kABox = NT * 8 * 128) {
  const uint32_t jm = lane >> 3, l7 = lane & 7, g = lane >> 2, tq = lane & 3;
  const uint32_t row = row0 + l7 + (jm & 1) * 8;
#pragma unroll
  for (int win = 0; win < 4; ++win) {  // 32-byte windows of the 128-byte row
    uint32_t bf[2][NT][2];             // [half window][n-tile][b0,b1]
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const uint32_t c16 = (win & 1) * 4 + h * 2 + (tq >> 1);
        lds64(sA + (win >> 1) * kABox + sw128(n * 8 + g, c16) + (tq & 1) * 8, bf[h][n][0], bf[h][n][1]);
      }
    uint32_t r[4];
    ldsm_x4(sWt + sw128(row, win * 2 + (jm >> 1)), r[0], r[1], r[2], r[3]);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t lo = r[2 * h] ^ 0x80808080u, hi = r[2 * h + 1] ^ 0x80808080u;
      const uint32_t a0 = cvt_u8pair<BF16>(lo, false), a1 = cvt_u8pair<BF16>(hi, false);
      const uint32_t a2 = cvt_u8pair<BF16>(lo, true), a3 = cvt_u8pair<BF16>(hi, true);
#pragma unroll
      for (int n = 0; n < NT; ++n) mma_16816<BF16>(acc[win][n], a0, a1, a2, a3, bf[h][n][0], bf[h][n][1]);
    }
  }
}

// Packed int4 weights, k contiguous: box of rows x 256 k (128 bytes per row).  A thread's ldmatrix word
// holds k = 8t..8t+7 of a 32-wide window as nibbles; nibbles (e, e+4) convert together, so the
// activation pairs are permuted to (k_e, k_{e+4}) with prmt.
// kABox: distance between the four activation boxes of the chunk.
template <bool BF16, int NT>
__device__ __forceinline__ void consume_k4(uint32_t sWt, uint32_t sA, int row0, float (&acc)[4][NT][4], int lane,
                                           const uint32_t kABox = NT * 8 * 128) {
  const uint32_t jm = lane >> 3, l7 = lane & 7, g = lane >> 2, tq = lane & 3;
  const uint32_t row = row0 + l7 + (jm & 1) * 8;
#pragma unroll
  for (int win = 0; win < 4; ++win) {  // 32-byte windows = 64 k = one activation box
    uint32_t bf[2][NT][4];             // [half][n-tile][(k0,k4),(k1,k5),(k2,k6),(k3,k7)]
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        uint32_t q0, q1, q2, q3;
        lds128(sA + win * kABox + sw128(n * 8 + g, h * 4 + tq), q0, q1, q2, q3);
        bf[h][n][0] = prmt(q0, q2, 0x5410u);
        bf[h][n][1] = prmt(q0, q2, 0x7632u);
        bf[h][n][2] = prmt(q1, q3, 0x5410u);
        bf[h][n][3] = prmt(q1, q3, 0x7632u);
      }
    uint32_t r[4];
    ldsm_x4(sWt + sw128(row, win * 2 + (jm >> 1)), r[0], r[1], r[2], r[3]);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t lo = r[h * 2] ^ 0x88888888u, hi = r[h * 2 + 1] ^ 0x88888888u;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const uint32_t a0 = cvt_u4pair<BF16>(lo, 2 * e), a1 = cvt_u4pair<BF16>(hi, 2 * e);
        const uint32_t a2 = cvt_u4pair<BF16>(lo, 2 * e + 1), a3 = cvt_u4pair<BF16>(hi, 2 * e + 1);
#pragma unroll
        for (int n = 0; n < NT; ++n) mma_16816<BF16>(acc[win][n], a0, a1, a2, a3, bf[h][n][2 * e], bf[h][n][2 * e + 1]);
      }
    }
  }
}

// Per-group scales (kScaleGroup contraction indices per scale).  One K-chunk is one group of int8 weights or two
// groups of int4 weights, and the chains acc[0..3] of a chunk are its four 32-byte windows in order, so after a
// chunk the chains are scaled into `tot` and cleared.  A thread holds rows g and g+8 of its warp's row group:
// `srow` points at the scales of row g (nullptr: row past M), `srow8` at those of row g+8; `gidx` is the first
// group of the chunk and `ngroups` the number of groups per row.
struct GroupScales {
  float s[2][2];  // [group of the chunk][row g / row g+8]
};
// Issued before the chunk is consumed, so that the loads are back when fold_scale_groups needs them.
__device__ __forceinline__ GroupScales load_scale_groups(const __half* srow, const __half* srow8, int gidx, int ngroups,
                                                         int wbits) {
  GroupScales r = {{{0.f, 0.f}, {0.f, 0.f}}};
  const int per_chunk = wbits == 8 ? 1 : 2;
#pragma unroll
  for (int q = 0; q < 2; ++q)
    if (q < per_chunk && gidx + q < ngroups) {
      if (srow) r.s[q][0] = __half2float(__ldg(srow + gidx + q));
      if (srow8) r.s[q][1] = __half2float(__ldg(srow8 + gidx + q));
    }
  return r;
}
template <int NT>
__device__ __forceinline__ void fold_scale_groups(float (&acc)[4][NT][4], float (&tot)[NT][4], const GroupScales& gs,
                                                  int wbits) {
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const int q = wbits == 8 ? 0 : (w >> 1);
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        tot[n][e] = fmaf(gs.s[q][e >> 1], acc[w][n][e], tot[n][e]);
        acc[w][n][e] = 0.f;
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
template <bool BF16>
__device__ __forceinline__ float2 unpack16x2(uint32_t w) {
  if constexpr (BF16) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  else return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack16x2(float a, float b) {
  if constexpr (BF16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  } else {
    const __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}
__device__ __forceinline__ float round_clamp_i8(float v) { return fminf(fmaxf(rintf(v), -128.f), 127.f); }
__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory"); }

}  // namespace blr
