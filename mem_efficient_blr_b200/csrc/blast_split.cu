// BLAST on 1..16 tokens as two dependent launches (see blast_split.h for the decomposition).
//
// Weights sit in shared memory as 128-byte-swizzled boxes of rows x 128 B written by TMA (the layout of the other
// weight-streaming kernels).  What happens to them depends on their width:
//
//   16-bit factors   mma.sync m16n8k16 on 16-bit activations, which are staged as boxes of [token][64 k] with
//                    128-byte rows swizzled by token; a box holds exactly N token rows (fragment loads of rows N..
//                    run into the next box: those rows only feed output columns that are dropped).
//   int8 / int4      integer mma.sync m16n8k32 straight on the stored bytes - no widening instruction per weight,
//                    which is what bounds a conversion-based path once everything is in shared memory.  The
//                    activations of a token row are turned into 16-bit fixed point, q = rint(a / s) with
//                    s = max|a| / 32512, and split into two signed bytes
//                    (q = 256 hi + lo, lo in [-128, 127]); sum_k w_k a_k = s (256 sum_k w_k hi_k + sum_k w_k lo_k) with exact integer
//                    sums, and the weight scales apply to the result.  The rounding of a to 16 bits of the row
//                    maximum is finer in norm than the 11-bit mantissa the activations arrive with.
//
// After the wait on the kernel ahead everything is in shared memory and the time goes to latencies, not bandwidth:
// sixteen consumer warps per CTA keep independent work in flight.  Registers are capped (launch bounds) so that a
// front CTA and a back CTA of neighbouring launches fit one SM together - that is what lets a launch fetch its
// weights while the launch before it computes.
#include "blast_split.h"

#include <stdlib.h>

#include "ptx.cuh"
#include "stream_device.cuh"
#include "tmap.h"

namespace blr {

// Profiling builds (-DBLR_TIMELINE) record %globaltimer stamps per CTA: 16 slots per CTA, 256 CTAs per launch,
// launches numbered by the host in order.  Off in the shipped library.
#ifdef BLR_TIMELINE
unsigned long long* g_split_timeline = nullptr;
int g_split_timeline_launches = 0, g_split_timeline_next = 0;
#define BLR_TL(slot)                                                                                              \
  do {                                                                                                            \
    if (p.timeline && threadIdx.x == 0 && blockIdx.x < 256) p.timeline[(size_t)blockIdx.x * 16 + (slot)] = globaltimer_ns(); \
  } while (0)
#define BLR_TLV(slot, val)                                                                                        \
  do {                                                                                                            \
    if (p.timeline && blockIdx.x < 256) p.timeline[(size_t)blockIdx.x * 16 + (slot)] = (unsigned long long)(val);  \
  } while (0)
#else
#define BLR_TL(slot) do { } while (0)
#define BLR_TLV(slot, val) do { } while (0)
#endif

static constexpr int kW = kSplitWarps;  // consumer warps per CTA

// ---------------------------------------------------------------------------------------------------- shared-memory maps
struct FrontLayout {
  uint32_t w, xs, sx, s, vs, ypart, ybuf, bar, total;
};
struct BackLayout {
  uint32_t ring, zs, sz, part, us, bars, total;
};
__host__ __device__ static inline uint32_t up16(uint32_t v) { return (v + 15u) & ~15u; }
// Warps that share one accumulation (an in-block of the front kernel, a 16-row group of the back kernel) when a CTA
// has fewer of those than warps: each takes every share-th chunk of the contraction.
__host__ __device__ static inline int split_share(int units) { return units >= kW ? 1 : kW / units; }
// Bytes of one token row of fixed-point activations over K contraction indices (2 bytes per index), padded so
// that the 16-byte fragment loads of neighbouring token rows fall into different banks.
__host__ __device__ static inline uint32_t fx_pitch(int K, int wbits) {
  const uint32_t body = wbits == 8 ? ((uint32_t)(K + 31) / 32) * 64 : ((uint32_t)(K + 63) / 64) * 128;
  return ((body + 127u) & ~127u) + (wbits == 8 ? 64u : 16u);
}

__host__ __device__ static inline FrontLayout front_layout(const SplitParams& p) {
  const uint32_t np = p.N <= 8 ? 8 : 16;
  const uint32_t abox = 16 / p.wbits, nbx = p.nch0 * abox, sl = split_share(p.b);
  FrontLayout L;
  uint32_t o = 0;
  L.w = o; o += (uint32_t)p.nch0 * p.b * 1024 + 1024;   // [chunk][in-block][8 rows][128 B] + one slab of slack
  L.xs = o;                                             // activations of every (in-block, token) row
  if (p.wbits == 16) o += (uint32_t)p.b * nbx * p.N * 128 + 2048;  // [in-block][box][token][128 B] + slack for rows N..15
  else o += (uint32_t)p.b * p.N * fx_pitch(p.P, p.wbits);          // [in-block][token][fixed-point row]
  L.sx = o; o += up16((uint32_t)p.b * p.N * 4);           // fixed-point scale of every (in-block, token) row
  L.s = o; o += up16((uint32_t)p.bo * (p.b * 16 + 16));   // [out-block][in-block][8 ranks] 16-bit, padded rows
  L.vs = o; o += (uint32_t)p.b * 8 * 4;                   // per-channel scales of the slice's rows
  L.ypart = o; o += sl > 1 ? (uint32_t)p.b * sl * 8 * np * 4 : 0u;  // [in-block][sharing warp][8 ranks][np tokens] fp32
  L.ybuf = o; o += (uint32_t)p.b * p.N * 8 * 4;           // [in-block][token][8 ranks] fp32
  L.bar = o; o += 32;                                     // barrier of the weights, abort flag, barrier of the bulk copy of x
  L.total = o + 1024;  // room to align the base to 1 KiB
  return L;
}

__host__ __device__ static inline BackLayout back_layout(const SplitParams& p) {
  const uint32_t np = p.N <= 8 ? 8 : 16;
  const uint32_t abox = 16 / p.wbits, nbz = p.nch1 * abox, sl = split_share(p.gpc);
  BackLayout L;
  uint32_t o = 0;
  L.ring = o; o += (uint32_t)p.nstages * kSplitStageBytes;
  L.zs = o;
  if (p.wbits == 16) o += nbz * p.N * 128 + 2048;         // [box][token][128 B] + slack
  else o += (uint32_t)p.N * fx_pitch(p.R, p.wbits);       // [token][fixed-point row]
  L.sz = o; o += 32 * 4;                                  // fixed-point scale per token, then per-warp maxima
  L.part = o; o += (uint32_t)p.gpc * sl * 16 * np * 4;    // [group][sharing warp][np tokens][16 rows] fp32
  L.us = o; o += (uint32_t)p.gpc * 16 * 4;                // per-channel scales of the CTA's rows
  L.bars = o; o += (2 * (uint32_t)p.nstages + 2) * 8;
  L.total = o + 1024;
  return L;
}

size_t split_fx_row_bytes(int K, int wbits) { return fx_pitch(K, wbits); }
size_t split_front_smem(const SplitParams& p) { return front_layout(p).total; }
size_t split_back_smem(const SplitParams& p) { return back_layout(p).total; }

// ---------------------------------------------------------------------------------------------------- small helpers
__device__ __forceinline__ void cp_async16_zfill(uint32_t smem_dst, const void* gsrc, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void named_bar(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ uint4 ld_global_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
// D (s32) += A (s8, 16 x 32) * B (s8, 32 x 8).
__device__ __forceinline__ void imma_s8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}


// ---------------------------------------------------------------------------------------------------- fixed-point activations
// Byte position, inside a token row, of the first of the 8 consecutive contraction indices k0 .. k0+7 (k0 a multiple
// of 8), and how the 8 values spread over 32-bit words.  The order inside a row is the order in which the integer
// MMA's B fragment wants them, so that a thread fetches a step's fragments of both planes with one 16-byte load:
//   int8 weights  block of 32 k = 64 B: [tq 0..3][plane hi|lo][half 0|1][4 B]   k = 32 blk + 16 half + 4 tq + e
//   int4 weights  block of 64 k = 128 B: [tq][parity][plane][half][4 B]          k = 64 blk + 2 (16 half + 4 tq + e) + parity
//                 (a stored byte holds indices 2B and 2B+1; the low nibbles of a word form one MMA operand, the high
//                 nibbles another, so even and odd indices are kept apart)
// Values 0..3 and 4..7 of the run go to two words per plane (int8: tq and tq + 1; int4: even and odd indices).
template <int WB>
__device__ __forceinline__ void fx_store8(uint32_t row_addr, int k0, const int (&q)[8]) {
  // q holds the fixed-point value + 128: byte 1 is the high plane, byte 0 with its top bit flipped the low plane, both
  // signed (value = 256 hi + lo, lo in [-128, 127], |hi| <= 127)
  constexpr uint32_t kFlip = 0x80808080u;
  if constexpr (WB == 8) {
    const uint32_t blk = (uint32_t)k0 >> 5, o = (uint32_t)k0 & 31u, half = o >> 4, tq = (o & 15u) >> 2;  // tq is 0 or 2
    const uint32_t base = row_addr + blk * 64u + tq * 16u + half * 4u;
    sts32(base, prmt(prmt(q[0], q[1], 0x0051u), prmt(q[2], q[3], 0x0051u), 0x5410u));            // hi, tq
    sts32(base + 8u, prmt(prmt(q[0], q[1], 0x0040u), prmt(q[2], q[3], 0x0040u), 0x5410u) ^ kFlip);       // lo, tq
    sts32(base + 16u, prmt(prmt(q[4], q[5], 0x0051u), prmt(q[6], q[7], 0x0051u), 0x5410u));      // hi, tq + 1
    sts32(base + 24u, prmt(prmt(q[4], q[5], 0x0040u), prmt(q[6], q[7], 0x0040u), 0x5410u) ^ kFlip);      // lo, tq + 1
  } else {
    const uint32_t blk = (uint32_t)k0 >> 6, B = ((uint32_t)k0 & 63u) >> 1, half = B >> 4, tq = (B & 15u) >> 2;
    const uint32_t base = row_addr + blk * 128u + tq * 32u + half * 4u;
    sts32(base, prmt(prmt(q[0], q[2], 0x0051u), prmt(q[4], q[6], 0x0051u), 0x5410u));            // even k, hi
    sts32(base + 8u, prmt(prmt(q[0], q[2], 0x0040u), prmt(q[4], q[6], 0x0040u), 0x5410u) ^ kFlip);       // even k, lo
    sts32(base + 16u, prmt(prmt(q[1], q[3], 0x0051u), prmt(q[5], q[7], 0x0051u), 0x5410u));      // odd k, hi
    sts32(base + 24u, prmt(prmt(q[1], q[3], 0x0040u), prmt(q[5], q[7], 0x0040u), 0x5410u) ^ kFlip);      // odd k, lo
  }
}

// rint(a * inv) + 128 for |a * inv| < 2^22, as the low bits of a float sum: 1.5 * 2^23 + 128 + q has q + 128 (two's
// complement) in its low mantissa bits, and fx_store8 only takes bytes 0 and 1.  One FMA instead of a multiply and a
// conversion.
__device__ __forceinline__ int fx_round(float a, float inv) { return __float_as_int(fmaf(a, inv, 12582912.f + 128.f)); }

template <bool BF16>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack16x2<BF16>(w[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// 8 packed 16-bit values: a := silu(a) * m, rounded back to the 16-bit type (what the unfused product would hold).
template <bool BF16>
__device__ __forceinline__ void silu_mul8(uint4& a, const uint4& m) {
  float fa[8], fm[8];
  unpack8<BF16>(a, fa);
  unpack8<BF16>(m, fm);
#pragma unroll
  for (int e = 0; e < 8; ++e) fa[e] = fa[e] / (1.f + __expf(-fa[e])) * fm[e];
  a.x = pack16x2<BF16>(fa[0], fa[1]); a.y = pack16x2<BF16>(fa[2], fa[3]);
  a.z = pack16x2<BF16>(fa[4], fa[5]); a.w = pack16x2<BF16>(fa[6], fa[7]);
}

// The fixed-point conversion works in place on rows that lie as plain 16-bit values at the start of their fixed-point
// rows in shared memory: a 32-index block of int8 rows (64-index block of int4 rows) covers the same bytes before and
// after, and the 4 (8) lanes that hold its 16-byte pieces all read before any of them writes.  The loops are rolled on
// purpose: this code runs once per launch, so that its size (instruction fetches) counts for more than its ILP.
// A warp's pieces of a row are base + lane for base = base0, base0 + step, ... (multiples of 32).
template <bool BF16>
__device__ __forceinline__ uint32_t absmax2(uint32_t m, uint32_t w) {
  if constexpr (BF16) {
    const __nv_bfloat162 r = __hmax2(__habs2(*reinterpret_cast<const __nv_bfloat162*>(&w)), *reinterpret_cast<const __nv_bfloat162*>(&m));
    return *reinterpret_cast<const uint32_t*>(&r);
  } else {
    const __half2 r = __hmax2(__habs2(*reinterpret_cast<const __half2*>(&w)), *reinterpret_cast<const __half2*>(&m));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
}

// Largest of the 64 packed non-negative 16-bit floats a warp holds in m2, as a float in every lane: non-negative
// floats order like their bit patterns, so one integer warp reduction does it.
template <bool BF16>
__device__ __forceinline__ float warp_max16(uint32_t m2) {
  const uint32_t m = __reduce_max_sync(0xffffffffu, max(m2 & 0xffffu, m2 >> 16));
  return unpack16x2<BF16>(m).x;
}

// Largest magnitude over the warp's pieces of a row (NaNs do not count), the same value in every lane.
template <bool BF16>
__device__ __forceinline__ float fx_row_absmax(uint32_t row_addr, int base0, int step, int pieces, int lane) {
  uint32_t m2 = 0;
#pragma unroll 1
  for (int base = base0; base < pieces; base += step) {
    const int pc = base + lane;
    if (pc < pieces) {
      uint32_t a, b, c, d;
      lds128(row_addr + (uint32_t)pc * 16u, a, b, c, d);
      m2 = absmax2<BF16>(absmax2<BF16>(m2, a), b);
      m2 = absmax2<BF16>(absmax2<BF16>(m2, c), d);
    }
  }
  return warp_max16<BF16>(m2);
}

// Scale of a row with largest magnitude m, and its inverse (an all-zero, infinite or NaN row reads as zeros).
__device__ __forceinline__ float fx_scale(float m, float& inv) {
  const bool fin = m > 0.f && m < 3.0e38f;
  inv = fin ? __fdividef(32512.f, m) : 0.f;
  return fin ? m * (1.f / 32512.f) : 0.f;
}

template <bool BF16, int WB>
__device__ __forceinline__ void fx_row_convert(uint32_t row_addr, int base0, int step, int pieces, float inv, int lane) {
#pragma unroll 1
  for (int base = base0; base < pieces; base += step) {  // warp-uniform bounds
    const int pc = base + lane;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (pc < pieces) lds128(row_addr + (uint32_t)pc * 16u, v.x, v.y, v.z, v.w);
    __syncwarp();
    if (pc < pieces) {
      float f[8];
      int q[8];
      unpack8<BF16>(v, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) q[e] = fx_round(f[e], inv);
      fx_store8<WB>(row_addr, pc * 8, q);
    }
  }
}

// Short rows (at most 32 pieces: one per lane), four rows of the warp at a time so that their dependent chains
// (load, maximum, shuffles, scale, conversion) overlap.  Rows rb .. rb + 3 with rb = 4 (warp + 16 it).
template <bool BF16, int WB>
__device__ __forceinline__ void fx_rows4(int nrows, int pieces, uint32_t rows0, uint32_t pitch, float* scales, int warp, int lane) {
  const bool have = lane < pieces;
#pragma unroll 1
  for (int rb = warp * 4; rb < nrows; rb += kW * 4) {
    uint4 v[4];
    float m[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = make_uint4(0, 0, 0, 0);
      if (have && rb + i < nrows) lds128(rows0 + (uint32_t)(rb + i) * pitch + (uint32_t)lane * 16u, v[i].x, v[i].y, v[i].z, v[i].w);
      m[i] = warp_max16<BF16>(absmax2<BF16>(absmax2<BF16>(absmax2<BF16>(absmax2<BF16>(0u, v[i].x), v[i].y), v[i].z), v[i].w));
    }
    __syncwarp();  // every lane has read its pieces: the stores below land on other lanes' pieces of the same block
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (rb + i < nrows) {  // warp-uniform
        float inv;
        const float sc = fx_scale(m[i], inv);
        if (lane == 0) scales[rb + i] = sc;
        if (have) {
          float f[8];
          int q[8];
          unpack8<BF16>(v[i], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) q[e] = fx_round(f[e], inv);
          fx_store8<WB>(rows0 + (uint32_t)(rb + i) * pitch, lane * 8, q);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------- chunk consumers
// One 128-byte K-chunk of a 16-row weight group (rows 0..15 of the box at sW).  The shared-memory loads of a batch of
// 32-byte windows are issued before the first use, so that their latencies overlap.
// 16-bit weights: activation boxes at sA (one 64-wide box per chunk).
template <bool BF16, int NT>
__device__ __forceinline__ void sp_k16(uint32_t sW, uint32_t sA, float (&acc)[4][NT][4], int lane) {
  const uint32_t jm = lane >> 3, l7 = lane & 7;
  const uint32_t row = l7 + (jm & 1) * 8;
  uint32_t a[4][4], bf[4][NT][2];
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    ldsm_x4(sW + sw128(row, ks * 2 + (jm >> 1)), a[ks][0], a[ks][1], a[ks][2], a[ks][3]);
    load_bfrag<NT>(sA, ks, lane, bf[ks]);
  }
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
#pragma unroll
    for (int n = 0; n < NT; ++n) mma_16816<BF16>(acc[ks][n], a[ks][0], a[ks][1], a[ks][2], a[ks][3], bf[ks][n][0], bf[ks][n][1]);
}

// int8 weights, 128 k per chunk: four 32-byte windows = four m16n8k32 steps per plane.  sA: fixed-point row of token
// 0 at the chunk's first index, rows `pitch` bytes apart; token rows past N read as zero.
template <int NT>
__device__ __forceinline__ void iq_k8(uint32_t sW, uint32_t sA, uint32_t pitch, int N, int (&hi)[NT][4], int (&lo)[NT][4], int lane) {
  const uint32_t jm = lane >> 3, l7 = lane & 7, g = lane >> 2, tq = lane & 3;
  const uint32_t row = l7 + (jm & 1) * 8;
  // token rows past N read token 0's row: their output columns are never looked at, and integers have no NaN
  uint32_t arow[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) arow[n] = sA + ((int)(n * 8 + g) < N ? (n * 8 + g) : 0u) * pitch + tq * 16;
  constexpr int WBATCH = NT == 1 ? 4 : 2;
#pragma unroll
  for (int w0 = 0; w0 < 4; w0 += WBATCH) {
    uint32_t a[WBATCH][4], b[WBATCH][NT][4];
#pragma unroll
    for (int i = 0; i < WBATCH; ++i) {
      const int win = w0 + i;
      ldsm_x4(sW + sw128(row, win * 2 + (jm >> 1)), a[i][0], a[i][1], a[i][2], a[i][3]);
#pragma unroll
      for (int n = 0; n < NT; ++n) lds128(arow[n] + win * 64, b[i][n][0], b[i][n][1], b[i][n][2], b[i][n][3]);
    }
#pragma unroll
    for (int i = 0; i < WBATCH; ++i)
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        imma_s8s8(hi[n], a[i][0], a[i][1], a[i][2], a[i][3], b[i][n][0], b[i][n][1]);
        imma_s8s8(lo[n], a[i][0], a[i][1], a[i][2], a[i][3], b[i][n][2], b[i][n][3]);
      }
  }
}

// Packed int4 weights, 256 k per chunk: a 32-byte window holds 64 indices; the low nibbles of its words (shifted into
// the high half of each byte: 16 v as a signed byte) multiply the even indices, the high nibbles the odd ones.  The
// factor 16 is divided out with the scales.
template <int NT, int WLO, int WHI>
__device__ __forceinline__ void iq_k4_win(uint32_t sW, uint32_t sA, uint32_t pitch, int N, int (&hi)[NT][4], int (&lo)[NT][4], int lane) {
  const uint32_t jm = lane >> 3, l7 = lane & 7, g = lane >> 2, tq = lane & 3;
  const uint32_t row = l7 + (jm & 1) * 8;
  uint32_t arow[NT];  // (token rows past N read token 0's row, see iq_k8)
#pragma unroll
  for (int n = 0; n < NT; ++n) arow[n] = sA + ((int)(n * 8 + g) < N ? (n * 8 + g) : 0u) * pitch + tq * 32;
  constexpr int WBATCH = NT == 1 ? 2 : 1;
#pragma unroll
  for (int w0 = WLO; w0 < WHI; w0 += WBATCH) {
    uint32_t r[WBATCH][4], be[WBATCH][NT][4], bo[WBATCH][NT][4];
#pragma unroll
    for (int i = 0; i < WBATCH; ++i) {
      const int win = w0 + i;
      ldsm_x4(sW + sw128(row, win * 2 + (jm >> 1)), r[i][0], r[i][1], r[i][2], r[i][3]);
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        lds128(arow[n] + win * 128, be[i][n][0], be[i][n][1], be[i][n][2], be[i][n][3]);
        lds128(arow[n] + win * 128 + 16, bo[i][n][0], bo[i][n][1], bo[i][n][2], bo[i][n][3]);
      }
    }
#pragma unroll
    for (int i = 0; i < WBATCH; ++i) {
      uint32_t ae[4], ao[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        ae[e] = (r[i][e] << 4) & 0xF0F0F0F0u;
        ao[e] = r[i][e] & 0xF0F0F0F0u;
      }
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        imma_s8s8(hi[n], ae[0], ae[1], ae[2], ae[3], be[i][n][0], be[i][n][1]);
        imma_s8s8(lo[n], ae[0], ae[1], ae[2], ae[3], be[i][n][2], be[i][n][3]);
        imma_s8s8(hi[n], ao[0], ao[1], ao[2], ao[3], bo[i][n][0], bo[i][n][1]);
        imma_s8s8(lo[n], ao[0], ao[1], ao[2], ao[3], bo[i][n][2], bo[i][n][3]);
      }
    }
  }
}

template <int NT>
__device__ __forceinline__ void iq_k4(uint32_t sW, uint32_t sA, uint32_t pitch, int N, int (&hi)[NT][4], int (&lo)[NT][4], int lane) {
  iq_k4_win<NT, 0, 4>(sW, sA, pitch, N, hi, lo, lane);
}
// Windows first .. first + 1 of the chunk: one scale group of 128 indices (first is 0 or 2).
template <int NT>
__device__ __forceinline__ void iq_k4_half(uint32_t sW, uint32_t sA, uint32_t pitch, int N, int (&hi)[NT][4], int (&lo)[NT][4], int lane,
                                           int first) {
  if (first == 0) iq_k4_win<NT, 0, 2>(sW, sA, pitch, N, hi, lo, lane);
  else iq_k4_win<NT, 2, 4>(sW, sA, pitch, N, hi, lo, lane);
}

// Up to 4 tokens, both planes in one MMA: output column c of the 8 holds token c % 4, plane c / 4 (high planes
// first), so lane (g, tq) fetches the 8 bytes of its plane of token g % 4 per window.  Half the MMAs and half the
// activation bytes of the two-MMA form.
template <int WLO, int WHI>
__device__ __forceinline__ void iq_k8_merged(uint32_t sW, uint32_t sA, uint32_t pitch, int N, int (&acc)[4], int lane) {
  const uint32_t jm = lane >> 3, l7 = lane & 7, g = lane >> 2, tq = lane & 3;
  const uint32_t row = l7 + (jm & 1) * 8;
  const uint32_t arow = sA + ((int)(g & 3) < N ? (g & 3) : 0u) * pitch + tq * 16 + (g >> 2) * 8;
  uint32_t a[WHI - WLO][4], b[WHI - WLO][2];
#pragma unroll
  for (int i = 0; i < WHI - WLO; ++i) {
    const int win = WLO + i;
    ldsm_x4(sW + sw128(row, win * 2 + (jm >> 1)), a[i][0], a[i][1], a[i][2], a[i][3]);
    lds64(arow + win * 64, b[i][0], b[i][1]);
  }
#pragma unroll
  for (int i = 0; i < WHI - WLO; ++i) imma_s8s8(acc, a[i][0], a[i][1], a[i][2], a[i][3], b[i][0], b[i][1]);
}
template <int WLO, int WHI>
__device__ __forceinline__ void iq_k4_merged(uint32_t sW, uint32_t sA, uint32_t pitch, int N, int (&acc)[4], int lane) {
  const uint32_t jm = lane >> 3, l7 = lane & 7, g = lane >> 2, tq = lane & 3;
  const uint32_t row = l7 + (jm & 1) * 8;
  const uint32_t arow = sA + ((int)(g & 3) < N ? (g & 3) : 0u) * pitch + tq * 32 + (g >> 2) * 8;
#pragma unroll
  for (int w0 = WLO; w0 < WHI; w0 += 2) {
    uint32_t r[2][4], be[2][2], bo[2][2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int win = w0 + i;
      ldsm_x4(sW + sw128(row, win * 2 + (jm >> 1)), r[i][0], r[i][1], r[i][2], r[i][3]);
      lds64(arow + win * 128, be[i][0], be[i][1]);
      lds64(arow + win * 128 + 16, bo[i][0], bo[i][1]);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t ae[4], ao[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        ae[e] = (r[i][e] << 4) & 0xF0F0F0F0u;
        ao[e] = r[i][e] & 0xF0F0F0F0u;
      }
      imma_s8s8(acc, ae[0], ae[1], ae[2], ae[3], be[i][0], be[i][1]);
      imma_s8s8(acc, ao[0], ao[1], ao[2], ao[3], bo[i][0], bo[i][1]);
    }
  }
}

// Accumulators of one work item: fp32 chains for 16-bit weights, integer planes for quantised weights, and the
// running fp32 total that per-group scales fold into.  MG (quantised weights, up to 4 tokens): one integer
// accumulator whose columns are (token, plane); finish() brings the planes of a token together (they sit two lanes
// apart), after which lanes with tq < 2 hold tokens 2 tq and 2 tq + 1 like the other forms and the other lanes'
// values belong to token columns 4..7, which nobody reads.
template <int NT, int WB, bool MG>
struct ItemAcc {
  float acc[WB == 16 ? 4 : 1][NT][4];
  int hi[NT][4], lo[MG ? 1 : NT][4];
  float tot[NT][4];
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        tot[n][e] = 0.f;
        hi[n][e] = 0;
        if constexpr (!MG) lo[n][e] = 0;
#pragma unroll
        for (int q = 0; q < (WB == 16 ? 4 : 1); ++q) acc[q][n][e] = 0.f;
      }
  }
  // integer planes -> tot, scaled by the two rows' group scales, and cleared (per-group scales)
  __device__ __forceinline__ void fold(float s_row, float s_row8) {
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float v = MG ? (float)hi[n][e] : fmaf((float)hi[n][e], 256.f, (float)lo[MG ? 0 : n][e]);
        tot[n][e] = fmaf(e < 2 ? s_row : s_row8, v, tot[n][e]);
        hi[n][e] = 0;
        if constexpr (!MG) lo[n][e] = 0;
      }
  }
  // once, after the last chunk and before value(): every lane of the warp
  __device__ __forceinline__ void finish(bool grouped) {
    if constexpr (MG) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mine = grouped ? tot[0][e] : (float)hi[0][e];
        const float other = __shfl_xor_sync(0xffffffffu, mine, 2);  // the low plane of lanes tq < 2
        tot[0][e] = fmaf(mine, 256.f, other);
      }
    }
  }
  // value of accumulator element (n, e) before the per-channel and activation scales
  __device__ __forceinline__ float value(int n, int e, bool grouped) const {
    if constexpr (WB == 16) return acc[0][n][e] + acc[1][n][e] + acc[2][n][e] + acc[3][n][e];
    else if constexpr (MG) return tot[0][e];
    else return grouped ? tot[n][e] : fmaf((float)hi[n][e], 256.f, (float)lo[n][e]);
  }
};

// ---------------------------------------------------------------------------------------------------- front
// Quotient by a small runtime divisor without a division: magic = ceil(2^32 / d), exact for t < 65536 (d = 1: magic 0).
__device__ __forceinline__ uint32_t fastdiv(uint32_t t, uint32_t d, uint32_t magic) { return d == 1u ? t : __umulhi(t, magic); }

// Clock stamps of profiling builds (thread 0, cycles since `tck`).
#ifdef BLR_TIMELINE
#define BLR_CK(slot) do { if (threadIdx.x == 0) BLR_TLV(slot, clock64() - tck); } while (0)
#else
#define BLR_CK(slot) do { } while (0)
#endif

// Fixed-point conversion of x once per call (more than 2 tokens, or an input transform: where every front CTA converting all of x itself
// costs more than this extra launch): CTA c takes rows 16 c .. 16 c + 15 of the b * N (in-block, token) rows, a warp a
// row, with the front kernel's own staging code, and writes the converted row and its scale to scratch in the layout
// the front kernel keeps in shared memory.
template <bool BF16, int WB, bool ACT>
__global__ void __launch_bounds__(kSplitFrontThreads) blr_blast_fx_kernel(const __grid_constant__ SplitParams p) {
  extern __shared__ __align__(16) uint8_t fx_smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int N = p.N, P = p.P, pieces = P >> 3, nrows = p.b * N;
  const uint32_t pitch = fx_pitch(P, WB);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int r = blockIdx.x * kW + warp;
  if (r >= nrows) return;
  const int j = (int)fastdiv((uint32_t)r, (uint32_t)N, p.magic_N), n = r - j * N;
  const long long off = (long long)n * p.ldx + (long long)j * P;
  const uint16_t* x = reinterpret_cast<const uint16_t*>(p.x) + off;
  const uint32_t row_addr = smem_u32(fx_smem) + (uint32_t)warp * pitch;
#pragma unroll 1
  for (int pc = lane; pc < pieces; pc += 32) cp_async16(row_addr + (uint32_t)pc * 16u, x + pc * 8);
  cp_async_wait_all();
  __syncwarp();
  if constexpr (ACT) {
    const uint16_t* xm = reinterpret_cast<const uint16_t*>(p.x_mul) + off;
#pragma unroll 1
    for (int pc = lane; pc < pieces; pc += 32) {
      const uint32_t a = row_addr + (uint32_t)pc * 16u;
      uint4 v;
      lds128(a, v.x, v.y, v.z, v.w);
      silu_mul8<BF16>(v, ld_global_cg_v4(xm + pc * 8));
      asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
    }
    __syncwarp();
  }
  float inv;
  const float sc = fx_scale(fx_row_absmax<BF16>(row_addr, 0, 32, pieces, lane), inv);
  fx_row_convert<BF16, WB>(row_addr, 0, 32, pieces, inv, lane);
  __syncwarp();
  // the converted row (its padding included: whatever it holds meets weights that TMA filled with zeros) and its scale
  uint8_t* dst = reinterpret_cast<uint8_t*>(p.xq) + (size_t)r * pitch;
#pragma unroll 1
  for (uint32_t o = (uint32_t)lane * 16u; o < pitch; o += 512u) {
    uint4 v;
    lds128(row_addr + o, v.x, v.y, v.z, v.w);
    *reinterpret_cast<uint4*>(dst + o) = v;
  }
  if (lane == 0) p.xq_scale[r] = sc;
}

template <bool BF16, int NT, bool GS, int WB, bool ACT, bool MG>
__global__ void __launch_bounds__(kSplitFrontThreads, 2) blr_blast_front_kernel(const __grid_constant__ SplitParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  constexpr int NP = NT * 8;
  constexpr int wbits = WB, abox = 16 / WB;
  constexpr bool FX = WB != 16;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int N = p.N, nb = p.b, bo = p.z_shared ? 1 : p.bo, nch = p.nch0, R = p.R;  // (one z for every out-block: see z_shared)
  const int nbx = nch * abox;
  const int r0 = blockIdx.x * kSplitRanks;
  const SplitProblem& q = p.pr[blockIdx.y];
  const uint32_t xbox = (uint32_t)N * 128u, xpitch = FX ? fx_pitch(p.P, WB) : 0u;
  const FrontLayout L = front_layout(p);
  const uint32_t bar = smem_base + L.bar;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.bar + 8);
  float* vs = reinterpret_cast<float*>(smem + L.vs);
  float* sx = reinterpret_cast<float*>(smem + L.sx);
  float* ypart = reinterpret_cast<float*>(smem + L.ypart);
  float* ybuf = reinterpret_cast<float*>(smem + L.ybuf);
#ifdef BLR_TIMELINE
  long long tck = 0;
#endif

  const uint32_t xbar = bar + 16;
  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar, 1);
    mbar_init(xbar, 1);
    mbar_init_fence();
  }
  BLR_TL(0);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __syncthreads();
  // ---- everything that does not depend on the kernel ahead: the slice's rows of every V_j, its coupling factors, scales
  if (tid == 0) {
    mbar_arrive_expect_tx(bar, (uint32_t)nch * nb * 1024u);
    constexpr int kstep = wbits == 16 ? 64 : 128;
#pragma unroll 1
    for (int c = 0; c < nch; ++c) tma_load_3d(smem_base + L.w + (uint32_t)c * nb * 1024u, &q.tmV, c * kstep, r0, 0, bar);
  }
  {
    const uint16_t* S = reinterpret_cast<const uint16_t*>(q.S);
    const bool s_vec = S != nullptr && p.s_r == 1 && ((p.s_i | p.s_j) & 7) == 0 && (reinterpret_cast<uintptr_t>(S) & 15) == 0;
    const uint32_t pitch = (uint32_t)nb * 16u + 16u;
#pragma unroll 1
    for (int i = warp; i < bo; i += kW)
#pragma unroll 1
      for (int j = lane; j < nb; j += 32) {
        uint16_t* d = reinterpret_cast<uint16_t*>(smem + L.s + i * pitch + j * 16);
        if (S == nullptr) {
#pragma unroll
          for (int k = 0; k < 8; ++k) d[k] = BF16 ? (uint16_t)0x3F80 : (uint16_t)0x3C00;
        } else if (s_vec) {
          cp_async16(smem_u32(d), S + i * p.s_i + j * p.s_j + r0);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) d[k] = S[i * p.s_i + j * p.s_j + (long long)(r0 + k) * p.s_r];
        }
      }
    if (tid < nb * 8) {
      float v = (!GS && q.v_scale != nullptr) ? __half2float(__ldg(q.v_scale + (long long)(tid >> 3) * R + r0 + (tid & 7))) : 1.f;
      if (WB == 4) v *= 0.0625f;  // the int4 operands are 16 v
      vs[tid] = v;
    }
  }
  // (divisions of the product phase, done here where nothing waits for them)
  const int share = split_share(nb);
  const int jw = share == 1 ? warp : warp / share, ws = share == 1 ? 0 : warp - jw * share;
  BLR_TL(1);
  // One warp waits for the kernel ahead; the others sleep at the barrier.
  if (warp == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
  __syncthreads();
  BLR_TL(2);
#ifdef BLR_TIMELINE
  tck = clock64();
#endif
  // ---- x, all of it, one (in-block, token) row per warp and turn
  bool x_bulk = false;
  {
    const uint16_t* x = reinterpret_cast<const uint16_t*>(p.x);
    const uint16_t* xm = reinterpret_cast<const uint16_t*>(p.x_mul);
    constexpr bool act = ACT;
    const int nrows = nb * N;
    if (FX && p.xq != nullptr) {
      // the rows were converted once for the whole grid by blr_blast_fx_kernel: same layout as here, one linear copy
      const uint8_t* src = reinterpret_cast<const uint8_t*>(p.xq);
      const uint32_t bytes = (uint32_t)nrows * xpitch;
      x_bulk = bytes < (1u << 20);  // (an mbarrier counts at most 2^20 - 1 bytes per phase)
      if (x_bulk) {
        if (tid == 0) {  // a few bulk copies by one thread instead of thousands of 16-byte ones by all
          mbar_arrive_expect_tx(xbar, bytes);
#pragma unroll 1
          for (uint32_t o = 0; o < bytes; o += 32768u) bulk_load(smem_base + L.xs + o, src + o, min(32768u, bytes - o), xbar);
        }
      } else {
        const int total = nrows * (int)(xpitch >> 4);
#pragma unroll 1
        for (int i = tid; i < total; i += kSplitFrontThreads) cp_async16(smem_base + L.xs + (uint32_t)i * 16u, src + (size_t)i * 16);
      }
#pragma unroll 1
      for (int i = tid; i < nrows; i += kSplitFrontThreads) sx[i] = __ldcg(p.xq_scale + i);
    } else if constexpr (FX) {
      // raw rows into the fixed-point rows (asynchronously, all of the warp's rows in flight), then in place: the
      // input transform where asked for, the row maximum, the conversion.  The warp's rows come in runs of rr:
      // rows rb .. rb + rr - 1 with rb = rr (warp + 16 it); short rows (one piece per lane) go four at a time.
      const long long ldx = p.ldx;
      const int P = p.P, pieces = P >> 3;
      const uint32_t mN = p.magic_N;
      auto row_off = [&](int r) {
        const int j = (int)fastdiv((uint32_t)r, (uint32_t)N, mN), n = r - j * N;
        return (long long)n * ldx + (long long)j * P;
      };
      const bool short_rows = pieces <= 32 && nrows > kW;  // (with at most one row per warp there is nothing to overlap)
      const int rr = short_rows ? 4 : 1;
#pragma unroll 1
      for (int rb = warp * rr; rb < nrows; rb += kW * rr)
#pragma unroll 1
        for (int r = rb; r < rb + rr && r < nrows; ++r) {
          const uint16_t* src = x + row_off(r);
          const uint32_t row_addr = smem_base + L.xs + (uint32_t)r * xpitch;
#pragma unroll 1
          for (int pc = lane; pc < pieces; pc += 32) cp_async16(row_addr + (uint32_t)pc * 16u, src + pc * 8);
        }
      if constexpr (ACT) {
        // the second operand straight from global memory, one piece ahead of its use
        int rb = warp * rr, r = rb, base = 0;
        auto advance = [&](int& rb_, int& r_, int& base_) {
          base_ += 32;
          if (base_ >= pieces) {
            base_ = 0;
            if (++r_ >= rb_ + rr || r_ >= nrows) r_ = rb_ += kW * rr;
          }
        };
        uint4 nxt = make_uint4(0, 0, 0, 0);
        if (r < nrows && lane < pieces) nxt = ld_global_cg_v4(xm + row_off(r) + lane * 8);
        cp_async_wait_all();
        __syncwarp();
#pragma unroll 1
        while (r < nrows) {
          const uint4 cur = nxt;
          int rb2 = rb, r2 = r, b2 = base;
          advance(rb2, r2, b2);
          if (r2 < nrows && b2 + lane < pieces) nxt = ld_global_cg_v4(xm + row_off(r2) + (b2 + lane) * 8);
          if (base + lane < pieces) {
            const uint32_t a = smem_base + L.xs + (uint32_t)r * xpitch + (uint32_t)(base + lane) * 16u;
            uint4 v;
            lds128(a, v.x, v.y, v.z, v.w);
            silu_mul8<BF16>(v, cur);
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
          }
          rb = rb2;
          r = r2;
          base = b2;
        }
      } else {
        cp_async_wait_all();
      }
      __syncwarp();
      if (short_rows) {
        fx_rows4<BF16, WB>(nrows, pieces, smem_base + L.xs, xpitch, sx, warp, lane);
      } else {
#pragma unroll 1
        for (int r = warp; r < nrows; r += kW) {
          const uint32_t row_addr = smem_base + L.xs + (uint32_t)r * xpitch;
          float inv;
          const float sc = fx_scale(fx_row_absmax<BF16>(row_addr, 0, 32, pieces, lane), inv);
          if (lane == 0) sx[r] = sc;
          fx_row_convert<BF16, WB>(row_addr, 0, 32, pieces, inv, lane);
        }
      }
    } else if constexpr (act) {
      // silu(x) * x_mul through registers into the same [in-block][64-wide box][token][128 B] layout, zero past P
      const int cpr = nbx * 8;
      for (int rowi = warp; rowi < nrows; rowi += kW) {
        const int j = (int)fastdiv((uint32_t)rowi, (uint32_t)N, p.magic_N), n = rowi - j * N;
        const long long off = (long long)n * p.ldx + (long long)j * p.P;
        const uint32_t dst0 = smem_base + L.xs + (uint32_t)(j * nbx * N + n) * 128u;
        for (int ch = lane; ch < cpr; ch += 32) {
          const int kb = ch >> 3, c16 = ch & 7, k = ch * 8;
          uint4 v = make_uint4(0, 0, 0, 0);
          if (k < p.P) {
            v = ld_global_cg_v4(x + off + k);
            silu_mul8<BF16>(v, ld_global_cg_v4(xm + off + k));
          }
          const uint32_t d = dst0 + (uint32_t)kb * xbox + (uint32_t)((c16 ^ (n & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(d), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
        }
      }
    } else {
      // [in-block][64-wide box][token][128 B], zero past P
      const int cpr = nbx * 8;  // 16-byte pieces per row
      for (int rowi = warp; rowi < nrows; rowi += kW) {
        const int j = (int)fastdiv((uint32_t)rowi, (uint32_t)N, p.magic_N), n = rowi - j * N;
        const uint16_t* src = x + (long long)n * p.ldx + (long long)j * p.P;
        const uint32_t dst0 = smem_base + L.xs + (uint32_t)(j * nbx * N + n) * 128u;
        for (int ch = lane; ch < cpr; ch += 32) {
          const int kb = ch >> 3, c16 = ch & 7, k = ch * 8;
          const bool in = k < p.P;
          cp_async16_zfill(dst0 + (uint32_t)kb * xbox + (uint32_t)((c16 ^ (n & 7)) << 4), src + (in ? k : 0), in ? 16u : 0u);
        }
      }
    }
  }
  cp_async_wait_all();
  BLR_CK(7);
  bool ok = mbar_wait(bar, 0, abort_flag);
  if (x_bulk) ok = mbar_wait(xbar, 0, abort_flag) && ok;
  if (__syncthreads_or(ok ? 0 : 1)) {
    if (tid == 0) atomicExch(p.status, 1u);
    return;
  }
  BLR_CK(8);
  // ---- y_j on the slice.  A warp owns an in-block (warps w, w + 16, ... beyond 16 in-blocks) and runs down its
  // chunks with one accumulator, then scales and stores y[j][n][r].  With fewer than 9 in-blocks `share` warps split
  // the chunks of one in-block and their sums meet in shared memory, added in a fixed order.  Rows 8..15 of the MMA are
  // the next block's rows (or slack) against the wrong activations: never read back.
  {
    const int g = lane >> 2, tq = lane & 3;
    const int ngroups = GS ? p.P / kScaleGroup : 0;
    constexpr uint32_t kChunkAct = WB == 8 ? 256u : 512u;  // fixed-point bytes of one chunk's indices in a token row
    ItemAcc<NT, WB, MG> A;
#pragma unroll 1
    for (int j = jw; j < nb; j += kW) {
      A.clear();
#pragma unroll 1
      for (int c = ws; c < nch; c += share) {
        const uint32_t sW = smem_base + L.w + (uint32_t)(c * nb + j) * 1024u;
        if constexpr (WB == 16) {
          sp_k16<BF16, NT>(sW, smem_base + L.xs + (uint32_t)(j * nbx + c) * xbox, A.acc, lane);
        } else {
          const uint32_t sA = smem_base + L.xs + (uint32_t)(j * N) * xpitch + (uint32_t)c * kChunkAct;
          float gsc = 0.f, gsc2 = 0.f;
          if constexpr (GS) {
            const __half* srow = q.v_scale + ((long long)j * R + r0 + g) * ngroups;
            const int gi = c * (WB == 8 ? 1 : 2);
            gsc = __half2float(__ldg(srow + gi));
            if (WB == 4 && gi + 1 < ngroups) gsc2 = __half2float(__ldg(srow + gi + 1));
          }
          if constexpr (MG && WB == 8) {
            iq_k8_merged<0, 4>(sW, sA, xpitch, N, A.hi[0], lane);
            if constexpr (GS) A.fold(gsc, 0.f);
          } else if constexpr (MG && !GS) {
            iq_k4_merged<0, 4>(sW, sA, xpitch, N, A.hi[0], lane);
          } else if constexpr (MG) {
            iq_k4_merged<0, 2>(sW, sA, xpitch, N, A.hi[0], lane);
            A.fold(gsc, 0.f);
            iq_k4_merged<2, 4>(sW, sA, xpitch, N, A.hi[0], lane);
            A.fold(gsc2, 0.f);
          } else if constexpr (WB == 8) {
            iq_k8<NT>(sW, sA, xpitch, N, A.hi, A.lo, lane);
            if constexpr (GS) A.fold(gsc, 0.f);
          } else if constexpr (!GS) {
            iq_k4<NT>(sW, sA, xpitch, N, A.hi, A.lo, lane);
          } else {
            // two scale groups per chunk: the first two windows, then the last two
            iq_k4_half<NT>(sW, sA, xpitch, N, A.hi, A.lo, lane, 0);
            A.fold(gsc, 0.f);
            iq_k4_half<NT>(sW, sA, xpitch, N, A.hi, A.lo, lane, 2);
            A.fold(gsc2, 0.f);
          }
        }
      }
      A.finish(GS);
      if (share == 1) {
        const float vsc = vs[j * 8 + g];
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int tok = n * 8 + tq * 2 + e;
            if (tok < N) {
              float y = A.value(n, e, GS) * vsc;
              if constexpr (FX) y *= sx[j * N + tok];
              if (p.round_y) y = round_clamp_i8(y);
              ybuf[(j * N + tok) * 8 + g] = y;
            }
          }
      } else {
        float* slot = ypart + ((j * share + ws) * 8 + g) * NP;
#pragma unroll
        for (int n = 0; n < NT; ++n)
          *reinterpret_cast<float2*>(slot + n * 8 + tq * 2) = make_float2(A.value(n, 0, GS), A.value(n, 1, GS));
      }
    }
    BLR_CK(9);
    __syncthreads();
    BLR_CK(10);
    BLR_TL(5);
    if (share > 1) {
      // y[j][n][r] = scales * sum of the sharing warps' slots (fixed order)
#pragma unroll 1
      for (int e = tid; e < nb * N * 8; e += kSplitFrontThreads) {
        const int gg = e & 7, t = e >> 3, j = (int)fastdiv((uint32_t)t, (uint32_t)N, p.magic_N), n = t - j * N;
        const float* yp = ypart + (j * share * 8 + gg) * NP + n;
        float y = yp[0];
#pragma unroll 1
        for (int cm = 1; cm < share; ++cm) y += yp[cm * 8 * NP];
        y *= vs[j * 8 + gg];
        if constexpr (FX) y *= sx[t];
        if (p.round_y) y = round_clamp_i8(y);
        ybuf[t * 8 + gg] = y;
      }
      __syncthreads();
    }
  }
  // ---- Monarch: no coupling; row m of in-block k goes to position k * per + jj of z_l, with (l, jj) = (m / per, m % per)
  // for grouped rows or (m % b, m / b) for the reference's torch layout (the permutation between the two factors)
  if (p.monarch) {
    const int per = p.mon_per;
#pragma unroll 1
    for (int e = tid; e < nb * N * 8; e += kSplitFrontThreads) {
      const int gg = e & 7, t = e >> 3, k = (int)fastdiv((uint32_t)t, (uint32_t)N, p.magic_N), n = t - k * N;
      const int m = r0 + gg;
      const int l = p.mon_torch ? m % nb : m / per, jj = p.mon_torch ? m / nb : m - l * per;
      float a = ybuf[t * 8 + gg];
      if (p.round_z) a = round_clamp_i8(a);
      store16<BF16>(q.z, ((long long)l * N + n) * R + (long long)k * per + jj, a);
    }
  }
  // ---- z[i][n][r] = sum_j S[i][j][r] y[j][n][r].  Few points (fewer than threads): a thread per point with four
  // partial sums (terms j = q mod 4), added in a fixed order.
  else if (bo * N * 8 <= kSplitFrontThreads / 2) {
    const uint32_t pitch = (uint32_t)nb * 16u + 16u;
#pragma unroll 1
    for (int e = tid; e < bo * N * 8; e += kSplitFrontThreads) {
      const int gg = e & 7, t = e >> 3, i = (int)fastdiv((uint32_t)t, (uint32_t)N, p.magic_N), n = t - i * N;
      const uint8_t* srow = smem + L.s + i * pitch + gg * 2;
      const float* yp = ybuf + n * 8 + gg;
      float a4[4] = {0.f, 0.f, 0.f, 0.f};
      int j = 0;
#pragma unroll 1
      for (; j + 4 <= nb; j += 4) {
#pragma unroll
        for (int q = 0; q < 4; ++q) a4[q] = fmaf(load16<BF16>(srow + (j + q) * 16, 0), yp[(j + q) * N * 8], a4[q]);
      }
#pragma unroll 1
      for (; j < nb; ++j) a4[0] = fmaf(load16<BF16>(srow + j * 16, 0), yp[j * N * 8], a4[0]);
      float a = (a4[0] + a4[1]) + (a4[2] + a4[3]);
      if (p.round_z) a = round_clamp_i8(a);
      store16<BF16>(q.z, (long long)t * R + r0 + gg, a);
    }
  }
  else {  // more points: four ranks per thread, the terms in rising j
    const uint32_t pitch = (uint32_t)nb * 16u + 16u;
#pragma unroll 1
    for (int e = tid; e < bo * N * 2; e += kSplitFrontThreads) {
      const int g4 = (e & 1) * 4, t = e >> 1, i = (int)fastdiv((uint32_t)t, (uint32_t)N, p.magic_N), n = t - i * N;
      const uint32_t srow = smem_base + L.s + (uint32_t)i * pitch + (uint32_t)g4 * 2u;
      const float* yp = ybuf + n * 8 + g4;
      float a[4] = {0.f, 0.f, 0.f, 0.f};
      auto term = [&](int j) {
        uint32_t s01, s23;
        asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(s01), "=r"(s23) : "r"(srow + (uint32_t)j * 16u));
        const float4 y = *reinterpret_cast<const float4*>(yp + j * N * 8);
        const float2 sa = unpack16x2<BF16>(s01), sb = unpack16x2<BF16>(s23);
        a[0] = fmaf(sa.x, y.x, a[0]);
        a[1] = fmaf(sa.y, y.y, a[1]);
        a[2] = fmaf(sb.x, y.z, a[2]);
        a[3] = fmaf(sb.y, y.w, a[3]);
      };
      int j = 0;
#pragma unroll 1
      for (; j + 4 <= nb; j += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) term(j + u);
      }
#pragma unroll 1
      for (; j < nb; ++j) term(j);
      if (p.round_z) {
#pragma unroll
        for (int c = 0; c < 4; ++c) a[c] = round_clamp_i8(a[c]);
      }
      uint32_t* dst = reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(q.z) + (long long)t * R + r0 + g4);
      asm volatile("st.global.v2.b32 [%0], {%1,%2};" ::"l"(dst), "r"(pack16x2<BF16>(a[0], a[1])), "r"(pack16x2<BF16>(a[2], a[3])) : "memory");
    }
  }
  BLR_CK(11);
  BLR_TL(6);
}

// ---------------------------------------------------------------------------------------------------- back
template <bool BF16, int NT, bool GS, int WB, bool MG>
__global__ void __launch_bounds__(kSplitBackThreads, 2) blr_blast_back_kernel(const __grid_constant__ SplitParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  constexpr int NP = NT * 8;
  constexpr int wbits = WB, abox = 16 / WB;
  constexpr bool FX = WB != 16;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int N = p.N, nch = p.nch1, R = p.R, Q = p.Q;
  const int nbz = nch * abox;
  const int nseg = (nch + kSplitStageChunks - 1) / kSplitStageChunks;
  const int NST = p.nstages;
  const int blk = blockIdx.x / p.cpb, part = blockIdx.x - blk * p.cpb;
  const SplitProblem& q = p.pr[blockIdx.y];
  const int gpb = (Q + 15) >> 4;
  const int g_lo = part * p.gpc, g_hi = min(gpb, g_lo + p.gpc), ng = g_hi - g_lo;
  const uint32_t zbox = (uint32_t)N * 128u, zpitch = FX ? fx_pitch(R, WB) : 0u;
  const BackLayout L = back_layout(p);
  const uint32_t full0 = smem_base + L.bars, empty0 = full0 + 8u * NST;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.bars + 16 * NST);
  float* partial = reinterpret_cast<float*>(smem + L.part);
  float* us = reinterpret_cast<float*>(smem + L.us);
  float* sz = reinterpret_cast<float*>(smem + L.sz);
  const bool resident = NST >= ng * nseg;  // the CTA's whole share has a stage of its own: no stage is reused
#ifdef BLR_TIMELINE
  long long tck = 0;
#endif

  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < NST; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, kW);
    }
    mbar_init_fence();
  }
  BLR_TL(0);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __syncthreads();
  if (ng <= 0) return;

  if (warp == kW) {
    // ------------------------------------------------ producer: the CTA's rows, one 16-row group x up to 8 chunks per stage.
    // The ring is as long as the CTA's whole share where that fits, so the loads below all leave before anything is
    // consumed, i.e. while the kernel ahead in the stream is still running.
    constexpr int kstep = wbits == 16 ? 64 : 128;
    RingPos rp;
    bool ok = true;
#pragma unroll 1
    for (int g = g_lo; g < g_hi && ok; ++g)
#pragma unroll 1
      for (int seg = 0; seg < nseg; ++seg) {
        if (!rp.first_pass) {
          int w_ok = 1;
          if (lane == 0) w_ok = mbar_wait(empty0 + 8 * rp.s, rp.use_parity ^ 1u, abort_flag) ? 1 : 0;
          w_ok = __shfl_sync(0xffffffffu, w_ok, 0);
          if (!w_ok) { ok = false; break; }
        }
        const int c_lo = seg * kSplitStageChunks, nc = min(kSplitStageChunks, nch - c_lo);
        const uint32_t dst = smem_base + L.ring + rp.s * kSplitStageBytes, fb = full0 + 8 * rp.s;
        if (lane == 0) mbar_arrive_expect_tx(fb, (uint32_t)nc * kSplitChunkBytes);
        __syncwarp();
        if (lane < nc) tma_load_3d(dst + lane * kSplitChunkBytes, &q.tmU, (c_lo + lane) * kstep, g * 16, blk, fb);
        rp.advance(NST);
      }
    return;
  }
  // ------------------------------------------------ consumers
  const int ctid = tid;
  constexpr int kCT = kW * 32;
  const int gq = lane >> 2, tq = lane & 3;
#pragma unroll 1
  for (int e = ctid; e < ng * 16; e += kCT) {
    const int qq = g_lo * 16 + e;
    float v = (!GS && q.u_scale != nullptr && qq < Q) ? __half2float(__ldg(q.u_scale + (long long)blk * Q + qq)) : 1.f;
    if (WB == 4) v *= 0.0625f;
    us[e] = v;
  }
  if (ctid < 16) sz[16 + ctid] = 0.f;  // row maxima of the fixed-point conversion
  // (divisions of the later phases, done here where nothing waits for them)
  const int share = split_share(p.gpc);
  const int gw = share == 1 ? warp : warp / share, ws = share == 1 ? 0 : warp - gw * share;
  const int wpr = N >= kW ? 1 : kW / N, zn = warp / wpr, zwl = warp - zn * wpr;
  const int cpr = nbz * 8, upr = (cpr + 31) >> 5;  // 16-bit path: 16-byte pieces and warp-wide runs per row of z
  const int un0 = warp / upr, ur0 = warp - un0 * upr, udn = kW / upr, udr = kW - udn * upr;
  BLR_TL(1);
  if (warp == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
  named_bar(1, kCT);
  BLR_TL(2);
#ifdef BLR_TIMELINE
  tck = clock64();
#endif
  // ---- z of this out-block
  {
    const uint16_t* z = reinterpret_cast<const uint16_t*>(q.z) + (p.z_shared ? 0ll : (long long)blk * N * R);
    if constexpr (FX) {
      // Every token row is shared out over wpr = 16 / N warps (at least one): each thread takes its 16-byte pieces,
      // the warps' maxima meet in shared memory, then every thread converts its own pieces.
      const int n = zn, wl = zwl;
      const int pieces = R >> 3, base0 = wl * 32, step = wpr * 32;
      float* pm = sz + 16;  // per-row maxima (16 floats after the 16 row scales)
      const bool have_row = n < N;
      const uint32_t row_addr = smem_base + L.zs + (uint32_t)n * zpitch;
      if (have_row) {
#pragma unroll 1
        for (int base = base0; base < pieces; base += step)
          if (base + lane < pieces) cp_async16(row_addr + (uint32_t)(base + lane) * 16u, z + (long long)n * R + (base + lane) * 8);
      }
      cp_async_wait_all();
      __syncwarp();
      if (have_row) {
        const float m = fx_row_absmax<BF16>(row_addr, base0, step, pieces, lane);
        // non-negative floats order like their bit patterns
        if (lane == 0) atomicMax(reinterpret_cast<int*>(pm) + n, __float_as_int(m));
      }
      named_bar(1, kCT);
      if (have_row) {
        float inv;
        const float sc = fx_scale(pm[n], inv);
        if (wl == 0 && lane == 0) sz[n] = sc;
        fx_row_convert<BF16, WB>(row_addr, base0, step, pieces, inv, lane);
      }
    } else {
      // [64-wide box][token][128 B], zero past R.  A warp per run of 32 pieces of a token row.
      // unit u = warp, warp + 16, ...: token u / upr, run u % upr, stepped without divisions
      int n = un0, run = ur0;
#pragma unroll 1
      for (int u = warp; u < N * upr; u += kW) {
        const int ch = run * 32 + lane;
        run += udr;
        const int n_now = n;
        n += udn;
        if (run >= upr) {
          run -= upr;
          ++n;
        }
        if (ch < cpr) {
          const int n = n_now;
          const int kb = ch >> 3, c16 = ch & 7, k = ch * 8;
          const bool in = k < R;
          cp_async16_zfill(smem_base + L.zs + (uint32_t)(kb * N + n) * 128u + (uint32_t)((c16 ^ (n & 7)) << 4),
                           z + (long long)n * R + (in ? k : 0), in ? 16u : 0u);
        }
      }
    }
  }
  cp_async_wait_all();
  named_bar(1, kCT);
  BLR_CK(7);
  BLR_TL(3);
  // ---- products.  A warp owns a 16-row group (groups w, w + 16, ... when the CTA has more than 16) and runs down
  // its chunks with one accumulator; a CTA with fewer than 9 groups lets `share` warps split the chunks of a group.
  // Every warp leaves its sum in its own slot; the slots of a group are added in a fixed order below.  Stage of
  // chunk c of group gl: gl*nseg + c / 8.  When the CTA's whole share is resident a warp only looks at the stages it
  // reads; with a shorter ring every warp walks every stage in order and frees it, used or not.
  bool ok = true;
  const int ngroups = GS ? R / kScaleGroup : 0;
  constexpr uint32_t kChunkAct = WB == 8 ? 256u : 512u;
  {
    ItemAcc<NT, WB, MG> A;
    auto flush = [&](int gl) {
      A.finish(GS);
      // [token][16 rows]: the sums below read neighbouring rows of a token from neighbouring banks
      float* slot = partial + (size_t)(gl * share + ws) * 16 * NP;
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int e = 0; e < 2; ++e) slot[(n * 8 + tq * 2 + e) * 16 + gq + 8 * h] = A.value(n, 2 * h + e, GS);
    };
    auto chunk = [&](int gl, int c, uint32_t s) {
      const int g = g_lo + gl;
      const uint32_t sW = smem_base + L.ring + s * kSplitStageBytes + (c & (kSplitStageChunks - 1)) * kSplitChunkBytes;
      if constexpr (WB == 16) {
        sp_k16<BF16, NT>(sW, smem_base + L.zs + (uint32_t)c * zbox, A.acc, lane);
      } else {
        const uint32_t sA = smem_base + L.zs + (uint32_t)c * kChunkAct;
        float ga = 0.f, ga8 = 0.f, gb = 0.f, gb8 = 0.f;
        if constexpr (GS) {
          const int m = g * 16 + gq, gi = c * (WB == 8 ? 1 : 2);
          const __half* srow = q.u_scale + ((long long)blk * Q + m) * ngroups;
          if (m < Q) ga = __half2float(__ldg(srow + gi));
          if (m + 8 < Q) ga8 = __half2float(__ldg(srow + 8 * ngroups + gi));
          if (WB == 4 && gi + 1 < ngroups) {
            if (m < Q) gb = __half2float(__ldg(srow + gi + 1));
            if (m + 8 < Q) gb8 = __half2float(__ldg(srow + 8 * ngroups + gi + 1));
          }
        }
        if constexpr (MG && WB == 8) {
          iq_k8_merged<0, 4>(sW, sA, zpitch, N, A.hi[0], lane);
          if constexpr (GS) A.fold(ga, ga8);
        } else if constexpr (MG && !GS) {
          iq_k4_merged<0, 4>(sW, sA, zpitch, N, A.hi[0], lane);
        } else if constexpr (MG) {
          iq_k4_merged<0, 2>(sW, sA, zpitch, N, A.hi[0], lane);
          A.fold(ga, ga8);
          iq_k4_merged<2, 4>(sW, sA, zpitch, N, A.hi[0], lane);
          A.fold(gb, gb8);
        } else if constexpr (WB == 8) {
          iq_k8<NT>(sW, sA, zpitch, N, A.hi, A.lo, lane);
          if constexpr (GS) A.fold(ga, ga8);
        } else if constexpr (!GS) {
          iq_k4<NT>(sW, sA, zpitch, N, A.hi, A.lo, lane);
        } else {
          iq_k4_half<NT>(sW, sA, zpitch, N, A.hi, A.lo, lane, 0);
          A.fold(ga, ga8);
          iq_k4_half<NT>(sW, sA, zpitch, N, A.hi, A.lo, lane, 2);
          A.fold(gb, gb8);
        }
      }
    };
    if (resident) {
#pragma unroll 1
      for (int gl = gw; gl < ng && ok; gl += kW) {
        A.clear();
        int s_seen = -1;
#pragma unroll 1
        for (int c = ws; c < nch; c += share) {
          const int s = gl * nseg + (c >> 3);
          if (s != s_seen) {
            if (!mbar_wait(full0 + 8 * s, 0, abort_flag)) { ok = false; break; }
            s_seen = s;
          }
          chunk(gl, c, (uint32_t)s);
        }
        flush(gl);
      }
    } else {
      RingPos rp;
#pragma unroll 1
      for (int gl = 0; gl < ng && ok; ++gl) {
        const bool mine = share == 1 ? (gl & (kW - 1)) == warp : gl == gw;
        int c = ws;  // this warp's next chunk of the group
        if (mine) A.clear();
#pragma unroll 1
        for (int seg = 0; seg < nseg; ++seg) {
          const uint32_t s = rp.s;
          if (!mbar_wait(full0 + 8 * s, rp.use_parity, abort_flag)) { ok = false; break; }
          if (mine) {
            const int c_end = min(nch, (seg + 1) * kSplitStageChunks);
#pragma unroll 1
            for (; c < c_end; c += share) chunk(gl, c, s);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(empty0 + 8 * s);
          rp.advance(NST);
        }
        if (mine && ok) flush(gl);
      }
    }
  }
  BLR_CK(8);
  named_bar(1, kCT);
  BLR_CK(9);
  BLR_TL(5);
  if (*abort_flag) {
    if (ctid == 0) atomicExch(p.status, 1u);
    return;
  }
  // ---- out[n][blk*Q + q] = scales * sum over the sharing warps' slots (fixed order); a thread takes two
  // neighbouring rows of a token, consecutive threads consecutive pairs
  {
    const int pairs_full = p.gpc * 8, rows = ng * 16;
    uint16_t* outp = reinterpret_cast<uint16_t*>(q.out);
#pragma unroll 1
    for (int e = ctid; e < pairs_full * N; e += kCT) {
      const int n = (int)fastdiv((uint32_t)e, (uint32_t)pairs_full, p.magic_rows), lr = (e - n * pairs_full) * 2;
      const int gl = lr >> 4, row = lr & 15, qq = g_lo * 16 + lr;
      if (lr >= rows || qq >= Q) continue;
      const float2* sp = reinterpret_cast<const float2*>(partial + (size_t)(gl * share) * 16 * NP + n * 16 + row);
      float s0 = sp[0].x, s1 = sp[0].y;
#pragma unroll 1
      for (int cs = 1; cs < share; ++cs) {
        const float2 v = sp[cs * 8 * NP];
        s0 += v.x;
        s1 += v.y;
      }
      s0 *= us[lr];
      s1 *= us[lr + 1];
      if constexpr (FX) {
        s0 *= sz[n];
        s1 *= sz[n];
      }
      if (p.out_interleaved) {  // Monarch's interleaved features: row s of block l is feature s * b + l
        const long long o0 = (long long)n * q.ldo + (long long)qq * p.bo + blk;
        store16<BF16>(q.out, o0, s0);
        if (qq + 1 < Q) store16<BF16>(q.out, o0 + p.bo, s1);
        continue;
      }
      const long long col = (long long)blk * Q + qq, o = (long long)n * q.ldo + col;
      const bool two = qq + 1 < Q;
      if (q.bias != nullptr) {
        s0 += load16<BF16>(q.bias, col);
        if (two) s1 += load16<BF16>(q.bias, col + 1);
      }
      if (q.residual != nullptr) {
        s0 += load16<BF16>(q.residual, (long long)n * q.ldr + col);
        if (two) s1 += load16<BF16>(q.residual, (long long)n * q.ldr + col + 1);
      }
      if (two && (o & 1) == 0) {
        *reinterpret_cast<uint32_t*>(outp + o) = pack16x2<BF16>(s0, s1);
      } else {
        store16<BF16>(q.out, o, s0);
        if (two) store16<BF16>(q.out, o + 1, s1);
      }
    }
  }
  BLR_CK(10);
  BLR_TL(6);
}

// ---------------------------------------------------------------------------------------------------- host side
template <bool BF16, int NT, bool GS, int WB, bool MG = false>
static int launch_split_impl(const SplitParams& p, cudaStream_t stream) {
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != BLR_OK) return rc;
  const size_t fs = split_front_smem(p), bs = split_back_smem(p);
  BLR_REQUIRE((int)fs <= di.max_smem_optin && (int)bs <= di.max_smem_optin, BLR_ERR_UNSUPPORTED,
              "needs %zu / %zu bytes of shared memory, device offers %d", fs, bs, di.max_smem_optin);
  const bool front_act = p.act == kSplitActSiluMul && p.xq == nullptr;
  auto front = front_act ? blr_blast_front_kernel<BF16, NT, GS, WB, true, MG> : blr_blast_front_kernel<BF16, NT, GS, WB, false, MG>;
  auto back = blr_blast_back_kernel<BF16, NT, GS, WB, MG>;
  {
    int dev = 0;
    BLR_CUDA_OK(cudaGetDevice(&dev));
    static bool configured[2][64] = {};  // per template instance and front variant
    bool& done = configured[front_act][dev & 63];
    if (!done) {
      BLR_CUDA_OK(cudaFuncSetAttribute(front, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem_optin));
      BLR_CUDA_OK(cudaFuncSetAttribute(back, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem_optin));
      done = true;
    }
  }
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
#ifdef BLR_TIMELINE
  SplitParams pf = p, pb = p;
  pf.timeline = pb.timeline = nullptr;
  if (g_split_timeline && g_split_timeline_next + 2 <= g_split_timeline_launches) {
    pf.timeline = g_split_timeline + (size_t)(g_split_timeline_next++) * 256 * 16;
    pb.timeline = g_split_timeline + (size_t)(g_split_timeline_next++) * 256 * 16;
  }
  void* args[] = {&pf};
  void* args_b[] = {&pb};
#else
  void* args[] = {const_cast<SplitParams*>(&p)};
  void** args_b = args;
#endif
  cudaLaunchConfig_t cfg = {};
  cfg.stream = stream;
  cfg.attrs = at;
  cfg.numAttrs = 1;
#ifdef BLR_TIMELINE
  if (getenv("BLR_NO_PDL")) cfg.numAttrs = 0;  // profiling builds only: launches fully serialised
#endif
  if constexpr (WB != 16) {
    if (p.xq != nullptr) {
      // x once for everybody (the input transform happens there, the front kernel then sees plain rows)
      auto fx = p.act == kSplitActSiluMul ? blr_blast_fx_kernel<BF16, WB, true> : blr_blast_fx_kernel<BF16, WB, false>;
      const size_t xs = (size_t)kW * fx_pitch(p.P, WB);
      if (xs > 48 * 1024) BLR_CUDA_OK(cudaFuncSetAttribute(fx, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)xs));
      cfg.gridDim = dim3((unsigned)((p.b * p.N + kW - 1) / kW));
      cfg.blockDim = dim3(kSplitFrontThreads);
      cfg.dynamicSmemBytes = xs;
      BLR_CUDA_OK(cudaLaunchKernelExC(&cfg, (const void*)fx, args));
    }
  }
  cfg.gridDim = dim3(p.R / kSplitRanks, p.nprob);
  cfg.blockDim = dim3(kSplitFrontThreads);
  cfg.dynamicSmemBytes = fs;
  BLR_CUDA_OK(cudaLaunchKernelExC(&cfg, (const void*)front, args));
  cfg.gridDim = dim3(p.bo * p.cpb, p.nprob);
  cfg.blockDim = dim3(kSplitBackThreads);
  cfg.dynamicSmemBytes = bs;
  BLR_CUDA_OK(cudaLaunchKernelExC(&cfg, (const void*)back, args_b));
  return BLR_OK;
}

int launch_blast_split(const SplitParams& p, int is_bf16, cudaStream_t stream) {
  BLR_REQUIRE(p.N >= 1 && p.N <= kStreamMaxTokens, BLR_ERR_UNSUPPORTED, "the two-launch decode path takes 1..%d tokens", kStreamMaxTokens);
  const bool gs = p.group != 0;
#define BLR_SP(BF, NTV, GSV)                                                        \
  (p.wbits == 16 ? launch_split_impl<BF, NTV, false, 16>(p, stream)                 \
                 : (p.wbits == 8 ? launch_split_impl<BF, NTV, GSV, 8>(p, stream) : launch_split_impl<BF, NTV, GSV, 4>(p, stream)))
  if (p.N <= 4 && p.wbits != 16) {
    // quantised factors, up to 4 tokens: both planes of the fixed-point activations in one integer MMA
#define BLR_SPM(BF, GSV) (p.wbits == 8 ? launch_split_impl<BF, 1, GSV, 8, true>(p, stream) : launch_split_impl<BF, 1, GSV, 4, true>(p, stream))
    if (gs) return is_bf16 ? BLR_SPM(true, true) : BLR_SPM(false, true);
    return is_bf16 ? BLR_SPM(true, false) : BLR_SPM(false, false);
#undef BLR_SPM
  }
  if (p.N <= 8) {
    if (gs) return is_bf16 ? BLR_SP(true, 1, true) : BLR_SP(false, 1, true);
    return is_bf16 ? BLR_SP(true, 1, false) : BLR_SP(false, 1, false);
  }
  if (gs) return is_bf16 ? BLR_SP(true, 2, true) : BLR_SP(false, 2, true);
  return is_bf16 ? BLR_SP(true, 2, false) : BLR_SP(false, 2, false);
#undef BLR_SP
}

}  // namespace blr

#ifdef BLR_TIMELINE
extern "C" int blr_debug_split_timeline(void* dev_ptr, int launches) {
  blr::g_split_timeline = static_cast<unsigned long long*>(dev_ptr);
  blr::g_split_timeline_launches = launches;
  blr::g_split_timeline_next = 0;
  return 0;
}
#endif
