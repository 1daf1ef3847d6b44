// The small kernels of a Llama-style decode step around the structured linears: RMSNorm, rotary embedding with the
// append to a static KV cache, and attention of one new token per sequence over the cache.  None of them has a
// counterpart among the reference's operator files: its network harness runs HuggingFace's modules for these
// (models/llama7b.py builds the model, network.py:60-94 times it), a dozen element-wise launches per layer each.
// Here a decoder layer is four structured-linear calls plus these four launches.
//
// All arithmetic is fp32 on 16-bit inputs, rounded once on the way out, like the PyTorch modules they stand in for.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/blr_b200.h"
#include "tmap.h"

namespace blr {

template <bool BF16>
__device__ __forceinline__ float2 up2(uint32_t w) {
  if constexpr (BF16) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  else return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <bool BF16>
__device__ __forceinline__ uint32_t down2(float a, float b) {
  if constexpr (BF16) {
    const __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&r);
  } else {
    const __half2 r = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&r);
  }
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_maxf(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ------------------------------------------------------------------------------------------------ RMSNorm
// out[r][:] = x[r][:] * rsqrt(mean(x[r][:]^2) + eps) * w[:].  One CTA per row, 16-byte accesses (d % 8 == 0).
template <bool BF16>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const uint16_t* __restrict__ x, long long ldx, const uint16_t* __restrict__ w,
                                                      float eps, int d, uint16_t* __restrict__ out, long long ldo) {
  __shared__ float red[8];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint16_t* xr = x + (long long)blockIdx.x * ldx;
  uint16_t* orow = out + (long long)blockIdx.x * ldo;
  const int pieces = d >> 3;
  float ss = 0.f;
  for (int p = threadIdx.x; p < pieces; p += 256) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + p * 8);
    const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = up2<BF16>(ws[i]);
      ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)d + eps);
  for (int p = threadIdx.x; p < pieces; p += 256) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + p * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(w + p * 8);
    const uint32_t vs[4] = {v.x, v.y, v.z, v.w}, gs[4] = {g.x, g.y, g.z, g.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = up2<BF16>(vs[i]), s = up2<BF16>(gs[i]);
      o[i] = down2<BF16>(f.x * inv * s.x, f.y * inv * s.y);
    }
    *reinterpret_cast<uint4*>(orow + p * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ------------------------------------------------------------------------------------------------ LayerNorm
// out[r][:] = (x[r][:] - mean) * rsqrt(var + eps) * w[:] + b[:]  (w, b optional; per group of rows_per_group rows when
// that is set, and 1 + w in place of w with w_plus_one: adaLN modulation).  A warp per row, the row in registers
// (up to 8 pieces of 8 values per lane: d <= 2048, d % 8 == 0), mean and variance in two passes over the registers.
template <bool BF16, int NP, int MINB>
__global__ void __launch_bounds__(256, MINB) layernorm_kernel(const uint16_t* __restrict__ x, long long ldx, const uint16_t* __restrict__ w,
                                                              const uint16_t* __restrict__ b, float eps, int d, long long rows,
                                                              uint16_t* __restrict__ out, long long ldo, long long rows_per_group,
                                                              long long ldw, long long ldb, int w_plus_one) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= rows) return;
  if (rows_per_group > 0) {  // weight and bias per group of consecutive rows (a modulation per image)
    const long long grp = r / rows_per_group;
    if (w != nullptr) w += grp * ldw;
    if (b != nullptr) b += grp * ldb;
  }
  const float w_add = w_plus_one ? 1.f : 0.f;
  const int lane = threadIdx.x & 31, pieces = d >> 3;
  const uint16_t* xr = x + r * ldx;
  // The row stays packed (NP 16-byte pieces per lane) so that enough warps fit an SM to keep the loads of several rows
  // in flight while others reduce and store; the three passes widen it again.
  uint4 t[NP];
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const int p = lane + 32 * i;
    t[i] = p < pieces ? *reinterpret_cast<const uint4*>(xr + p * 8) : make_uint4(0, 0, 0, 0);
  }
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const uint32_t ws[4] = {t[i].x, t[i].y, t[i].z, t[i].w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = up2<BF16>(ws[k]);
      sum += f.x + f.y;
    }
  }
  const float mean = warp_sum(sum) / (float)d;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < NP; ++i)
    if (lane + 32 * i < pieces) {
      const uint32_t ws[4] = {t[i].x, t[i].y, t[i].z, t[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = up2<BF16>(ws[k]);
        const float c0 = f.x - mean, c1 = f.y - mean;
        sq = fmaf(c0, c0, sq);
        sq = fmaf(c1, c1, sq);
      }
    }
  const float inv = rsqrtf(warp_sum(sq) / (float)d + eps);
  uint16_t* orow = out + r * ldo;
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const int p = lane + 32 * i;
    if (p < pieces) {
      uint4 gw = make_uint4(0, 0, 0, 0), hb = make_uint4(0, 0, 0, 0);
      if (w != nullptr) gw = *reinterpret_cast<const uint4*>(w + p * 8);
      if (b != nullptr) hb = *reinterpret_cast<const uint4*>(b + p * 8);
      const uint32_t ws[4] = {t[i].x, t[i].y, t[i].z, t[i].w}, gs[4] = {gw.x, gw.y, gw.z, gw.w}, hs[4] = {hb.x, hb.y, hb.z, hb.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = up2<BF16>(ws[k]);
        float2 g = make_float2(1.f, 1.f), h = make_float2(0.f, 0.f);
        if (w != nullptr) {
          g = up2<BF16>(gs[k]);
          g.x += w_add, g.y += w_add;
        }
        if (b != nullptr) h = up2<BF16>(hs[k]);
        o[k] = down2<BF16>(fmaf((f.x - mean) * inv, g.x, h.x), fmaf((f.y - mean) * inv, g.y, h.y));
      }
      *reinterpret_cast<uint4*>(orow + p * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ gated residual
// out[r][:] = x[r][:] + gate[r / rows_per_group][:] * y[r][:]: 16-byte accesses, one thread per 8 values.
template <bool BF16>
__global__ void __launch_bounds__(256) gated_add_kernel(const uint16_t* __restrict__ x, long long ldx, const uint16_t* __restrict__ y,
                                                        long long ldy, const uint16_t* __restrict__ gate, long long ldg,
                                                        long long rows_per_group, int d, long long total, uint16_t* __restrict__ out,
                                                        long long ldo) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const long long id = (long long)blockIdx.x * 256 + threadIdx.x;
  if (id >= total) return;
  const int pieces = d >> 3;
  const long long r = id / pieces;
  const int p = (int)(id - r * pieces);
  const uint4 a = *reinterpret_cast<const uint4*>(x + r * ldx + p * 8);
  const uint4 c = *reinterpret_cast<const uint4*>(y + r * ldy + p * 8);
  const uint4 g = *reinterpret_cast<const uint4*>(gate + (r / rows_per_group) * ldg + p * 8);
  const uint32_t as[4] = {a.x, a.y, a.z, a.w}, cs[4] = {c.x, c.y, c.z, c.w}, gs[4] = {g.x, g.y, g.z, g.w};
  uint32_t o[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 fa = up2<BF16>(as[k]), fc = up2<BF16>(cs[k]), fg = up2<BF16>(gs[k]);
    o[k] = down2<BF16>(fmaf(fg.x, fc.x, fa.x), fmaf(fg.y, fc.y, fa.y));
  }
  *reinterpret_cast<uint4*>(out + r * ldo + p * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

// ------------------------------------------------------------------------------------------------ rotary embedding + cache append
// Row r = (sequence b, token t) of q, k, v (rows of H * hd values, row strides ldq / ldk / ldv).  Pairs (i, i + hd/2) of
// every head of q and k are rotated by the angle of cache slot pos[t] (cos, sin tables (slots, hd/2), fp32); q is
// rewritten in place, the rotated k and v go to kc / vc [b][h][pos[t]][:] (caches (B, H, slots, hd)).
template <bool BF16>
__global__ void __launch_bounds__(256) rope_append_kernel(uint16_t* __restrict__ q, long long ldq, const uint16_t* __restrict__ k,
                                                          long long ldk, const uint16_t* __restrict__ v, long long ldv,
                                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                          const long long* __restrict__ pos, int T, int H, int hd, int slots,
                                                          uint16_t* __restrict__ kc, uint16_t* __restrict__ vc) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int r = blockIdx.x, b = r / T, t = r - b * T, half = hd >> 1;
  const long long slot = pos[t];
  const float* cs = cos_t + slot * half;
  const float* sn = sin_t + slot * half;
  uint16_t* qr = q + (long long)r * ldq;
  const uint16_t* kr = k + (long long)r * ldk;
  const uint16_t* vr = v + (long long)r * ldv;
  // two values per thread and step: pair index i = 2 u, 2 u + 1 of head h
  const int per_head = half >> 1;
  for (int e = threadIdx.x; e < H * per_head; e += 256) {
    const int h = e / per_head, i = (e - h * per_head) * 2;
    const float c0 = cs[i], c1 = cs[i + 1], s0 = sn[i], s1 = sn[i + 1];
    const long long o1 = (long long)h * hd + i, o2 = o1 + half;
    const long long dst = (((long long)b * H + h) * slots + slot) * hd;
    {
      const float2 a = up2<BF16>(*reinterpret_cast<const uint32_t*>(qr + o1)), bb = up2<BF16>(*reinterpret_cast<const uint32_t*>(qr + o2));
      *reinterpret_cast<uint32_t*>(qr + o1) = down2<BF16>(a.x * c0 - bb.x * s0, a.y * c1 - bb.y * s1);
      *reinterpret_cast<uint32_t*>(qr + o2) = down2<BF16>(bb.x * c0 + a.x * s0, bb.y * c1 + a.y * s1);
    }
    {
      const float2 a = up2<BF16>(*reinterpret_cast<const uint32_t*>(kr + o1)), bb = up2<BF16>(*reinterpret_cast<const uint32_t*>(kr + o2));
      *reinterpret_cast<uint32_t*>(kc + dst + i) = down2<BF16>(a.x * c0 - bb.x * s0, a.y * c1 - bb.y * s1);
      *reinterpret_cast<uint32_t*>(kc + dst + half + i) = down2<BF16>(bb.x * c0 + a.x * s0, bb.y * c1 + a.y * s1);
    }
    *reinterpret_cast<uint32_t*>(vc + dst + i) = *reinterpret_cast<const uint32_t*>(vr + o1);
    *reinterpret_cast<uint32_t*>(vc + dst + half + i) = *reinterpret_cast<const uint32_t*>(vr + o2);
  }
}

// ------------------------------------------------------------------------------------------------ attention of one token over the cache
// CTA (split, head, sequence): keys [k0, k0 + ks) of the head's cache.  A key (and value) row of hd 16-bit values is
// read by hd / 8 neighbouring lanes, 16 bytes each, so a warp's load covers whole rows back to back; a lane keeps its
// 8 values of q in registers.  One pass with a running maximum per row slot (a warp's position in its load): the dot
// product is reduced over the row's lanes by shuffles, the slot's sum and its 8 output dimensions per lane are rescaled
// when the maximum moves; the slots' (maximum, sum, output) meet in shared memory at the end.  Partial result (unnormalised output, maximum, sum) per split; the combine kernel merges the
// splits of a head.  hd / 8 must divide 32 (hd = 8, 16, 32, 64, 128 or 256).
static constexpr int kAttnThreads = 256;

template <bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 3) attn_decode_partial_kernel(const uint16_t* __restrict__ q, long long ldq,
                                                                         const uint16_t* __restrict__ kc, const uint16_t* __restrict__ vc,
                                                                         int H, int hd, int slots, int n_keys, int ks, float scale,
                                                                         float* __restrict__ part) {
  extern __shared__ float sm[];  // per slot (warp, key of the warp's load): maximum, sum | acc[slot][hd]
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lpk = hd >> 3, kpw = 32 / lpk, sub = lane / lpk, piece = lane - sub * lpk;
  const int nslot = (kAttnThreads / 32) * kpw;
  float* ml = sm;               // [nslot][2]
  float* accs = sm + 2 * nslot;  // [nslot][hd]
  const int k0 = split * ks, nk = min(ks, n_keys - k0), kstep = (kAttnThreads / 32) * kpw;
  const uint16_t* kh = kc + (((long long)b * H + h) * slots + k0) * hd + piece * 8;
  const uint16_t* vh = vc + (((long long)b * H + h) * slots + k0) * hd + piece * 8;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  float qf[8];
  {
    const uint4 v = *reinterpret_cast<const uint4*>(q + (long long)b * ldq + (long long)h * hd + piece * 8);
    const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = up2<BF16>(ws[i]);
      qf[2 * i] = f.x * scale;
      qf[2 * i + 1] = f.y * scale;
    }
  }
  // ---- one pass over the keys with a running maximum: the key and the value row of a step are loaded together, so
  // both streams are in flight all the time and nothing waits at a barrier between them
  float m = -3.0e38f, l = 0.f;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  constexpr int kAhead = 4;  // steps whose key and value rows are requested before the first is used
#pragma unroll 1
  for (int j0 = warp * kpw; j0 < nk; j0 += kAhead * kstep) {  // warp-uniform bounds
    uint4 kv[kAhead], vv[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int j = j0 + u * kstep + sub;
      kv[u] = vv[u] = make_uint4(0, 0, 0, 0);
      if (j < nk) {
        kv[u] = *reinterpret_cast<const uint4*>(kh + (long long)j * hd);
        vv[u] = *reinterpret_cast<const uint4*>(vh + (long long)j * hd);
      }
    }
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int j = j0 + u * kstep + sub;
      float s = 0.f;
      {
        const uint32_t ws[4] = {kv[u].x, kv[u].y, kv[u].z, kv[u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = up2<BF16>(ws[i]);
          s = fmaf(f.x, qf[2 * i], fmaf(f.y, qf[2 * i + 1], s));
        }
      }
      for (int o = lpk >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (j < nk) {
        const float mn = fmaxf(m, s), corr = __expf(m - mn), p = __expf(s - mn);
        m = mn;
        l = fmaf(l, corr, p);
        const uint32_t ws[4] = {vv[u].x, vv[u].y, vv[u].z, vv[u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = up2<BF16>(ws[i]);
          acc[2 * i] = fmaf(acc[2 * i], corr, p * f.x);
          acc[2 * i + 1] = fmaf(acc[2 * i + 1], corr, p * f.y);
        }
      }
    }
  }
  // slot (warp, sub): maximum, sum and the partial output over all hd dimensions
  {
    const int slot = warp * kpw + sub;
    if (piece == 0) {
      ml[2 * slot] = m;
      ml[2 * slot + 1] = l;
    }
    float* a = accs + (slot * hd + piece * 8);
    *reinterpret_cast<float4*>(a) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(a + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  __syncthreads();
  float M = -3.0e38f;
  for (int g = 0; g < nslot; ++g) M = fmaxf(M, ml[2 * g]);
  float* dst = part + (((long long)b * H + h) * gridDim.x + split) * (hd + 2);
  for (int d = tid; d < hd; d += kAttnThreads) {
    float o = 0.f;
    for (int g = 0; g < nslot; ++g) o = fmaf(accs[g * hd + d], __expf(ml[2 * g] - M), o);  // (empty slots: 0 * exp(0))
    dst[d] = o;
  }
  if (tid == 0) {
    float lt = 0.f;
    for (int g = 0; g < nslot; ++g) lt = fmaf(ml[2 * g + 1], __expf(ml[2 * g] - M), lt);
    dst[hd] = M;
    dst[hd + 1] = lt;
  }
}

template <bool BF16>
__global__ void __launch_bounds__(128) attn_decode_combine_kernel(const float* __restrict__ part, int nsplit, int hd, uint16_t* __restrict__ out,
                                                                  long long ldo, int H) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int h = blockIdx.x, b = blockIdx.y;
  const float* p0 = part + (((long long)b * H + h) * nsplit) * (hd + 2);
  float m = -3.0e38f;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, p0[s * (hd + 2) + hd]);
  float L = 0.f;
  for (int s = 0; s < nsplit; ++s) L += p0[s * (hd + 2) + hd + 1] * __expf(p0[s * (hd + 2) + hd] - m);
  const float invL = 1.f / L;
  for (int dp = threadIdx.x; dp < hd / 2; dp += 128) {
    float ox = 0.f, oy = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float w = __expf(p0[s * (hd + 2) + hd] - m);
      ox = fmaf(w, p0[s * (hd + 2) + 2 * dp], ox);
      oy = fmaf(w, p0[s * (hd + 2) + 2 * dp + 1], oy);
    }
    *reinterpret_cast<uint32_t*>(out + (long long)b * ldo + (long long)h * hd + 2 * dp) = down2<BF16>(ox * invL, oy * invL);
  }
}

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

// Splits of a head's keys.  Three CTAs share an SM, so the grid runs in waves of 3 x 148 CTAs and a wave that is
// nearly empty costs as much as a full one (16 sequences x 32 heads in one split each are 1.15 waves: 3.8 TB/s).
// Among 1..16 splits of at least 128 keys, take the one with the smallest waves x (keys per CTA + a CTA's fixed cost,
// about the time of 96 keys).
static int attn_splits(int64_t B, int H, int n_keys) {
  const int64_t wave = 3 * 148;
  int best = 1;
  int64_t best_cost = -1;
  for (int ns = 1; ns <= 16; ++ns) {
    const int keys = (n_keys + ns - 1) / ns;
    if (ns > 1 && keys < 128) break;
    const int64_t waves = (B * H * ns + wave - 1) / wave, cost = waves * (keys + 96);
    if (best_cost < 0 || cost < best_cost) best = ns, best_cost = cost;
  }
  return best;
}

}  // namespace blr

using namespace blr;

extern "C" {

int blr_rmsnorm(const void* x, int64_t ldx, int64_t rows, int d, const void* weight, float eps, int dtype, void* out, int64_t ldo,
                void* stream) {
  BLR_REQUIRE(rows >= 0 && d > 0 && d % 8 == 0 && ldx % 8 == 0 && ldo % 8 == 0, BLR_ERR_ARG,
              "rmsnorm needs d, ldx and ldo to be multiples of 8 (d = %d)", d);
  BLR_REQUIRE(dtype == BLR_DTYPE_F16 || dtype == BLR_DTYPE_BF16, BLR_ERR_ARG, "unknown dtype %d", dtype);
  if (rows == 0) return BLR_OK;
  BLR_REQUIRE(x != nullptr && weight != nullptr && out != nullptr, BLR_ERR_ARG, "null pointer");
  BLR_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) & 15) == 0, BLR_ERR_ARG,
              "rmsnorm needs 16-byte aligned pointers");
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  const uint16_t* wp = static_cast<const uint16_t*>(weight);
  uint16_t* op = static_cast<uint16_t*>(out);
  const long long lx = ldx, lo = ldo;
  if (dtype == BLR_DTYPE_BF16) return launch_pdl(rmsnorm_kernel<true>, dim3((unsigned)rows), dim3(256), 0, st, xp, lx, wp, eps, d, op, lo);
  return launch_pdl(rmsnorm_kernel<false>, dim3((unsigned)rows), dim3(256), 0, st, xp, lx, wp, eps, d, op, lo);
}

int blr_gated_add(const void* x, int64_t ldx, const void* y, int64_t ldy, const void* gate, int64_t ldg, int64_t rows,
                  int64_t rows_per_group, int d, int dtype, void* out, int64_t ldo, void* stream) {
  BLR_REQUIRE(rows >= 0 && rows_per_group > 0 && d > 0 && d % 8 == 0 && ldx % 8 == 0 && ldy % 8 == 0 && ldg % 8 == 0 && ldo % 8 == 0,
              BLR_ERR_ARG, "gated_add needs d and the row strides to be multiples of 8 (d = %d)", d);
  BLR_REQUIRE(dtype == BLR_DTYPE_F16 || dtype == BLR_DTYPE_BF16, BLR_ERR_ARG, "unknown dtype %d", dtype);
  if (rows == 0) return BLR_OK;
  BLR_REQUIRE(x && y && gate && out, BLR_ERR_ARG, "null pointer");
  BLR_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(gate) |
                reinterpret_cast<uintptr_t>(out)) & 15) == 0, BLR_ERR_ARG, "gated_add needs 16-byte aligned pointers");
  const long long total = rows * (d >> 3);
  BLR_REQUIRE((total + 255) / 256 < (1ll << 31), BLR_ERR_SHAPE, "too many rows");
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  const uint16_t* yp = static_cast<const uint16_t*>(y);
  const uint16_t* gp = static_cast<const uint16_t*>(gate);
  uint16_t* op = static_cast<uint16_t*>(out);
  const long long lx = ldx, ly = ldy, lg = ldg, lo = ldo, rpg = rows_per_group;
  const dim3 grid((unsigned)((total + 255) / 256));
  if (dtype == BLR_DTYPE_BF16) return launch_pdl(gated_add_kernel<true>, grid, dim3(256), 0, st, xp, lx, yp, ly, gp, lg, rpg, d, total, op, lo);
  return launch_pdl(gated_add_kernel<false>, grid, dim3(256), 0, st, xp, lx, yp, ly, gp, lg, rpg, d, total, op, lo);
}

int blr_layernorm(const void* x, int64_t ldx, int64_t rows, int d, const void* weight, const void* bias, float eps, int dtype, void* out,
                  int64_t ldo, int64_t rows_per_group, int64_t ldw, int64_t ldb, int weight_plus_one, void* stream) {
  BLR_REQUIRE(rows_per_group >= 0 && (rows_per_group == 0 || (ldw % 8 == 0 && ldb % 8 == 0)), BLR_ERR_ARG,
              "layernorm: per-group weights need row strides that are multiples of 8");
  BLR_REQUIRE(rows >= 0 && d > 0 && d % 8 == 0 && ldx % 8 == 0 && ldo % 8 == 0, BLR_ERR_ARG,
              "layernorm needs d, ldx and ldo to be multiples of 8 (d = %d)", d);
  BLR_REQUIRE(d <= 2048, BLR_ERR_UNSUPPORTED, "layernorm keeps a row in a warp's registers: d <= 2048, got %d", d);
  BLR_REQUIRE(dtype == BLR_DTYPE_F16 || dtype == BLR_DTYPE_BF16, BLR_ERR_ARG, "unknown dtype %d", dtype);
  if (rows == 0) return BLR_OK;
  BLR_REQUIRE(x && out, BLR_ERR_ARG, "null pointer");
  BLR_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(weight) |
                reinterpret_cast<uintptr_t>(bias)) & 15) == 0, BLR_ERR_ARG, "layernorm needs 16-byte aligned pointers");
  BLR_REQUIRE((rows + 7) / 8 < (1ll << 31), BLR_ERR_SHAPE, "too many rows");
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  const uint16_t* wp = static_cast<const uint16_t*>(weight);
  const uint16_t* bp = static_cast<const uint16_t*>(bias);
  uint16_t* op = static_cast<uint16_t*>(out);
  const long long lx = ldx, lo = ldo, nr = rows, rpg = rows_per_group, lw = ldw, lb = ldb;
  const dim3 grid((unsigned)((rows + 7) / 8));
  auto go = [&](auto kernel) { return launch_pdl(kernel, grid, dim3(256), 0, st, xp, lx, wp, bp, eps, d, nr, op, lo, rpg, lw, lb, weight_plus_one); };
  const bool bf = dtype == BLR_DTYPE_BF16;
  // pieces per lane by width: 3 (d <= 768), 5 (<= 1280), 8 (<= 2048), each with the occupancy its registers allow
  if (d <= 768) return bf ? go(layernorm_kernel<true, 3, 5>) : go(layernorm_kernel<false, 3, 5>);
  if (d <= 1280) return bf ? go(layernorm_kernel<true, 5, 4>) : go(layernorm_kernel<false, 5, 4>);
  return bf ? go(layernorm_kernel<true, 8, 3>) : go(layernorm_kernel<false, 8, 3>);
}

int blr_rope_append(void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, const float* cos_table,
                    const float* sin_table, const int64_t* pos, int64_t n_seq, int n_tok, int heads, int head_dim, int slots, int dtype,
                    void* k_cache, void* v_cache, void* stream) {
  BLR_REQUIRE(n_seq >= 0 && n_tok > 0 && heads > 0 && head_dim > 0 && head_dim % 4 == 0 && slots > 0, BLR_ERR_ARG,
              "rope_append: head_dim must be a multiple of 4 (got %d)", head_dim);
  BLR_REQUIRE(dtype == BLR_DTYPE_F16 || dtype == BLR_DTYPE_BF16, BLR_ERR_ARG, "unknown dtype %d", dtype);
  BLR_REQUIRE(ldq % 2 == 0 && ldk % 2 == 0 && ldv % 2 == 0, BLR_ERR_ARG, "rope_append: row strides must be even");
  if (n_seq == 0) return BLR_OK;
  BLR_REQUIRE(q && k && v && cos_table && sin_table && pos && k_cache && v_cache, BLR_ERR_ARG, "null pointer");
  BLR_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 3) == 0, BLR_ERR_ARG,
              "rope_append needs 4-byte aligned pointers");
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint16_t* qp = static_cast<uint16_t*>(q);
  const uint16_t* kp = static_cast<const uint16_t*>(k);
  const uint16_t* vp = static_cast<const uint16_t*>(v);
  uint16_t* kcp = static_cast<uint16_t*>(k_cache);
  uint16_t* vcp = static_cast<uint16_t*>(v_cache);
  const long long lq = ldq, lk = ldk, lv = ldv;
  const long long* pp = reinterpret_cast<const long long*>(pos);
  const dim3 grid((unsigned)(n_seq * n_tok));
  if (dtype == BLR_DTYPE_BF16)
    return launch_pdl(rope_append_kernel<true>, grid, dim3(256), 0, st, qp, lq, kp, lk, vp, lv, cos_table, sin_table, pp, n_tok, heads, head_dim, slots, kcp, vcp);
  return launch_pdl(rope_append_kernel<false>, grid, dim3(256), 0, st, qp, lq, kp, lk, vp, lv, cos_table, sin_table, pp, n_tok, heads, head_dim, slots, kcp, vcp);
}

size_t blr_attention_decode_scratch_bytes(int64_t n_seq, int heads, int head_dim, int n_keys) {
  if (n_seq <= 0 || heads <= 0 || head_dim <= 0 || n_keys <= 0) return 0;
  return (size_t)n_seq * heads * attn_splits(n_seq, heads, n_keys) * (head_dim + 2) * sizeof(float);
}

int blr_attention_decode(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, int64_t n_seq, int heads, int head_dim,
                         int slots, int n_keys, float scale, int dtype, void* out, int64_t ldo, void* scratch, size_t scratch_bytes,
                         void* stream) {
  BLR_REQUIRE(n_seq >= 0 && heads > 0 && head_dim >= 8 && head_dim <= 256 && (head_dim & (head_dim - 1)) == 0 && slots > 0 && n_keys > 0 &&
                  n_keys <= slots,
              BLR_ERR_ARG, "attention_decode: head_dim must be a power of two from 8 to 256 and 1 <= n_keys <= slots");
  BLR_REQUIRE(dtype == BLR_DTYPE_F16 || dtype == BLR_DTYPE_BF16, BLR_ERR_ARG, "unknown dtype %d", dtype);
  BLR_REQUIRE(ldq % 8 == 0 && ldo % 2 == 0, BLR_ERR_ARG, "attention_decode: ldq must be a multiple of 8, ldo even");
  if (n_seq == 0) return BLR_OK;
  BLR_REQUIRE(q && k_cache && v_cache && out && scratch, BLR_ERR_ARG, "null pointer");
  BLR_REQUIRE(scratch_bytes >= blr_attention_decode_scratch_bytes(n_seq, heads, head_dim, n_keys), BLR_ERR_WORKSPACE,
              "attention_decode: scratch of %zu bytes is too small", scratch_bytes);
  BLR_REQUIRE(((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(q) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0, BLR_ERR_ARG,
              "attention_decode needs 16-byte aligned caches and q, 4-byte aligned out");
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int ns = attn_splits(n_seq, heads, n_keys), ks = (n_keys + ns - 1) / ns;
  const int nslot = (kAttnThreads / 32) * (32 / (head_dim >> 3));
  const size_t smem = (size_t)nslot * (head_dim + 2) * sizeof(float);  // 8 KB + 2 floats per slot for every head size
  const uint16_t* qp = static_cast<const uint16_t*>(q);
  const uint16_t* kp = static_cast<const uint16_t*>(k_cache);
  const uint16_t* vp = static_cast<const uint16_t*>(v_cache);
  uint16_t* op = static_cast<uint16_t*>(out);
  float* part = static_cast<float*>(scratch);
  const long long lq = ldq, lo = ldo;
  const dim3 grid((unsigned)ns, (unsigned)heads, (unsigned)n_seq);
  int rc;
  if (dtype == BLR_DTYPE_BF16) {
    if (smem > 48 * 1024) BLR_CUDA_OK(cudaFuncSetAttribute(attn_decode_partial_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    rc = launch_pdl(attn_decode_partial_kernel<true>, grid, dim3(kAttnThreads), smem, st, qp, lq, kp, vp, heads, head_dim, slots, n_keys, ks, scale, part);
    if (rc) return rc;
    return launch_pdl(attn_decode_combine_kernel<true>, dim3((unsigned)heads, (unsigned)n_seq), dim3(128), 0, st, (const float*)part, ns, head_dim, op, lo, heads);
  }
  if (smem > 48 * 1024) BLR_CUDA_OK(cudaFuncSetAttribute(attn_decode_partial_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  rc = launch_pdl(attn_decode_partial_kernel<false>, grid, dim3(kAttnThreads), smem, st, qp, lq, kp, vp, heads, head_dim, slots, n_keys, ks, scale, part);
  if (rc) return rc;
  return launch_pdl(attn_decode_combine_kernel<false>, dim3((unsigned)heads, (unsigned)n_seq), dim3(128), 0, st, (const float*)part, ns, head_dim, op, lo, heads);
}

}  // extern "C"
