// Weight-streaming kernel for decode-size token counts (N <= 16) on sm_100a.
//
// One persistent CTA per SM.  Two single-thread producers feed a ring of shared-memory stages with
// TMA tile loads: one streams weight tiles (it never waits for anything but a free stage, so HBM
// stays busy across the grid barriers), the other streams the matching activation boxes (it waits
// at the grid barrier before it touches activations written by other CTAs).  A stage holds up to
// 128 weight rows for one K-chunk; each of the eight consumer warps owns one 16-row group of them
// for the whole K loop, so the products (mma.sync m16n8k16, weights as the 16-row
// operand, tokens as the 8-column operand; int8 / int4 weights are widened in registers right
// before the MMA) accumulate in registers and are written straight from them.
// Every CTA walks the K-chunks of its tiles starting at a different offset, so that the CTAs do not
// all pull the same address window of every weight row at the same time.
#include <stdlib.h>

#include "ptx.cuh"
#include "stream.h"
#include "stream_device.cuh"
#include "tmap.h"

namespace blr {

struct Batch {
  int g, mt0, nt;  // block, first unit within the block, number of units
};

__device__ __forceinline__ bool next_batch(const PhaseDesc& ph, int& t, int t_hi, Batch& b) {
  if (t >= t_hi) return false;
  b.g = t / ph.tiles_per_g;
  b.mt0 = t - b.g * ph.tiles_per_g;
  const int end = min(t_hi, (b.g + 1) * ph.tiles_per_g);
  b.nt = min(kBatchRows / ph.unit_rows, end - t);
  t += b.nt;
  return true;
}
__device__ __forceinline__ void tile_range(const PhaseDesc& ph, int& lo, int& hi) {
  lo = (int)(((long long)ph.ntiles * blockIdx.x) / gridDim.x);
  hi = (int)(((long long)ph.ntiles * (blockIdx.x + 1)) / gridDim.x);
}
// First K-chunk this CTA visits (it then walks the chunks cyclically).  The producer and consumer loops
// are single-warp scalar code, so they keep ring slot, phase bit and chunk index incrementally:
// a division per stage would cost more cycles than the stage's data takes to arrive.
__device__ __forceinline__ int first_chunk(const PhaseDesc& ph) {
  return (int)((blockIdx.x * 5u) % (unsigned)ph.nstage_chunks);
}

// Share of the (n, r) plane this CTA couples: [lo, hi) in units of 8 consecutive r.
__device__ __forceinline__ void couple_range(const StreamParams& p, int& lo, int& hi) {
  const int nvec = (int)(((long long)p.N * p.R) >> 3);
  lo = (int)(((long long)nvec * blockIdx.x) / gridDim.x);
  hi = (int)(((long long)nvec * (blockIdx.x + 1)) / gridDim.x);
}
__device__ __forceinline__ bool couple_vectorised(const StreamParams& p) {
  return p.s_r == 1 && (p.R & 7) == 0 && (p.s_i & 7) == 0 && (p.s_j & 7) == 0 && p.b <= 16;
}
// The coupling factors of a thread's first work item: S does not depend on the grid barrier, so they are
// fetched before the thread waits at it.
struct CoupleRegs {
  uint4 s[16];
};
__device__ __forceinline__ void couple_item(const StreamParams& p, int e, int nv, int lo, int& i, long long& pt, int& r) {
  const int v = e % nv;
  i = e / nv;
  pt = (long long)(lo + v) << 3;
  r = (int)(pt % p.R);
}
__device__ __forceinline__ void couple_preload(const StreamParams& p, int ctid, CoupleRegs& cr) {
  if (!couple_vectorised(p)) return;
  int lo, hi;
  couple_range(p, lo, hi);
  const int nv = hi - lo;
  if (ctid >= nv * p.b_out) return;
  int i, r;
  long long pt;
  couple_item(p, ctid, nv, lo, i, pt, r);
#pragma unroll
  for (int j = 0; j < 16; ++j)
    if (j < p.b) cr.s[j] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.S) + i * p.s_i + j * p.s_j + r));
}

// BLAST coupling z[i][n][r] = sum_j S[i][j][r] * y[j][n][r] for this CTA's share of the (n, r) points.
// y was written by other CTAs before the grid barrier (the acquire at the barrier makes plain loads see
// it).  The CTA first copies its slice of y into shared memory (ybuf, [b][nv] vectors of 8 floats), so
// that the b threads sharing a y vector read it from there, and every global load of the phase is
// issued in one go.
template <bool BF16>
__device__ __forceinline__ void couple(const StreamParams& p, int ctid, const CoupleRegs& cr, float4* ybuf) {
  const long long plane = (long long)p.N * p.R;
  const int bb = p.b;
  int lo, hi;
  couple_range(p, lo, hi);
  if (couple_vectorised(p) && (long long)bb * (hi - lo) * 32 <= p.mix_bytes) {
    const int nv = hi - lo, nq = nv * 2;  // float4 per in-block
    const float* ysrc = p.y32 + ((long long)lo << 3);
    for (int e = ctid; e < bb * nq; e += kConsumerWarps * 32) {
      const int j = e / nq, q = e - j * nq;
      ybuf[e] = *reinterpret_cast<const float4*>(ysrc + j * plane + q * 4);
    }
    consumer_bar();
    for (int e = ctid; e < nv * p.b_out; e += kConsumerWarps * 32) {
      int i, r;
      long long pt;
      couple_item(p, e, nv, lo, i, pt, r);
      const int v = e % nv;
      float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      const bool pre = e == ctid;  // first item: factors already in registers
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (j < bb) {
          uint4 w;
          if (pre) w = cr.s[j];
          else w = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.S) + i * p.s_i + j * p.s_j + r));
          const float4 ya = ybuf[(j * nv + v) * 2], yb = ybuf[(j * nv + v) * 2 + 1];
          const float2 s0 = unpack16x2<BF16>(w.x), s1 = unpack16x2<BF16>(w.y), s2 = unpack16x2<BF16>(w.z), s3 = unpack16x2<BF16>(w.w);
          s[0] = fmaf(s0.x, ya.x, s[0]); s[1] = fmaf(s0.y, ya.y, s[1]);
          s[2] = fmaf(s1.x, ya.z, s[2]); s[3] = fmaf(s1.y, ya.w, s[3]);
          s[4] = fmaf(s2.x, yb.x, s[4]); s[5] = fmaf(s2.y, yb.y, s[5]);
          s[6] = fmaf(s3.x, yb.z, s[6]); s[7] = fmaf(s3.y, yb.w, s[7]);
        }
      }
      if (p.round_z) {
#pragma unroll
        for (int k = 0; k < 8; ++k) s[k] = round_clamp_i8(s[k]);
      }
      uint4 o;
      o.x = pack16x2<BF16>(s[0], s[1]); o.y = pack16x2<BF16>(s[2], s[3]);
      o.z = pack16x2<BF16>(s[4], s[5]); o.w = pack16x2<BF16>(s[6], s[7]);
      *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.z16) + i * plane + pt) = o;
    }
  } else {
    // generic strides (e.g. S stored (R, b_out, b_in)): one thread per (point, out block)
    const int NR = (int)plane;
    const int plo = (int)(((long long)NR * blockIdx.x) / gridDim.x);
    const int phi = (int)(((long long)NR * (blockIdx.x + 1)) / gridDim.x);
    const int npts = phi - plo;
    const int bo = p.b_out;
    for (int e = ctid; e < npts * bo; e += kConsumerWarps * 32) {
      const int i = e % bo, nr = plo + e / bo, r = nr % p.R;
      float s = 0.f;
#pragma unroll 8
      for (int j = 0; j < bb; ++j)
        s = fmaf(load16<BF16>(p.S, i * p.s_i + j * p.s_j + r * p.s_r), p.y32[j * plane + nr], s);
      if (p.round_z) s = round_clamp_i8(s);
      store16<BF16>(p.z16, i * plane + nr, s);
    }
  }
}

// ------------------------------------------------------------------ kernel
template <bool BF16, int NT, bool GS>
__global__ void __launch_bounds__(kStreamThreads, 1) blr_stream_kernel(const __grid_constant__ StreamParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // Carve: [stages][barriers]
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t NST = p.nstages, stage_bytes = p.stage_bytes;
  float4* ybuf = reinterpret_cast<float4*>(smem + (size_t)NST * stage_bytes);                       // coupling scratch
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)NST * stage_bytes + p.mix_bytes);  // full[16], empty[16]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * 16);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kABoxBytes = NT * 8 * 128;
  // optional per-CTA time stamps (16 slots per CTA) for profiling runs
#ifdef BLR_TIMELINE  // profiling builds only: 16 time stamps per CTA
  unsigned long long* tl = p.timeline ? p.timeline + (size_t)blockIdx.x * 16 : nullptr;
#define BLR_STAMP(slot) do { if (tl) tl[slot] = globaltimer_ns(); } while (0)
#else
#define BLR_STAMP(slot) do { } while (0)
#endif
  if (threadIdx.x == 0) BLR_STAMP(0);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (uint32_t s = 0; s < NST; ++s) {
      mbar_init(full0 + 8 * s, 2);
      mbar_init(empty0 + 8 * s, kConsumerWarps);
    }
    mbar_init_fence();
  }
  // Programmatic dependent launch: let the next kernel in the stream begin its own set-up as SMs free up, and
  // do not touch memory the previous kernel may still be writing (workspace, activations) before it is done.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------------------------ weight producer (lane 0 paces; K-major: one box per
    // stage; M-major: lanes 0..3 issue one 32-column box each)
    if (lane == 0) {
      tma_prefetch_desc(&p.ph[0].tmW[0]);
      if (p.nphases > 1) tma_prefetch_desc(&p.ph[1].tmW[0]);
    }
    RingPos rp;
    bool ok = true;
    for (int phs = 0; phs < p.nphases && ok; ++phs) {
      const PhaseDesc& ph = p.ph[phs];
      int t, t_hi;
      tile_range(ph, t, t_hi);
      Batch b;
      const int kstep = ph.kmajor ? (ph.wbits == 16 ? 64 : 128) : 64;
      const int nchunks = ph.nstage_chunks, kmajor = ph.kmajor, c_first = first_chunk(ph), ksub = ph.ks;
      while (ok && next_batch(ph, t, t_hi, b)) {
        int kc = c_first;
        for (int c = 0; c < nchunks; ++c) {
          if (!rp.first_pass) {
            int w_ok = 1;
            if (lane == 0) w_ok = mbar_wait(empty0 + 8 * rp.s, rp.use_parity ^ 1u, abort_flag) ? 1 : 0;
            w_ok = __shfl_sync(0xffffffffu, w_ok, 0);
            if (!w_ok) { ok = false; break; }
          }
          const uint32_t dst = smem_base + rp.s * stage_bytes, bar = full0 + 8 * rp.s;
          const int k0 = kc * ksub * kstep;
          // sub-chunks past the end of K read out-of-range coordinates: zero fill, no memory traffic
          if (kmajor) {
            if (lane == 0) {
              mbar_arrive_expect_tx(bar, ksub * b.nt * 16 * 128);
              for (int sub = 0; sub < ksub; ++sub)
                tma_load_3d(dst + sub * ph.sub_bytes, &ph.tmW[b.nt - 1], k0 + sub * kstep, b.mt0 * 16, b.g, bar);
            }
          } else {
            if (lane == 0) mbar_arrive_expect_tx(bar, ksub * b.nt * kTileBytes);
            __syncwarp();
            // lane = sub * 4 + tile
            if (lane < ksub * 4 && (lane & 3) < b.nt)
              tma_load_3d(dst + (lane >> 2) * kSubBytes + (lane & 3) * kTileBytes, &ph.tmW[0], (b.mt0 + (lane & 3)) * 32,
                          k0 + (lane >> 2) * kstep, b.g, bar);
          }
          rp.advance(NST);
          if (++kc == nchunks) kc = 0;
        }
      }
      if (lane == 0) BLR_STAMP(1 + phs);  // all weight loads of this phase issued
    }
  } else if (warp == kConsumerWarps + 1) {
    // ------------------------------------------------ activation producer
    if (lane == 0) {
      tma_prefetch_desc(&p.ph[0].tmA);
      if (p.nphases > 1) tma_prefetch_desc(&p.ph[1].tmA);
      RingPos rp;
      bool ok = true;
      for (int phs = 0; phs < p.nphases && ok; ++phs) {
        const PhaseDesc& ph = p.ph[phs];
        int t, t_hi;
        tile_range(ph, t, t_hi);
        if (phs == 1 && t < t_hi) {
          // activations of the second phase are produced by the whole grid
          ok = wait_counter(p.counters + (p.mix ? 1 : 0), gridDim.x, abort_flag);
          fence_proxy_async();
        }
        Batch b;
        const int nchunks = ph.nstage_chunks, a_boxes = ph.a_boxes * ph.ks, c_first = first_chunk(ph);
        while (ok && next_batch(ph, t, t_hi, b)) {
          int kc = c_first;
          for (int c = 0; c < nchunks; ++c) {
            if (!rp.first_pass && !mbar_wait(empty0 + 8 * rp.s, rp.use_parity ^ 1u, abort_flag)) { ok = false; break; }
            const uint32_t dst = smem_base + rp.s * stage_bytes + p.w_bytes, bar = full0 + 8 * rp.s;
            const int k0 = kc * a_boxes * 64;
            mbar_arrive_expect_tx(bar, a_boxes * kABoxBytes);
            for (int bx = 0; bx < a_boxes; ++bx) tma_load_3d(dst + bx * kABoxBytes, &ph.tmA, k0 + bx * 64, 0, b.g, bar);
            rp.advance(NST);
            if (++kc == nchunks) kc = 0;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------ consumers: warp w owns rows [16w, 16w+16) of the batch
    const int ctid = threadIdx.x;  // 0..255
    const int row0 = warp * 16;  // this warp's rows within a batch
    const int g = lane >> 2, tq = lane & 3;
    RingPos rp;
    bool ok = true;
    bool first_stage = true;
    for (int phs = 0; phs < p.nphases; ++phs) {
      const PhaseDesc& ph = p.ph[phs];
      int t, t_hi;
      tile_range(ph, t, t_hi);
      Batch b;
      const int nchunks = ph.nstage_chunks, wbits = ph.wbits, kmajor = ph.kmajor, ksub = ph.ks;
      const uint32_t a_sub = ph.a_boxes * kABoxBytes, sub_bytes = ph.sub_bytes;
      while (next_batch(ph, t, t_hi, b)) {
        float acc[4][NT][4];  // four independent accumulation chains (one per k16 step / window of a chunk)
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
          for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[q][n][e] = 0.f;
        const bool active = row0 < b.nt * ph.unit_rows;
        // grouped scales: rows of the scale table for this thread's two weight rows
        const int ngroups = ph.K / kScaleGroup;
        const __half* srow = nullptr;
        const __half* srow8 = nullptr;
        float tot[NT][4];
        if constexpr (GS) {
          const int m = b.mt0 * ph.unit_rows + row0 + g;
          if (active && m < ph.M) srow = ph.scale + ((long long)b.g * ph.M + m) * ngroups;
          if (active && m + 8 < ph.M) srow8 = ph.scale + ((long long)b.g * ph.M + m + 8) * ngroups;
#pragma unroll
          for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) tot[n][e] = 0.f;
        }
        int kc = first_chunk(ph);  // the producers walk the stages of a batch from a rotated start
        for (int c = 0; c < nchunks && ok; ++c) {
          const uint32_t s = rp.s;
          if (!mbar_wait(full0 + 8 * s, rp.use_parity, abort_flag)) { ok = false; break; }
          if (first_stage) {
            first_stage = false;
            if (ctid == 0) BLR_STAMP(3);  // first stage landed
          }
          if (active) {
            uint32_t sW = smem_base + s * stage_bytes, sA = sW + p.w_bytes;
            for (int sub = 0; sub < ksub; ++sub, sW += sub_bytes, sA += a_sub) {
              GroupScales gs;
              if constexpr (GS) gs = load_scale_groups(srow, srow8, (kc * ksub + sub) * (wbits == 8 ? 1 : 2), ngroups, wbits);
              if (wbits == 16) {
                if (kmajor) consume_k16<BF16, NT>(sW, sA, row0, acc, lane);
                else consume_m16<BF16, NT>(sW + (warp >> 1) * kTileBytes, sA, warp & 1, acc, lane);
              } else if (wbits == 8) {
                consume_k8<BF16, NT>(sW, sA, row0, acc, lane);
              } else {
                consume_k4<BF16, NT>(sW, sA, row0, acc, lane);
              }
              if constexpr (GS) fold_scale_groups<NT>(acc, tot, gs, wbits);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(empty0 + 8 * s);
          rp.advance(NST);
          if (++kc == nchunks) kc = 0;
        }
        // ---- epilogue straight from the accumulator fragment: rows g / g+8, tokens 2*tq / 2*tq+1 (+8 per n-tile)
        if (active) {
          const int m_lo = b.mt0 * ph.unit_rows + row0 + g;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int mg = m_lo + 8 * h;
            if (mg < ph.M) {
              const float sc = (!GS && ph.scale) ? __half2float(ph.scale[(long long)b.g * ph.M + mg]) : 1.f;
              const long long base = b.g * ph.os_g + (mg / ph.per) * ph.os_hi + (mg % ph.per) * ph.os_lo;
#pragma unroll
              for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  const int tok = n * 8 + tq * 2 + e;
                  if (tok < p.N) {
                    float v = GS ? tot[n][2 * h + e]
                                 : (acc[0][n][2 * h + e] + acc[1][n][2 * h + e] + acc[2][n][2 * h + e] + acc[3][n][2 * h + e]) * sc;
                    if (ph.round_out) v = round_clamp_i8(v);
                    const long long off = base + tok * ph.os_n;
                    if (ph.out_f32) reinterpret_cast<float*>(ph.out)[off] = v;
                    else store16<BF16>(ph.out, off, v);
                  }
                }
            }
          }
        }
      }
      if (ctid == 0) BLR_STAMP(4 + 4 * phs);  // phase consumed and written
      // ---- end of phase: publish, then (BLAST) apply the coupling
      if (phs + 1 < p.nphases) {
        // bar.sync orders the CTA's stores before thread 0; its gpu-scope release is cumulative over them
        consumer_bar();
        if (ctid == 0) red_release_gpu_add(p.counters + 0, 1u);
        if (p.mix) {
          CoupleRegs cr;
          couple_preload(p, ctid, cr);
          if (ctid == 0) {
            if (!wait_counter(p.counters + 0, gridDim.x, abort_flag)) ok = false;
          }
          consumer_bar();
          if (ctid == 0) BLR_STAMP(5);  // grid barrier 0 passed
          if (!*abort_flag) couple<BF16>(p, ctid, cr, ybuf);
          consumer_bar();
          if (ctid == 0) {
            red_release_gpu_add(p.counters + 1, 1u);
            BLR_STAMP(6);  // coupling written
          }
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
  if (threadIdx.x == 0) BLR_STAMP(9);
#undef BLR_STAMP
  if (*abort_flag) {
    // let tile loads that may still be in flight land before the shared memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
}

// ------------------------------------------------------------------ host launcher
template <bool BF16, int NT, bool GS>
static int launch_impl(const StreamParams& p, cudaStream_t stream) {
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != BLR_OK) return rc;
  BLR_REQUIRE(di.coop, BLR_ERR_UNSUPPORTED, "device does not support cooperative launch");
  const size_t smem = (size_t)p.nstages * p.stage_bytes + p.mix_bytes + kStreamTailBytes;
  BLR_REQUIRE((int)smem <= di.max_smem_optin, BLR_ERR_UNSUPPORTED, "needs %zu bytes of shared memory, device offers %d",
              smem, di.max_smem_optin);
  auto kern = blr_stream_kernel<BF16, NT, GS>;
  int dev;
  BLR_CUDA_OK(cudaGetDevice(&dev));
  static bool configured[64] = {};  // one flag per device for this template instance
  if (!configured[dev & 63]) {
    BLR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem_optin));
    configured[dev & 63] = true;
  }
  void* args[] = {const_cast<StreamParams*>(&p)};
  // Cooperative launch: the grid barriers need every CTA resident, and this makes the launch fail
  // instead of deadlock when they cannot be.
  // Programmatic dependent launch on top of it: the next launch in the stream may start its set-up while this
  // grid drains (see the griddepcontrol pair in the kernel).
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(di.sm_count);
  cfg.blockDim = dim3(kStreamThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  at[1].id = cudaLaunchAttributeCooperative;
  at[1].val.cooperative = 1;
  cfg.attrs = at;
  cfg.numAttrs = 2;
  BLR_CUDA_OK(cudaLaunchKernelExC(&cfg, (const void*)kern, args));
  return BLR_OK;
}

#ifdef BLR_TIMELINE
unsigned long long* g_stream_timeline = nullptr;
void set_stream_timeline(unsigned long long* dev_ptr) { g_stream_timeline = dev_ptr; }
#endif

int launch_stream(const StreamParams& p_in, int is_bf16, cudaStream_t stream) {
  StreamParams p = p_in;
#ifdef BLR_TIMELINE
  p.timeline = g_stream_timeline;
#endif
  BLR_REQUIRE(p.N >= 1 && p.N <= kStreamMaxTokens, BLR_ERR_ARG, "stream kernel handles 1..%d tokens, got %d",
              kStreamMaxTokens, p.N);
  if (p.ph[0].group != 0) {  // one scale per kScaleGroup contraction indices: its own instantiation
    if (p.N <= 8) return is_bf16 ? launch_impl<true, 1, true>(p, stream) : launch_impl<false, 1, true>(p, stream);
    return is_bf16 ? launch_impl<true, 2, true>(p, stream) : launch_impl<false, 2, true>(p, stream);
  }
  if (p.N <= 8) return is_bf16 ? launch_impl<true, 1, false>(p, stream) : launch_impl<false, 1, false>(p, stream);
  return is_bf16 ? launch_impl<true, 2, false>(p, stream) : launch_impl<false, 2, false>(p, stream);
}

}  // namespace blr
