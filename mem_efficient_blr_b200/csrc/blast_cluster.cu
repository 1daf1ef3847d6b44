// Two-stage decode kernel built on thread-block clusters (see blast_cluster.h for the decomposition): BLAST,
// low-rank (BLAST with an all-ones coupling) and Monarch.
//
// Per CTA (block index `blk` = rank in the cluster, slice `sl` = blockIdx.y, row part = blockIdx.z): one producer
// warp streams, through a ring of TMA stages, first its first-stage rows (BLAST: rows [sl*rs, (sl+1)*rs) of V_blk)
// with the matching boxes of x, then its part of the rows of U_blk restricted to the slice's columns; eight
// consumer warps turn the stages into mma.sync products exactly like the grid-wide streaming kernel (one 16-row
// group per warp).  Between the two phases the cluster exchanges the first stage's outputs through distributed
// shared memory, guarded by mbarriers that peers arrive on remotely, in one of three forms (template parameter).
// All waits are bounded; nothing here spins on another cluster.
#include "blast_cluster.h"
#include "ptx.cuh"
#include "stream_device.cuh"
#include "tmap.h"

namespace blr {

// XCH: how the cluster turns the first phase's outputs into the second phase's activations -
// kXchPull (every CTA pulls all of every y_j), kXchSubslice (coupling by rank sub-slice), kXchMonarch (permutation).
template <bool BF16, int NT, bool GS, int XCH>
__global__ void __launch_bounds__(kClusterThreads, 2) blr_blast_cluster_kernel(const __grid_constant__ ClusterParams p) {
  constexpr bool MON = XCH == kXchMonarch, SUB = XCH == kXchSubslice;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  constexpr int NP = NT * 8;                    // token rows kept everywhere
  constexpr uint32_t kABoxBytes = NP * 128;     // one [tokens][64 k] activation box
  const uint32_t NST = p.nstages, stage_bytes = p.stage_bytes;
  const int rs = p.rs;
  // [ring][ybuf: NP x rs 16-bit][sbuf: b x rs 16-bit][gbuf: NP x rs 16-bit][zbuf: rs/64 boxes][barriers]
  uint8_t* ybuf = smem + (size_t)NST * stage_bytes;
  uint8_t* sbuf = ybuf + NP * rs * 2;
  uint8_t* gbuf = sbuf + 16 * rs * 2;  // sub-slice coupling: y_j[token][this CTA's w ranks] of every in-block j
  uint8_t* zbuf = gbuf + NP * rs * 2;
  uint64_t* bars = reinterpret_cast<uint64_t*>(zbuf + (rs / 64) * kABoxBytes);
  // full[16], empty[16], y_ready, read_done
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + 16);
  const uint32_t y_ready = smem_u32(bars + 32), read_done = smem_u32(bars + 33), z_ready = smem_u32(bars + 35);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 34);
  int* last_flag = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int blk = blockIdx.x, sl = blockIdx.y, part = blockIdx.z, nb = p.b;
  const int q_lo = part * p.q_part, q_hi = min(p.Q, q_lo + p.q_part);
  const int r_begin = sl * rs, r_len = min(rs, p.R - r_begin);
  // first phase: weight/activation block and row range of this CTA (BLAST: its own block, the slice's ranks;
  // Monarch: a share of the rows of one of the first-stage blocks that feed the slice)
  const int blk0 = MON ? sl * p.mblk + blk / p.cpb : blk;
  const int r_begin0 = MON ? (blk % p.cpb) * rs : r_begin, r_len0 = MON ? rs : r_len;
  const PhaseDesc& ph0 = p.ph[0];
  const PhaseDesc& ph1 = p.ph[1];

#ifdef BLR_TIMELINE  // profiling builds only: 16 cycle stamps per CTA
  unsigned long long* tl = p.timeline ? p.timeline + (size_t)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 : nullptr;
#define BLR_STAMP(slot) do { if (tl) tl[slot] = (unsigned long long)clock64(); } while (0)
  if (threadIdx.x == 0 && tl) { tl[0] = globaltimer_ns(); tl[15] = (unsigned long long)clock64(); }
#else
#define BLR_STAMP(slot) do { } while (0)
#endif
  if (warp == kConsumerWarps) {
    // descriptors this CTA will use: one per batch height for k-contiguous weights (full batches and the last one)
    const int rows0 = r_len0, rows1 = min(p.Q, (int)(blockIdx.z + 1) * p.q_part) - (int)blockIdx.z * p.q_part;
    const int hf0 = (min(rows0, kBatchRows) + 15) >> 4, hl0 = (((rows0 - 1) % kBatchRows) + 16) >> 4;
    const int hf1 = (min(rows1, kBatchRows) + 15) >> 4, hl1 = (((rows1 - 1) % kBatchRows) + 16) >> 4;
    if (lane == 0) tma_prefetch_desc(&ph0.tmW[ph0.kmajor ? hf0 - 1 : 0]);
    if (lane == 1) tma_prefetch_desc(&ph0.tmA);
    if (lane == 2) tma_prefetch_desc(&ph1.tmW[ph1.kmajor ? hf1 - 1 : 0]);
    if (lane == 3 && ph0.kmajor && hl0 != hf0) tma_prefetch_desc(&ph0.tmW[hl0 - 1]);
    if (lane == 4 && ph1.kmajor && hl1 != hf1) tma_prefetch_desc(&ph1.tmW[hl1 - 1]);
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *last_flag = 0;
    for (uint32_t s = 0; s < NST; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, kConsumerWarps);
    }
    mbar_init(y_ready, nb);
    mbar_init(read_done, nb);
    mbar_init(z_ready, nb);
    mbar_init_fence();
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __syncthreads();
  // Peers arrive on this CTA's barriers only after their first phase; the cluster barrier that makes the
  // barriers visible to them is split so that nobody waits for it here.
  cluster_arrive();
  if (threadIdx.x == 0) BLR_STAMP(1);

  if (warp == kConsumerWarps) {
    // ------------------------------------------------ producer (lane 0; for m-contiguous weights lanes 0..7 issue tiles)
    // One ring stage of phase `phs`: batch of rows at r0, chunk group c.  Weights and activations complete on
    // the same barrier; they can be issued separately (do_w announces the bytes of both).
    auto issue = [&](int phs, int r0, int row_hi, int c, uint32_t slot, bool do_w, bool do_x) {
      const PhaseDesc& ph = p.ph[phs];
      const int ksub = phs == 0 ? p.ks0 : p.ks1;
      const int kstep = ph.kmajor ? (ph.wbits == 16 ? 64 : 128) : 64;             // coordinate units per chunk
      // K range: whole P in phase 0, the slice in phase 1 (coordinates are elements, or bytes for int8 / int4)
      const int k_base = phs == 0 ? 0 : (ph.kmajor && ph.wbits == 4 ? r_begin / 2 : r_begin);
      const int rows = min(kBatchRows, row_hi - r0), wblk = phs == 0 ? blk0 : blk;
      const int h = (rows + 15) >> 4, tiles = (rows + 31) >> 5;
      const uint32_t dst = smem_base + slot * stage_bytes, bar = full0 + 8 * slot;
      const int k0 = k_base + c * ksub * kstep;
      const uint32_t a_bytes = phs == 0 ? ksub * ph.a_boxes * kABoxBytes : 0u;
      if (do_w) {
        if (ph.kmajor) {
          if (lane == 0) {
            mbar_arrive_expect_tx(bar, ksub * h * 16 * 128 + a_bytes);
            for (int sub = 0; sub < ksub; ++sub)
              tma_load_3d(dst + sub * kSubBytes, &ph.tmW[h - 1], k0 + sub * kstep, r0, wblk, bar);
          }
        } else {
          if (lane == 0) mbar_arrive_expect_tx(bar, ksub * tiles * kTileBytes + a_bytes);
          __syncwarp();
          if (lane < ksub * 4 && (lane & 3) < tiles)
            tma_load_3d(dst + (lane >> 2) * kSubBytes + (lane & 3) * kTileBytes, &ph.tmW[0], r0 + (lane & 3) * 32,
                        k0 + (lane >> 2) * kstep, wblk, bar);
        }
      }
      if (do_x && phs == 0 && lane == 0) {
        const int nbox = ksub * ph.a_boxes, ka = c * nbox * 64;
        for (int bx = 0; bx < nbox; ++bx) tma_load_3d(dst + p.w_bytes + bx * kABoxBytes, &ph.tmA, ka + bx * 64, 0, blk0, bar);
      }
    };
    // The weights do not depend on the kernel before this one in the stream, the activations do: fill the
    // ring with first-phase weights, wait for the previous kernel, then add the activations.
    const int nstage0 = (ph0.nchunks + p.ks0 - 1) / p.ks0;
    int pre = 0;
    for (int pass = 0; pass < 2; ++pass) {
      pre = 0;
      for (int r0 = r_begin0; r0 < r_begin0 + r_len0 && pre < (int)NST; r0 += kBatchRows)
        for (int c = 0; c < nstage0 && pre < (int)NST; ++c, ++pre) issue(0, r0, r_begin0 + r_len0, c, pre, pass == 0, pass == 1);
      if (pass == 0) {
        if (lane == 0) BLR_STAMP(12);
        asm volatile("griddepcontrol.wait;" ::: "memory");
      }
    }
    if (lane == 0) BLR_STAMP(13);
    RingPos rp;
    bool ok = true;
    int skip = pre;
    for (int phs = 0; phs < 2 && ok; ++phs) {
      const int ksub = phs == 0 ? p.ks0 : p.ks1;
      const int row_lo = phs == 0 ? r_begin0 : q_lo, row_hi = phs == 0 ? r_begin0 + r_len0 : q_hi;
      const int nstage = phs == 0 ? nstage0 : (p.nchunks1 + ksub - 1) / ksub;
      for (int r0 = row_lo; r0 < row_hi && ok; r0 += kBatchRows) {
        for (int c = 0; c < nstage; ++c) {
          if (skip > 0) {  // issued above
            --skip;
            rp.advance(NST);
            continue;
          }
          if (!rp.first_pass) {
            int w_ok = 1;
            if (lane == 0) w_ok = mbar_wait(empty0 + 8 * rp.s, rp.use_parity ^ 1u, abort_flag) ? 1 : 0;
            w_ok = __shfl_sync(0xffffffffu, w_ok, 0);
            if (!w_ok) { ok = false; break; }
          }
          issue(phs, r0, row_hi, c, rp.s, true, true);
          rp.advance(NST);
        }
      }
    }
    cluster_wait();
  } else {
    // ------------------------------------------------ consumers
    const int ctid = threadIdx.x;
    const int row0 = warp * 16, g = lane >> 2, tq = lane & 3;
    RingPos rp;
    bool ok = true;
    // (a) the coupling factors of this CTA's out-block on the slice -> sbuf[j][r], asynchronously
    const bool s_vec = p.s_r == 1 && ((p.s_i | p.s_j) & 7) == 0 && (reinterpret_cast<uintptr_t>(p.S) & 15) == 0;
    {
      const uint16_t* S = reinterpret_cast<const uint16_t*>(p.S);
      const int nv = rs >> 3;
      const int w = rs / nb, wv = w >> 3;  // sub-slice coupling: ranks and 8-rank vectors per CTA
      for (int e = ctid; e < (SUB ? nb * nb * wv : 0); e += kConsumerWarps * 32) {
        // sbuf[i][j][t] = S[i][j][r_begin + blk*w + t]: the factors of every (out, in) pair on this CTA's ranks
        const int ij = e / wv, v = e - ij * wv, i = ij / nb, j = ij - i * nb, r = r_begin + blk * w + v * 8;
        uint16_t* d = reinterpret_cast<uint16_t*>(sbuf) + ij * w + v * 8;
        if (S == nullptr) {
          for (int k = 0; k < 8; ++k) d[k] = r + k < p.R ? (BF16 ? (uint16_t)0x3F80 : (uint16_t)0x3C00) : (uint16_t)0;
        } else if (s_vec && r + 8 <= p.R) {
          cp_async16(smem_u32(d), S + i * p.s_i + j * p.s_j + r);
        } else {
          for (int k = 0; k < 8; ++k) d[k] = r + k < p.R ? S[i * p.s_i + j * p.s_j + (long long)(r + k) * p.s_r] : (uint16_t)0;
        }
      }
      for (int e = ctid; e < (XCH == kXchPull ? nb * nv : 0); e += kConsumerWarps * 32) {  // Monarch has no factors
        const int j = e / nv, v = e - j * nv, r = r_begin + v * 8;
        const uint32_t dst = smem_u32(sbuf) + (j * rs + v * 8) * 2;
        if (S == nullptr) {  // no coupling factors: all ones (a plain sum over the in-blocks), zero past R
          uint16_t* d = reinterpret_cast<uint16_t*>(sbuf) + j * rs + v * 8;
          for (int k = 0; k < 8; ++k) d[k] = r + k < p.R ? (BF16 ? (uint16_t)0x3F80 : (uint16_t)0x3C00) : (uint16_t)0;
        } else if (s_vec && r + 8 <= p.R) {
          cp_async16(dst, S + blk * p.s_i + j * p.s_j + r);
        } else {
          uint16_t* d = reinterpret_cast<uint16_t*>(sbuf) + j * rs + v * 8;
          for (int k = 0; k < 8; ++k) d[k] = r + k < p.R ? S[blk * p.s_i + j * p.s_j + (long long)(r + k) * p.s_r] : (uint16_t)0;
        }
      }
      // (b) clear the coupled activations (token rows past N and ranks past the slice stay zero)
      for (int e = ctid; e < (rs / 64) * (int)kABoxBytes / 16; e += kConsumerWarps * 32) reinterpret_cast<uint4*>(zbuf)[e] = make_uint4(0, 0, 0, 0);
      for (int e = ctid; e < NP * rs * 2 / 16; e += kConsumerWarps * 32) reinterpret_cast<uint4*>(ybuf)[e] = make_uint4(0, 0, 0, 0);
    }
    consumer_bar();
    asm volatile("griddepcontrol.wait;" ::: "memory");  // out32, the counters and x belong to the previous kernel until here
    if (ctid == 0) BLR_STAMP(14);
    for (int phs = 0; phs < 2; ++phs) {
      const PhaseDesc& ph = p.ph[phs];
      const int ksub = phs == 0 ? p.ks0 : p.ks1, wbits = ph.wbits, kmajor = ph.kmajor;
      const int row_lo = phs == 0 ? r_begin0 : q_lo, row_hi = phs == 0 ? r_begin0 + r_len0 : q_hi;
      const int nstage = phs == 0 ? (ph.nchunks + ksub - 1) / ksub : (p.nchunks1 + ksub - 1) / ksub;
      const uint32_t a_sub = ph.a_boxes * kABoxBytes;
      for (int r0 = row_lo; r0 < row_hi; r0 += kBatchRows) {
        const int rows = min(kBatchRows, row_hi - r0);
        const bool active = row0 < rows;
        // per-row scales of quantised weights: fetched now, used after the batch's last stage
        float sc2[2] = {1.f, 1.f};
        if (!GS && phs == 0 && ph.scale && active) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int m = r0 + row0 + g + 8 * h;
            if (m < row_hi) sc2[h] = __half2float(__ldg(ph.scale + (long long)blk0 * ph.M + m));
          }
        }
        // grouped scales: rows of the scale table for this thread's two weight rows, first group of the K range
        const int ngroups = ph.K / kScaleGroup, gbase = phs == 0 ? 0 : r_begin / kScaleGroup;
        const __half* srow = nullptr;
        const __half* srow8 = nullptr;
        float tot[NT][4];
        if constexpr (GS) {
          const int m = r0 + row0 + g;
          const int sblk = phs == 0 ? blk0 : blk;
          if (active && m < row_hi) srow = ph.scale + ((long long)sblk * ph.M + m) * ngroups;
          if (active && m + 8 < row_hi) srow8 = ph.scale + ((long long)sblk * ph.M + m + 8) * ngroups;
#pragma unroll
          for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) tot[n][e] = 0.f;
        }
        float acc[4][NT][4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
          for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[q][n][e] = 0.f;
        for (int c = 0; c < nstage && ok; ++c) {
          const uint32_t s = rp.s;
          if (!mbar_wait(full0 + 8 * s, rp.use_parity, abort_flag)) { ok = false; break; }
          if (ctid == 0 && c == 0 && r0 == row_lo) BLR_STAMP(9 + phs);
          if (active) {
            uint32_t sW = smem_base + s * stage_bytes;
            uint32_t sA = phs == 0 ? sW + p.w_bytes : smem_u32(zbuf) + c * ksub * a_sub;
            for (int sub = 0; sub < ksub; ++sub, sW += kSubBytes, sA += a_sub) {
              GroupScales gs;
              if constexpr (GS) gs = load_scale_groups(srow, srow8, gbase + (c * ksub + sub) * (wbits == 8 ? 1 : 2), ngroups, wbits);
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
        }
        if (ctid == 0 && phs == 1 && r0 + kBatchRows >= row_hi) BLR_STAMP(11);
        if (active) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int m = r0 + row0 + g + 8 * h;
            if (m < row_hi) {
              if (phs == 0) {
                // y_blk[token][r - r_begin] (16-bit) into this CTA's shared memory, for the whole cluster to read
                const float sc = sc2[h];
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                  for (int e = 0; e < 2; ++e) {
                    float v = GS ? tot[n][2 * h + e]
                                 : (acc[0][n][2 * h + e] + acc[1][n][2 * h + e] + acc[2][n][2 * h + e] + acc[3][n][2 * h + e]) * sc;
                    if (p.round_y) v = round_clamp_i8(v);
                    store16<BF16>(ybuf, (long long)(n * 8 + tq * 2 + e) * rs + (m - r_begin0), v);
                  }
              } else {
                // partial out over this slice: fp32 reduction into out32[blk*Q + m][token]
                float* dst = p.out32 + ((long long)blk * p.Q + m) * NP;
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                  const int tok = n * 8 + tq * 2;
                  if (tok < p.N) {
                    if constexpr (GS)
                      red_add_v2_f32(dst + tok, tot[n][2 * h], tot[n][2 * h + 1]);
                    else
                      red_add_v2_f32(dst + tok, acc[0][n][2 * h] + acc[1][n][2 * h] + acc[2][n][2 * h] + acc[3][n][2 * h],
                                     acc[0][n][2 * h + 1] + acc[1][n][2 * h + 1] + acc[2][n][2 * h + 1] + acc[3][n][2 * h + 1]);
                  }
                }
              }
            }
          }
        }
      }
      if (phs == 0) {
        // ---- exchange y inside the cluster and couple this CTA's out-block on the slice
        consumer_bar();  // all of y_blk is in ybuf
        if (ctid == 0) BLR_STAMP(2);
        cluster_wait();  // every CTA of the cluster has initialised its barriers (long since)
        if (ctid < nb) mbar_arrive_remote(mapa_shared(y_ready, ctid));
        if (!mbar_wait_cluster(y_ready, 0, abort_flag)) ok = false;
        cp_async_wait_all();
        consumer_bar();  // sbuf complete for every thread
        if (ctid == 0) BLR_STAMP(3);
        if (MON && !*abort_flag) {
          // Monarch: the exchange is the permutation.  Element t of this CTA's slice of z_l is the first-stage output
          // (block sl*mblk + t / per, column q); that column was computed by CTA (t / per)*cpb + q / rs as its local
          // row q % rs.
          const uint32_t ybase = smem_u32(ybuf);
          for (int e = ctid; e < p.N * rs; e += kConsumerWarps * 32) {
            const int n = e / rs, t = e - n * rs;
            const int kk = t / p.per, jj = t - kk * p.per;
            const int q = p.w1_grouped ? blk * p.per + jj : jj * nb + blk;
            const int c = kk * p.cpb + q / rs, loc = q % rs;
            const uint16_t v = ld_shared_cluster_u16(mapa_shared(ybase + (n * rs + loc) * 2, c));
            *reinterpret_cast<uint16_t*>(zbuf + (t >> 6) * kABoxBytes + sw128(n, (t & 63) >> 3) + (t & 7) * 2) = v;
          }
        } else if (SUB && !*abort_flag) {
          // Coupling by rank sub-slice.  This CTA takes ranks [blk*w, (blk+1)*w) of the slice for every pair of blocks:
          // (1) gather those ranks of every y_j, (2) z_i = sum_j S_ij . y_j on them for every out-block i,
          // (3) write z_i's piece into CTA i's zbuf.  Traffic through distributed shared memory: 2 N rs values per CTA.
          const int w = rs / nb, wv = w >> 3;
          const uint32_t ybase = smem_u32(ybuf), gbase = smem_u32(gbuf), sbase = smem_u32(sbuf), zbase = smem_u32(zbuf);
          // (two remote loads in flight per thread: their latency is what this step costs)
          for (int e0 = ctid; e0 < nb * p.N * wv; e0 += 2 * kConsumerWarps * 32) {
            const int e1 = e0 + kConsumerWarps * 32;
            const bool two = e1 < nb * p.N * wv;
            const int j0 = e0 / (p.N * wv), rem0 = e0 - j0 * (p.N * wv), n0 = rem0 / wv, v0 = rem0 - n0 * wv;
            const int ee = two ? e1 : e0;
            const int j1 = ee / (p.N * wv), rem1 = ee - j1 * (p.N * wv), n1 = rem1 / wv, v1 = rem1 - n1 * wv;
            const uint4 ya = ld_shared_cluster_v4(mapa_shared(ybase + (n0 * rs + blk * w + v0 * 8) * 2, j0));
            uint4 yb = ya;
            if (two) yb = ld_shared_cluster_v4(mapa_shared(ybase + (n1 * rs + blk * w + v1 * 8) * 2, j1));
            *reinterpret_cast<uint4*>(gbuf + ((j0 * NP + n0) * w + v0 * 8) * 2) = ya;
            if (two) *reinterpret_cast<uint4*>(gbuf + ((j1 * NP + n1) * w + v1 * 8) * 2) = yb;
          }
          consumer_bar();  // gbuf complete; this CTA no longer reads its peers' ybuf
          if (ctid < nb) mbar_arrive_remote_relaxed(mapa_shared(read_done, ctid));
          if constexpr (NT == 2) {
            // 9..16 tokens: one thread couples two out-blocks x two tokens (n, n + 8) on 8 ranks, so that every
            // unpacked factor and activation feeds two products
            const int ipairs = (nb + 1) >> 1;
            for (int e = ctid; e < ipairs * 8 * wv; e += kConsumerWarps * 32) {
              const int ip = e / (8 * wv), rem = e - ip * (8 * wv), n0 = rem / wv, v = rem - n0 * wv;
              const int i0 = 2 * ip, i1 = i0 + 1 < nb ? i0 + 1 : i0, n1 = n0 + 8;  // (clamped: the extra result is dropped)
              float a[2][2][8];
#pragma unroll
              for (int x = 0; x < 2; ++x)
#pragma unroll
                for (int y = 0; y < 2; ++y)
#pragma unroll
                  for (int k = 0; k < 8; ++k) a[x][y][k] = 0.f;
              for (int j = 0; j < nb; ++j) {
                uint4 sv[2], yv[2];
                lds128(sbase + ((i0 * nb + j) * w + v * 8) * 2, sv[0].x, sv[0].y, sv[0].z, sv[0].w);
                lds128(sbase + ((i1 * nb + j) * w + v * 8) * 2, sv[1].x, sv[1].y, sv[1].z, sv[1].w);
                lds128(gbase + ((j * NP + n0) * w + v * 8) * 2, yv[0].x, yv[0].y, yv[0].z, yv[0].w);
                lds128(gbase + ((j * NP + n1) * w + v * 8) * 2, yv[1].x, yv[1].y, yv[1].z, yv[1].w);
                float sf[2][8], yf[2][8];
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                  const uint32_t sw[4] = {sv[x].x, sv[x].y, sv[x].z, sv[x].w}, yw[4] = {yv[x].x, yv[x].y, yv[x].z, yv[x].w};
#pragma unroll
                  for (int k = 0; k < 4; ++k) {
                    const float2 fs = unpack16x2<BF16>(sw[k]), fy = unpack16x2<BF16>(yw[k]);
                    sf[x][2 * k] = fs.x, sf[x][2 * k + 1] = fs.y, yf[x][2 * k] = fy.x, yf[x][2 * k + 1] = fy.y;
                  }
                }
#pragma unroll
                for (int x = 0; x < 2; ++x)
#pragma unroll
                  for (int y = 0; y < 2; ++y)
#pragma unroll
                    for (int k = 0; k < 8; ++k) a[x][y][k] = fmaf(sf[x][k], yf[y][k], a[x][y][k]);
              }
              const int col = blk * w + v * 8;  // column of the slice, a multiple of 8
#pragma unroll
              for (int x = 0; x < 2; ++x) {
                if (x == 1 && i0 + 1 >= nb) break;
#pragma unroll
                for (int y = 0; y < 2; ++y) {
                  const int n = y ? n1 : n0;
                  if (n >= p.N) continue;
                  float* r = a[x][y];
                  if (p.round_z) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) r[k] = round_clamp_i8(r[k]);
                  }
                  uint4 o;
                  o.x = pack16x2<BF16>(r[0], r[1]); o.y = pack16x2<BF16>(r[2], r[3]);
                  o.z = pack16x2<BF16>(r[4], r[5]); o.w = pack16x2<BF16>(r[6], r[7]);
                  st_shared_cluster_v4(mapa_shared(zbase + (col >> 6) * kABoxBytes + sw128(n, (col & 63) >> 3), x ? i1 : i0), o);
                }
              }
            }
          } else
          for (int e = ctid; e < nb * p.N * wv; e += kConsumerWarps * 32) {
            const int i = e / (p.N * wv), rem = e - i * (p.N * wv), n = rem / wv, v = rem - n * wv;
            float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < nb; ++j) {
              uint4 sv, yv;
              lds128(sbase + ((i * nb + j) * w + v * 8) * 2, sv.x, sv.y, sv.z, sv.w);
              lds128(gbase + ((j * NP + n) * w + v * 8) * 2, yv.x, yv.y, yv.z, yv.w);
              const float2 s0 = unpack16x2<BF16>(sv.x), s1 = unpack16x2<BF16>(sv.y), s2 = unpack16x2<BF16>(sv.z), s3 = unpack16x2<BF16>(sv.w);
              const float2 y0 = unpack16x2<BF16>(yv.x), y1 = unpack16x2<BF16>(yv.y), y2 = unpack16x2<BF16>(yv.z), y3 = unpack16x2<BF16>(yv.w);
              s[0] = fmaf(s0.x, y0.x, s[0]); s[1] = fmaf(s0.y, y0.y, s[1]);
              s[2] = fmaf(s1.x, y1.x, s[2]); s[3] = fmaf(s1.y, y1.y, s[3]);
              s[4] = fmaf(s2.x, y2.x, s[4]); s[5] = fmaf(s2.y, y2.y, s[5]);
              s[6] = fmaf(s3.x, y3.x, s[6]); s[7] = fmaf(s3.y, y3.y, s[7]);
            }
            if (p.round_z) {
#pragma unroll
              for (int k = 0; k < 8; ++k) s[k] = round_clamp_i8(s[k]);
            }
            uint4 o;
            o.x = pack16x2<BF16>(s[0], s[1]); o.y = pack16x2<BF16>(s[2], s[3]);
            o.z = pack16x2<BF16>(s[4], s[5]); o.w = pack16x2<BF16>(s[6], s[7]);
            const int col = blk * w + v * 8;  // column of the slice, a multiple of 8
            st_shared_cluster_v4(mapa_shared(zbase + (col >> 6) * kABoxBytes + sw128(n, (col & 63) >> 3), i), o);
          }
          consumer_bar();  // this CTA's pieces are written (the arrive below releases them to the cluster)
          if (ctid < nb) mbar_arrive_remote(mapa_shared(z_ready, ctid));
          if (!mbar_wait_cluster(z_ready, 0, abort_flag)) ok = false;  // every CTA's pieces of z_blk are here
        } else if (XCH == kXchPull && !*abort_flag) {
          // One item = 8 ranks of one token; two neighbouring lanes share an item, each gathers eight of the
          // (up to) sixteen in-blocks with all its remote loads in flight at once, then the halves are added.
          const int nv = rs >> 3, items = p.N * nv * 2;
          const uint32_t ybase = smem_u32(ybuf), sbase = smem_u32(sbuf);
          for (int base = 0; base < items; base += kConsumerWarps * 32) {
            const int e = base + ctid, pe = e >> 1, j0 = (e & 1) * 8;
            const bool valid = e < items;
            const int n = valid ? pe / nv : 0, v = valid ? pe - n * nv : 0;
            float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            const uint32_t yoff = ybase + (n * rs + v * 8) * 2;
            uint4 yv[8];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj)
              yv[jj] = (valid && j0 + jj < nb) ? ld_shared_cluster_v4(mapa_shared(yoff, j0 + jj)) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              if (valid && j0 + jj < nb) {
                uint4 sv;
                lds128(sbase + ((j0 + jj) * rs + v * 8) * 2, sv.x, sv.y, sv.z, sv.w);
                const float2 s0 = unpack16x2<BF16>(sv.x), s1 = unpack16x2<BF16>(sv.y), s2 = unpack16x2<BF16>(sv.z), s3 = unpack16x2<BF16>(sv.w);
                const float2 y0 = unpack16x2<BF16>(yv[jj].x), y1 = unpack16x2<BF16>(yv[jj].y), y2 = unpack16x2<BF16>(yv[jj].z), y3 = unpack16x2<BF16>(yv[jj].w);
                s[0] = fmaf(s0.x, y0.x, s[0]); s[1] = fmaf(s0.y, y0.y, s[1]);
                s[2] = fmaf(s1.x, y1.x, s[2]); s[3] = fmaf(s1.y, y1.y, s[3]);
                s[4] = fmaf(s2.x, y2.x, s[4]); s[5] = fmaf(s2.y, y2.y, s[5]);
                s[6] = fmaf(s3.x, y3.x, s[6]); s[7] = fmaf(s3.y, y3.y, s[7]);
              }
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) s[k] += __shfl_xor_sync(0xffffffffu, s[k], 1);
            if (valid && (e & 1) == 0) {
              if (p.round_z) {
#pragma unroll
                for (int k = 0; k < 8; ++k) s[k] = round_clamp_i8(s[k]);
              }
              uint4 o;
              o.x = pack16x2<BF16>(s[0], s[1]); o.y = pack16x2<BF16>(s[2], s[3]);
              o.z = pack16x2<BF16>(s[4], s[5]); o.w = pack16x2<BF16>(s[6], s[7]);
              *reinterpret_cast<uint4*>(zbuf + (v >> 3) * kABoxBytes + sw128(n, v & 7)) = o;
            }
          }
        }
        consumer_bar();  // zbuf complete; this CTA no longer reads its peers' ybuf
        if (ctid == 0) BLR_STAMP(4);
        if (ctid < nb && !SUB) mbar_arrive_remote_relaxed(mapa_shared(read_done, ctid));  // (sub-slice: done above)
      }
    }
    if (ctid == 0) BLR_STAMP(5);
    // ---- the last slice to finish a block converts it
    __threadfence();
    consumer_bar();
    if (ctid == 0) BLR_STAMP(6);
    if (ctid == 0) {
      int last = 0;
      if (!*abort_flag) {
        const unsigned prev = atomicAdd(p.counters + part * nb + blk, 1u);
        last = prev == (unsigned)p.nslices - 1 ? 1 : 0;
      } else {
        atomicExch(p.status, 1u);
      }
      *last_flag = last;
    }
    consumer_bar();
    if (*last_flag) {
      __threadfence();
      // one output row per thread and step, three steps in flight: the fp32 partial sums of a row are NP
      // consecutive floats, so the loads are whole 32-byte sectors and do not wait on one another
      const __half* usc = GS ? nullptr : ph1.scale;  // grouped scales were applied before the reduction
      constexpr int kRowsInFlight = 3, kV4 = NP / 4;
      for (int q0 = q_lo + ctid; q0 < q_hi; q0 += kRowsInFlight * kConsumerWarps * 32) {
        float4 v[kRowsInFlight][kV4];
        float sc[kRowsInFlight];
#pragma unroll
        for (int i = 0; i < kRowsInFlight; ++i) {
          const int q = q0 + i * kConsumerWarps * 32;
          sc[i] = 1.f;
          if (q < q_hi) {
            const float4* src = reinterpret_cast<const float4*>(p.out32 + ((long long)blk * p.Q + q) * NP);
#pragma unroll
            for (int k = 0; k < kV4; ++k) v[i][k] = __ldcg(src + k);
            if (usc) sc[i] = __half2float(__ldg(usc + (long long)blk * p.Q + q));
          }
        }
#pragma unroll
        for (int i = 0; i < kRowsInFlight; ++i) {
          const int q = q0 + i * kConsumerWarps * 32;
          if (q < q_hi) {
            float4* src = reinterpret_cast<float4*>(p.out32 + ((long long)blk * p.Q + q) * NP);
#pragma unroll
            for (int k = 0; k < kV4; ++k) {
              src[k] = make_float4(0.f, 0.f, 0.f, 0.f);
              const float e4[4] = {v[i][k].x, v[i][k].y, v[i][k].z, v[i][k].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int n = k * 4 + e;
                if (n < p.N) store16<BF16>(p.out, (long long)n * p.ldo + blk * p.out_blk + q * p.out_q, e4[e] * sc[i]);
              }
            }
          }
        }
      }
      if (ctid == 0) p.counters[part * nb + blk] = 0u;
    }
    if (ctid == 0) BLR_STAMP(7);
    // ---- peers may still be reading this CTA's ybuf: stay until all of them are done
    mbar_wait_cluster(read_done, 0, abort_flag);
  }
  __syncthreads();
  if (threadIdx.x == 0) BLR_STAMP(8);
#undef BLR_STAMP
  // No CTA leaves while a peer may still read its ybuf, write its zbuf or arrive on its barriers: every wait above
  // is bounded, so every thread of the cluster gets here, also after a time-out.
  cluster_sync_all();
}

// ------------------------------------------------------------------ host side
size_t cluster_smem_bytes(const ClusterParams& p, int np) {
  return (size_t)p.nstages * p.stage_bytes + (size_t)np * p.rs * 2 + 16 * p.rs * 2 + (size_t)np * p.rs * 2 + (p.rs / 64) * np * 128 + 40 * 8 + 1024;
}

template <bool BF16, int NT, bool GS, int XCH>
static int cluster_capacity_impl(int b, int smem_bytes) {
  DeviceInfo di;
  if (device_info(&di) != BLR_OK) return 0;
  auto kern = blr_blast_cluster_kernel<BF16, NT, GS, XCH>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem_optin) != cudaSuccess) return 0;
  if (b > 8 && cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(b, 1, 1);
  cfg.blockDim = dim3(kClusterThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = b;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, (const void*)kern, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

// Resident clusters of b CTAs when every CTA takes smem_bytes of dynamic shared memory; the answer depends on
// whether one or two CTAs fit an SM, so it is cached for those two classes of size.
int cluster_capacity(int b, int is_bf16, int variant, int n_tokens, int smem_bytes) {
  static int cache[64][17][2][3][2];
  static bool have[64][17][2][3][2] = {};
  DeviceInfo di;
  int dev = 0;
  if (device_info(&di) != BLR_OK || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || b < 1 || b > 16) return 0;
  if (n_tokens > kClusterMaxTokens) return 0;
  // variant: 0 BLAST with per-channel scales or none, a scale-group width, kClusterVariantMonarch
  const int bf = is_bf16 ? 1 : 0, gsi = variant == kClusterVariantMonarch ? 2 : (variant ? 1 : 0), two = smem_bytes <= kClusterHalfSmem ? 1 : 0;
  if (!have[dev][b][bf][gsi][two]) {
    const int sm = two ? kClusterHalfSmem : di.max_smem_optin - 1024;
    int n;
    // all instantiations of a variant have the same launch bounds and take the shared memory they are given, so
    // the one-tile pull form stands for the others
    if (gsi == 2) n = bf ? cluster_capacity_impl<true, 1, false, kXchMonarch>(b, sm) : cluster_capacity_impl<false, 1, false, kXchMonarch>(b, sm);
    else if (gsi) n = bf ? cluster_capacity_impl<true, 1, true, kXchPull>(b, sm) : cluster_capacity_impl<false, 1, true, kXchPull>(b, sm);
    else n = bf ? cluster_capacity_impl<true, 1, false, kXchPull>(b, sm) : cluster_capacity_impl<false, 1, false, kXchPull>(b, sm);
    cache[dev][b][bf][gsi][two] = n;
    have[dev][b][bf][gsi][two] = true;
  }
  return cache[dev][b][bf][gsi][two];
}

template <bool BF16, int NT, bool GS, int XCH>
static int launch_cluster_impl(const ClusterParams& p, cudaStream_t stream) {
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != BLR_OK) return rc;
  const size_t smem = cluster_smem_bytes(p, NT * 8);
  BLR_REQUIRE((int)smem <= di.max_smem_optin, BLR_ERR_UNSUPPORTED, "needs %zu bytes of shared memory, device offers %d",
              smem, di.max_smem_optin);
  auto kern = blr_blast_cluster_kernel<BF16, NT, GS, XCH>;
  {
    // the occupancy query configured only the instantiation that stands for this one's resource class
    int dev = 0;
    BLR_CUDA_OK(cudaGetDevice(&dev));
    static bool configured[64] = {}, big_clusters[64] = {};  // per template instance
    if (!configured[dev & 63]) {
      BLR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem_optin));
      configured[dev & 63] = true;
    }
    if (p.b > 8 && !big_clusters[dev & 63]) {  // clusters of more than 8 CTAs need the function's consent
      BLR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
      big_clusters[dev & 63] = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.b, p.nslices, p.qsplit);
  cfg.blockDim = dim3(kClusterThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = p.b;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 2;
  void* args[] = {const_cast<ClusterParams*>(&p)};
  BLR_CUDA_OK(cudaLaunchKernelExC(&cfg, (const void*)kern, args));
  return BLR_OK;
}

#ifdef BLR_TIMELINE
extern unsigned long long* g_stream_timeline;
#endif

int launch_blast_cluster(const ClusterParams& p_in, int is_bf16, cudaStream_t stream) {
  ClusterParams p = p_in;
#ifdef BLR_TIMELINE
  p.timeline = g_stream_timeline;
#endif
  BLR_REQUIRE(p.N >= 1 && p.N <= kClusterMaxTokens, BLR_ERR_UNSUPPORTED, "the cluster kernel takes 1..%d tokens", kClusterMaxTokens);
  const bool gs = p.ph[0].group != 0;
#define BLR_CL(BF, NTV, GSV, X) launch_cluster_impl<BF, NTV, GSV, X>(p, stream)
  if (p.monarch) return is_bf16 ? BLR_CL(true, 1, false, kXchMonarch) : BLR_CL(false, 1, false, kXchMonarch);
  if (p.N > 8) {  // two token tiles: sub-slice coupling only (the caller has checked that it applies)
    BLR_REQUIRE(p.subslice, BLR_ERR_UNSUPPORTED, "more than 8 tokens need the sub-slice coupling");
    if (gs) return is_bf16 ? BLR_CL(true, 2, true, kXchSubslice) : BLR_CL(false, 2, true, kXchSubslice);
    return is_bf16 ? BLR_CL(true, 2, false, kXchSubslice) : BLR_CL(false, 2, false, kXchSubslice);
  }
  if (p.subslice) {
    if (gs) return is_bf16 ? BLR_CL(true, 1, true, kXchSubslice) : BLR_CL(false, 1, true, kXchSubslice);
    return is_bf16 ? BLR_CL(true, 1, false, kXchSubslice) : BLR_CL(false, 1, false, kXchSubslice);
  }
  if (gs) return is_bf16 ? BLR_CL(true, 1, true, kXchPull) : BLR_CL(false, 1, true, kXchPull);
  return is_bf16 ? BLR_CL(true, 1, false, kXchPull) : BLR_CL(false, 1, false, kXchPull);
#undef BLR_CL
}

}  // namespace blr
