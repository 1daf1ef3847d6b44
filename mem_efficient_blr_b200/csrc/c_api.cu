// C ABI: argument checking, descriptor set-up and dispatch between the weight-streaming kernel
// (N <= 16 tokens) and the tensor-core pipeline (N > 16).
#include "../../include/blr_b200.h"

#include <atomic>
#include <mutex>
#include <unordered_map>

#include "blast_cluster.h"
#include "blast_split.h"
#include "pipeline.h"
#include "stream.h"
#include "tmap.h"

namespace blr {
const char* last_error();

static constexpr size_t kCtrlBytes = 1024;  // words 0..127: grid-wide streaming kernel; 128..254: cluster kernel counters; 255: its status
static inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

struct Workspace {
  unsigned* counters;
  void* region_a;  // 4 bytes per intermediate element
  void* region_b;  // 2 bytes per intermediate element
  void* region_c;  // expanded coupling factors (only sized for more than 16 tokens)
  float* out32;    // fp32 accumulation area of the cluster kernel (kClusterOut32Bytes)
};

// Above the streaming kernels' token counts a call runs as passes over at most this many tokens, so that the two 16-bit
// intermediates of a pass (groups x tokens x width values each) stay in L2 between the kernels that write and read them
// (measured on the headline layer: 47 ns per token at 4096 tokens, 65 at 16384, 77 at 32768 in one pass), and so that
// the workspace stops growing with the token count.
static int64_t pass_tokens(int64_t groups, int64_t width) {
  const int64_t per_token = groups * width * 2;
  int64_t t = per_token > 0 ? (128ll << 20) / per_token / 256 * 256 : (1ll << 30);
  return t < 256 ? 256 : t;
}
// Tokens per pass for a call of N tokens: equal passes, multiples of 128 tokens.
static int64_t pass_size(int64_t N, int64_t groups, int64_t width) {
  const int64_t most = pass_tokens(groups, width);
  if (N <= most) return N;
  const int64_t passes = (N + most - 1) / most;
  return ((N + passes - 1) / passes + 127) / 128 * 128;
}
// Tokens the workspace is laid out for.
static int64_t ws_tokens(int64_t N, int64_t groups, int64_t width) {
  return N <= kStreamMaxTokens ? N : pass_size(N, groups, width);
}

// Third region of a workspace, above 16 tokens: BLAST's expanded coupling factors ((width / 16) matrices of
// (16 groups)^2 16-bit values); with one group (low rank) the partial results of a first stage whose contraction is cut
// into up to 16 slices, which happens up to 1024 tokens.
static size_t region_c_bytes(int64_t n_tokens, int64_t groups, int64_t width) {
  if (n_tokens <= kStreamMaxTokens) return 0;
  const size_t c = (size_t)groups * groups * ((size_t)width + 16) * 32;
  if (groups != 1) return c;
  const int64_t t = ws_tokens(n_tokens, groups, width);
  const size_t parts = (size_t)16 * (size_t)(t < 1024 ? t : 1024) * (size_t)width * 2;
  return parts > c ? parts : c;
}

static int carve(void* ws, size_t ws_bytes, int64_t N, int64_t groups, int64_t width, Workspace* w) {
  const size_t need = blr_workspace_bytes(N, groups, width);
  N = ws_tokens(N, groups, width);
  BLR_REQUIRE(ws != nullptr && ws_bytes >= need, BLR_ERR_WORKSPACE, "workspace of %zu bytes needed, got %zu", need,
              ws == nullptr ? (size_t)0 : ws_bytes);
  BLR_REQUIRE((reinterpret_cast<uintptr_t>(ws) & 255) == 0, BLR_ERR_ALIGN, "workspace must be 256-byte aligned");
  uint8_t* p = static_cast<uint8_t*>(ws);
  w->counters = reinterpret_cast<unsigned*>(p);
  w->out32 = reinterpret_cast<float*>(p + kCtrlBytes);  // fixed place and size: it has to stay zero between calls
  p += kClusterOut32Bytes;
  w->region_a = p + kCtrlBytes;
  w->region_b = p + kCtrlBytes + align256((size_t)groups * N * width * 4);
  w->region_c = static_cast<uint8_t*>(w->region_b) + align256((size_t)groups * N * width * 2);
  return BLR_OK;
}

static CUtensorMapDataType dt16(int dtype) {
  return dtype == BLR_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

// Fills the weight side of a phase.  row_stride / grp_stride (elements; 0 = packed) describe blocks that are
// column or row slices of a larger matrix: the distance between consecutive rows of a block (K-major: output
// rows; M-major: contraction rows) and between blocks.
static int phase_weights(PhaseDesc& ph, int dtype, const void* W, int layout, int wbits, int G, int M, int K,
                         int64_t row_stride = 0, int64_t grp_stride = 0) {
  ph.G = G; ph.M = M; ph.K = K; ph.kmajor = layout == BLR_W_KMAJOR; ph.wbits = wbits;
  ph.unit_rows = ph.kmajor ? 16 : 32;
  ph.tiles_per_g = (M + ph.unit_rows - 1) / ph.unit_rows;
  ph.ntiles = G * ph.tiles_per_g;
  ph.a_boxes = 16 / wbits;
  if (!ph.kmajor) {
    BLR_REQUIRE(wbits == 16, BLR_ERR_UNSUPPORTED, "quantised factors must have the contraction index contiguous");
    BLR_REQUIRE(M % 8 == 0, BLR_ERR_SHAPE, "block output width %d must be a multiple of 8", M);
    const uint64_t dims[3] = {(uint64_t)M, (uint64_t)K, (uint64_t)G};
    const uint64_t str[2] = {(uint64_t)(row_stride ? row_stride : M) * 2, (uint64_t)(grp_stride ? grp_stride : (int64_t)M * K) * 2};
    const uint32_t box[3] = {32, 64, 1};
    ph.nchunks = (K + 63) / 64;
    return encode_tmap_3d(&ph.tmW[0], dt16(dtype), W, dims, str, box, Swz::B64);
  }
  // contraction index contiguous: rows of kb bytes, 128 bytes of every row per stage
  const int kb = wbits == 16 ? K * 2 : (wbits == 8 ? K : K / 2);
  BLR_REQUIRE(kb % 16 == 0 && (wbits != 4 || K % 2 == 0), BLR_ERR_SHAPE,
              "weight rows must be multiples of 16 bytes: contraction length %d must be a multiple of 8 (16-bit), 16 (int8) or 32 (int4)", K);
  const uint64_t inner = wbits == 16 ? (uint64_t)K : (uint64_t)kb;
  const uint64_t dims[3] = {inner, (uint64_t)M, (uint64_t)G};
  BLR_REQUIRE((row_stride == 0 && grp_stride == 0) || wbits == 16, BLR_ERR_UNSUPPORTED, "strided blocks are 16-bit only");
  const uint64_t str[2] = {row_stride ? (uint64_t)row_stride * 2 : (uint64_t)kb,
                           grp_stride ? (uint64_t)grp_stride * 2 : (uint64_t)M * kb};
  ph.nchunks = (kb + 127) / 128;
  const CUtensorMapDataType dt = wbits == 16 ? dt16(dtype) : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  for (int h = 1; h <= 8; ++h) {
    const uint32_t box[3] = {wbits == 16 ? 64u : 128u, (uint32_t)(16 * h), 1};
    int rc = encode_tmap_3d(&ph.tmW[h - 1], dt, W, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  return BLR_OK;
}

// Activation side: A[g][n][k] with element strides (1, ld_n, ld_g).
static int phase_acts(PhaseDesc& ph, int dtype, const void* A, int K, int64_t N, int G, int64_t ld_n, int64_t ld_g) {
  BLR_REQUIRE(ld_n % 8 == 0 && ld_g % 8 == 0, BLR_ERR_ALIGN,
              "activation strides (%lld, %lld elements) must be multiples of 8", (long long)ld_n, (long long)ld_g);
  const uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)G};
  const uint64_t str[2] = {(uint64_t)ld_n * 2, (uint64_t)(G > 1 ? ld_g : ld_n * N) * 2};
  const uint32_t box[3] = {64, (uint32_t)(N <= 8 ? 8 : 16), 1};
  return encode_tmap_3d(&ph.tmA, dt16(dtype), A, dims, str, box, Swz::B128);
}

static void phase_out(PhaseDesc& ph, void* out, int out_f32, long long os_g, long long os_n, int per, long long os_hi,
                      long long os_lo, const void* scale, int round_out) {
  ph.out = out; ph.out_f32 = out_f32; ph.os_g = os_g; ph.os_n = os_n; ph.per = per; ph.os_hi = os_hi; ph.os_lo = os_lo;
  ph.scale = static_cast<const __half*>(scale); ph.round_out = round_out;
}

static void finish_params(StreamParams& p, int64_t N) {
  p.N = (int)N;
  const int nb = N <= 8 ? 8 : 16;
  DeviceInfo di;
  const int grid = device_info(&di) == BLR_OK && di.sm_count > 0 ? di.sm_count : 148;
  int wmax = 0, amax = 0;
  for (int i = 0; i < p.nphases; ++i) {
    PhaseDesc& ph = p.ph[i];
    // two K-chunks per ring stage halve the producer/consumer hand-offs; one when K is a single chunk
    ph.ks = ph.nchunks >= 2 ? 2 : 1;
    ph.sub_bytes = kSubBytes;
    if (ph.kmajor) {
      // A CTA with few 16-row groups per batch (few output rows, long contraction) would move 2 KB per group and
      // chunk: pack the chunks of a stage densely and take more of them, up to about 32 KB of weights per stage,
      // as long as the activation producer does not have to issue more than 8 boxes per stage.
      int per_cta = (ph.ntiles + grid - 1) / grid;
      if (per_cta > ph.tiles_per_g) per_cta = ph.tiles_per_g;
      if (per_cta > kBatchRows / 16) per_cta = kBatchRows / 16;
      if (per_cta < 1) per_cta = 1;
      ph.sub_bytes = per_cta * 16 * 128;
      while (ph.ks < 8 && ph.ks * 2 <= ph.nchunks && ph.ks * 2 * ph.sub_bytes <= 32768 && ph.ks * 2 * ph.a_boxes <= 8) ph.ks *= 2;
    }
    ph.nstage_chunks = (ph.nchunks + ph.ks - 1) / ph.ks;
    wmax = ph.ks * ph.sub_bytes > wmax ? ph.ks * ph.sub_bytes : wmax;
    const int a = ph.ks * ph.a_boxes * nb * 128;
    amax = a > amax ? a : amax;
  }
  p.w_bytes = wmax;
  p.stage_bytes = wmax + amax;
  p.mix_bytes = 0;
  if (p.mix) {
    // the coupling keeps [b][nv] vectors of 8 floats per CTA; nv = its share of the N*R/8 vectors
    const long long nvec = ((long long)N * p.R) / 8;
    const long long nv_max = nvec / 128 + 2;  // grids have at least 128 CTAs on the parts this targets
    p.mix_bytes = (int)(((long long)p.b * nv_max * 32 + 1023) / 1024 * 1024);
  }
  const int budget = 232448 - kStreamTailBytes - p.mix_bytes;
  int nst = budget / p.stage_bytes;
  p.nstages = nst > 16 ? 16 : nst;
}

// Returns 1 for an empty batch (nothing to do, not an error), 0 when the call may proceed, < 0 on error.
static int check_common(const void* x, int64_t ldx, int64_t N, int dtype, const void* out, int64_t ldo) {
  BLR_REQUIRE(N >= 0, BLR_ERR_ARG, "token count must not be negative, got %lld", (long long)N);
  if (N == 0) return 1;
  BLR_REQUIRE(x != nullptr && out != nullptr, BLR_ERR_ARG, "x and out must not be null");
  BLR_REQUIRE(dtype == BLR_DTYPE_F16 || dtype == BLR_DTYPE_BF16, BLR_ERR_ARG, "unknown dtype %d", dtype);
  BLR_REQUIRE(ldx > 0 && ldo > 0, BLR_ERR_ARG, "leading dimensions must be positive");
  return BLR_OK;
}
static int check_layout(int layout) {
  BLR_REQUIRE(layout == BLR_W_KMAJOR || layout == BLR_W_MMAJOR, BLR_ERR_ARG, "unknown weight layout %d", layout);
  return BLR_OK;
}

// ---------------------------------------------------------------------------------- BLAST (16-bit and quantised)
static constexpr int kSubsliceMinTokens = 4;
// 0: automatic, 1: grid-wide streaming kernel only, 2: no two-launch path (cluster kernel where it applies)
static std::atomic<int> g_decode_path{0};

// Set around the kernels of a host-buffer call: such calls are bound by the rate at which the host can enqueue work (two
// copies, event operations and the launches per call), not by the GPU, so the extra launch that converts x once per call
// costs them more than the conversion it saves.
static thread_local bool t_host_call = false;

// One layer of a two-launch call (all layers of a call share x, the shapes and the strides of S).
struct SplitLayer {
  const void *U, *u_scale, *V, *v_scale, *S, *bias, *residual;
  void* out;
  int64_t ldo, ldr;
  int64_t v_row = 0, v_blk = 0;  // V as column blocks of a wider matrix: elements between rows / blocks (0: packed)
  int monarch = 0, mon_torch = 0, out_interleaved = 0;  // Monarch on the same kernels: permuted hand-over instead of coupling
};

// Two-launch path (blast_split.cu): returns 0 when launched, 1 when the call does not fit it, < 0 on error.
// `zbase` is 16-bit scratch for nprob * bo * N * R values.
static int split_blast_multi(const void* x, int64_t ldx, const void* x_mul, int act, int64_t N, int dtype, int nprob,
                             const SplitLayer* layers, int u_layout, int v_layout, int wb, int group, int64_t s_i, int64_t s_j,
                             int64_t s_r, int b, int bo, int P, int Q, int R, int act8, void* zbase, unsigned* status,
                             cudaStream_t stream, void* xscratch = nullptr, size_t xscratch_bytes = 0,
                             bool may_decline = false) {
  // Measured against the cluster kernel on the Llama-7B shapes, the two-launch path wins at every token count it
  // takes (1..16) with 16-bit, int8 and packed int4 factors.
  if (g_decode_path.load(std::memory_order_relaxed) != 0 || N > kStreamMaxTokens) return 1;
  if (u_layout != BLR_W_KMAJOR || v_layout != BLR_W_KMAJOR || b > kSplitMaxBlocks || nprob < 1 || nprob > kSplitMaxProblems) return 1;
  const long long kbV = (long long)P * wb / 8, kbU = (long long)R * wb / 8;
  if (R % kSplitRanks != 0 || P % 8 != 0 || kbV % 16 != 0 || kbU % 16 != 0 || (wb == 4 && ((P | R) & 1))) return 1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || ldx % 8 != 0) return 1;
  if (act != kSplitActNone && (x_mul == nullptr || (reinterpret_cast<uintptr_t>(x_mul) & 15) != 0)) return 1;
  if (group != 0 && (group != kScaleGroup || P % kScaleGroup != 0 || R % kScaleGroup != 0)) return 1;
  if (wb != 16 && (P > 2048 || R > 2048)) return 1;  // a warp holds a whole activation row in registers while it scales it
  DeviceInfo di;
  int rc;
  if ((rc = device_info(&di))) return rc;
  SplitParams p = {};
  p.x = x; p.x_mul = x_mul; p.act = act; p.nprob = nprob; p.status = status;
  p.ldx = ldx; p.s_i = s_i; p.s_j = s_j; p.s_r = s_r;
  p.N = (int)N; p.b = b; p.bo = bo; p.P = P; p.Q = Q; p.R = R;
  p.wbits = wb; p.group = group; p.round_y = act8; p.round_z = act8;
  p.monarch = layers[0].monarch; p.mon_torch = layers[0].mon_torch; p.mon_per = R / b; p.out_interleaved = layers[0].out_interleaved;
  p.z_shared = (nprob == 1 && layers[0].S == nullptr && !p.monarch) ? 1 : 0;
  p.nch0 = (int)((kbV + 127) / 128);
  p.nch1 = (int)((kbU + 127) / 128);
  // back kernel: every CTA a run of 16-row groups of one out-block, about one CTA per SM over all layers of the call
  const int gpb = (Q + 15) / 16;
  int cpb = di.sm_count / (bo * nprob);
  if (cpb < 1) cpb = 1;
  if (cpb > gpb) cpb = gpb;
  p.gpc = (gpb + cpb - 1) / cpb;
  p.cpb = (gpb + p.gpc - 1) / p.gpc;
  auto magic = [](int d) { return d <= 1 ? 0u : (unsigned)((0x100000000ull + (unsigned)d - 1) / (unsigned)d); };
  p.magic_N = magic((int)N); p.magic_rows = magic(p.gpc * 8);
  if ((long long)b * N >= 65536 || (long long)p.gpc * 16 * N >= 65536) return 1;
  // quantised factors, more than 2 tokens or an input transform: x is transformed and converted to fixed point once,
  // by a launch of its own, instead of by every front CTA
  if (wb != 16 && (N > 2 || act != kSplitActNone) && xscratch != nullptr) {
    const size_t pitch = split_fx_row_bytes(P, wb);
    const size_t rows_bytes = align256((size_t)b * N * pitch);
    if (rows_bytes + (size_t)b * N * 4 <= xscratch_bytes) {
      p.xq = xscratch;
      p.xq_scale = reinterpret_cast<float*>(static_cast<uint8_t*>(xscratch) + rows_bytes);
    }
  }
  p.nstages = 2;
  const int fs = (int)split_front_smem(p);
  if (fs > di.max_smem_optin) return 1;
  // A front grid that needs two waves (ranks beyond 8 x SMs x the CTAs that fit an SM: rank 1488 with many tokens or
  // long input blocks) loses to the cluster kernel from 4 tokens on (measured: int8 down projection, 4 tokens, 20.5 vs
  // 15.8 us; fp16 gate projection, 16 tokens, 27.6 vs 24.8); callers that have that alternative take it.
  if (may_decline && N >= 4) {
    int per_sm = (227 * 1024) / fs;
    if (per_sm < 1) per_sm = 1;
    if ((long long)(R / kSplitRanks) * nprob > (long long)di.sm_count * per_sm) return 1;
  }
  // ring of the back kernel: the CTA's whole share if it fits beside a front CTA of the next call on the same SM
  // (228 KB per SM, 1 KB of it reserved per CTA), else what fits, but never fewer than 4 stages
  const int nseg = (p.nch1 + kSplitStageChunks - 1) / kSplitStageChunks, total = p.gpc * nseg;
  const int other = (int)split_back_smem(p) - 2 * kSplitStageBytes;
  int nst = (228 * 1024 - 2048 - fs - other) / kSplitStageBytes;
  if (nst < 4) nst = 4;
  if (nst > total) nst = total;
  if (nst > (di.max_smem_optin - other) / kSplitStageBytes) nst = (di.max_smem_optin - other) / kSplitStageBytes;
  if (nst < 1 || (nst < 2 && total > 1)) return 1;
  p.nstages = nst;
  const CUtensorMapDataType dt = wb == 16 ? dt16(dtype) : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const uint32_t inner_box = wb == 16 ? 64u : 128u;
  for (int i = 0; i < nprob; ++i) {
    const SplitLayer& l = layers[i];
    SplitProblem& q = p.pr[i];
    q.S = l.S; q.v_scale = static_cast<const __half*>(l.v_scale); q.u_scale = static_cast<const __half*>(l.u_scale);
    q.z = static_cast<uint8_t*>(zbase) + (size_t)i * align256((size_t)bo * N * R * 2);
    q.out = l.out; q.ldo = l.ldo; q.bias = l.bias; q.residual = l.residual; q.ldr = l.ldr;
    {
      const uint64_t dims[3] = {wb == 16 ? (uint64_t)P : (uint64_t)kbV, (uint64_t)R, (uint64_t)b};
      const uint64_t esz = wb == 16 ? 2 : 1;  // (strided views only come with 16-bit factors)
      const uint64_t str[2] = {l.v_row ? (uint64_t)l.v_row * esz : (uint64_t)kbV, l.v_blk ? (uint64_t)l.v_blk * esz : (uint64_t)R * kbV};
      const uint32_t box[3] = {inner_box, (uint32_t)kSplitRanks, (uint32_t)b};
      if ((rc = encode_tmap_3d(&q.tmV, dt, l.V, dims, str, box, Swz::B128))) return rc;
    }
    {
      const uint64_t dims[3] = {wb == 16 ? (uint64_t)R : (uint64_t)kbU, (uint64_t)Q, (uint64_t)bo};
      const uint64_t str[2] = {(uint64_t)kbU, (uint64_t)Q * kbU};
      const uint32_t box[3] = {inner_box, 16u, 1u};
      if ((rc = encode_tmap_3d(&q.tmU, dt, l.U, dims, str, box, Swz::B128))) return rc;
    }
  }
  return launch_blast_split(p, dtype == BLR_DTYPE_BF16, stream);
}

static int split_blast(const void* x, int64_t ldx, int64_t N, int dtype, const void* U, int u_layout, int u_bits,
                       const void* u_scale, const void* V, int v_layout, int v_bits, const void* v_scale, int group, const void* S,
                       int64_t s_i, int64_t s_j, int64_t s_r, int b, int bo, int P, int Q, int R, int act8, void* out,
                       int64_t ldo, const Workspace& w, cudaStream_t stream) {
  if (u_bits != v_bits) return 1;
  const SplitLayer l = {U, u_scale, V, v_scale, S, nullptr, nullptr, out, ldo, 0};
  return split_blast_multi(x, ldx, nullptr, kSplitActNone, N, dtype, 1, &l, u_layout, v_layout, u_bits, group, s_i, s_j, s_r, b, bo,
                           P, Q, R, act8, w.region_b, w.counters + 255, stream, t_host_call ? nullptr : w.region_a,
                           (size_t)(static_cast<uint8_t*>(w.region_b) - static_cast<uint8_t*>(w.region_a)),
                           /*may_decline=*/g_decode_path.load(std::memory_order_relaxed) == 0);
}

// Cluster kernel (blast_cluster.cu): returns 0 when launched, 1 when the call does not fit it, < 0 on error.
static int cluster_blast(const void* x, int64_t ldx, int64_t N, int dtype, const void* U, int u_layout, int u_bits,
                         const void* u_scale, const void* V, int v_layout, int v_bits, const void* v_scale, int group, const void* S,
                         int64_t s_i, int64_t s_j, int64_t s_r, int b, int bo, int P, int Q, int R, int act8, void* out,
                         int64_t ldo, const Workspace& w, cudaStream_t stream, int64_t v_row = 0, int64_t v_grp = 0,
                         int64_t u_row = 0, int64_t u_grp = 0) {
  const int np = N <= 8 ? 8 : 16;
  if (g_decode_path.load(std::memory_order_relaxed) == 1 || N > kClusterMaxTokens || b > 16 || bo != b || u_bits != v_bits || R % 8 != 0) return 1;
  if ((long long)b * Q * np * 4 > kClusterOut32Bytes) return 1;
  const int bf = dtype == BLR_DTYPE_BF16;
  ClusterParams p = {};
  int rc;
  if ((rc = phase_weights(p.ph[0], dtype, V, v_layout, v_bits, b, R, P, v_row, v_grp))) return rc;
  if ((rc = phase_acts(p.ph[0], dtype, x, P, N, b, ldx, P))) return rc;
  if ((rc = phase_weights(p.ph[1], dtype, U, u_layout, u_bits, b, Q, R, u_row, u_grp))) return rc;
  p.ph[0].scale = static_cast<const __half*>(v_scale);
  p.ph[1].scale = static_cast<const __half*>(u_scale);
  p.ph[0].group = p.ph[1].group = group;
  DeviceInfo di;
  if ((rc = device_info(&di))) return rc;
  // Shape of the launch: ranks per slice (a multiple of what one second-phase chunk covers), row parts of U_i,
  // and whether two CTAs share an SM.  All clusters must be resident at once.  Among the shapes that are, a cost
  // fitted to measurements on the headline layer picks one: weight bytes per CTA (a part repeats the first phase,
  // so that term does not shrink with the parts), 20 % off when a CTA has an SM and the whole ring to itself,
  // plus the equivalent of 20 KB per slice for the reductions and the finaliser's wait.
  const int kx = p.ph[1].kmajor ? (u_bits == 16 ? 64 : (u_bits == 8 ? 128 : 256)) : 64;
  int best_rs = 0, best_parts = 1, best_two = 0;
#ifdef BLR_TIMELINE
  static const char* forced = getenv("BLR_CLUSTER_SHAPE");  // profiling builds only: "rs,parts,two"
#else
  const char* forced = nullptr;
#endif
  if (forced) {
    if (sscanf(forced, "%d,%d,%d", &best_rs, &best_parts, &best_two) != 3) return 1;
    if (best_rs % kx != 0 || best_rs < kx || best_rs > kClusterMaxSlice || best_parts < 1 || best_parts > kClusterMaxParts) return 1;
  } else {
    const int cap[2] = {cluster_capacity(b, bf, group, (int)N, di.max_smem_optin - 1024),
                        cluster_capacity(b, bf, group, (int)N, kClusterHalfSmem)};
    const int max_parts = Q / kBatchRows < 1 ? 1 : (Q / kBatchRows > kClusterMaxParts ? kClusterMaxParts : Q / kBatchRows);
    const int r_up = (R + kx - 1) / kx * kx;
    double best = -1.;
    for (int rs = kx; rs <= kClusterMaxSlice && rs <= r_up; rs += kx) {
      if (group != 0 && rs % kScaleGroup != 0) continue;
      const int nsl = (R + rs - 1) / rs;
      if ((long long)nsl * rs - R >= kx) continue;  // a last slice that is mostly padding only delays the others
      for (int two = 0; two < 2; ++two)
        for (int parts = 1; parts <= max_parts && nsl * parts <= cap[two]; ++parts) {
          const int qp = ((Q + parts - 1) / parts + 15) / 16 * 16;
          const double kb = ((double)rs * P + (double)qp * rs) * u_bits / 8. / 1024.;
          const double cost = kb * (two ? 1.0 : 0.8) + 20. * nsl;
          if (best < 0. || cost < best) { best = cost; best_rs = rs; best_parts = parts; best_two = two; }
        }
    }
    if (best < 0.) return 1;  // more slices than resident clusters at every width: grid-wide kernel
  }
  const int rs = best_rs;
  p.N = (int)N; p.b = b; p.R = R; p.Q = Q; p.rs = rs; p.nslices = (R + rs - 1) / rs;
  p.qsplit = best_parts;
  p.q_part = ((Q + best_parts - 1) / best_parts + 15) / 16 * 16;
  p.nchunks1 = rs / kx;
  // chunks per stage: two where that divides both phases' chunk counts (a chunk past the slice would read the
  // next slice's columns), else one, so that every stage of the ring carries a full load in both phases
  p.ks0 = p.ks1 = (p.nchunks1 % 2 == 0 && p.ph[0].nchunks % 2 == 0) ? 2 : 1;
  p.round_y = act8; p.round_z = act8;
  p.s_i = s_i; p.s_j = s_j; p.s_r = s_r; p.S = S;
  p.out = out; p.ldo = ldo; p.out32 = w.out32; p.counters = w.counters + 128; p.status = w.counters + 255;
  p.out_blk = Q; p.out_q = 1;
  // Coupling by rank sub-slice moves 2 N rs values per CTA through distributed shared memory instead of b N rs, at
  // the price of a second exchange step: it wins from about 4 tokens on, and is the only form for two token tiles.
  p.subslice = rs % (8 * b) == 0 && N >= kSubsliceMinTokens;
  if (N > 8 && !p.subslice) return 1;
  const int budget = best_two ? kClusterHalfSmem : di.max_smem_optin - 1024;
  for (;;) {
    p.w_bytes = p.ks0 * kSubBytes;
    p.stage_bytes = p.w_bytes + p.ks0 * p.ph[0].a_boxes * np * 128;
    p.nstages = 2;
    const int extras = (int)cluster_smem_bytes(p, np) - 2 * p.stage_bytes;
    const int nst = (budget - extras) / p.stage_bytes;
    p.nstages = nst > 16 ? 16 : nst;
    if (p.nstages >= 2) break;
    if (p.ks0 == 1) return 1;
    p.ks0 = p.ks1 = 1;  // two chunks per stage leave no room for a second stage: one chunk per stage
  }
  if (forced && p.nslices * p.qsplit > cluster_capacity(b, bf, group, (int)N, budget)) return 1;
  rc = launch_blast_cluster(p, bf, stream);
  return rc;
}

// Monarch for 1..8 tokens on the cluster kernel: the first stage's blocks that feed a slice of the second stage's
// contraction index are shared out over the cluster's CTAs, the permutation between the stages is the exchange
// through distributed shared memory, and the second stage runs like BLAST's.  Returns 0 / 1 / < 0 like cluster_blast.
static int cluster_monarch(const void* x, int64_t ldx, int64_t N, int dtype, const void* w1, int w1_layout, int grouped,
                           const void* w2, int w2_layout, int b, int P, int rank, int Qs, int interleaved, void* out,
                           int64_t ldo, const Workspace& w, cudaStream_t stream) {
  const int np = 8;
  // one token tile; the permutation is gathered element by element, which for the torch layout (stride b between a
  // CTA's elements) overtakes the grid-wide kernel's barrier from about 6 tokens on
  if (g_decode_path.load(std::memory_order_relaxed) == 1 || N > (grouped ? 8 : 5) || b > 16 || b < 2 || rank % b != 0 || rank % 8 != 0) return 1;
  if ((long long)b * Qs * np * 4 > kClusterOut32Bytes) return 1;
  const int per = rank / b, bf = dtype == BLR_DTYPE_BF16;
  DeviceInfo di;
  int rc;
  if ((rc = device_info(&di))) return rc;
  ClusterParams p = {};
  if ((rc = phase_weights(p.ph[0], dtype, w1, w1_layout, 16, b, rank, P))) return rc;
  if ((rc = phase_acts(p.ph[0], dtype, x, P, N, b, ldx, P))) return rc;
  if ((rc = phase_weights(p.ph[1], dtype, w2, w2_layout, 16, b, Qs, rank))) return rc;
  // slice = mblk whole first-stage blocks (mblk divides b), rs = mblk * per ranks, a multiple of the 64-wide K-chunk
  const int cap[2] = {cluster_capacity(b, bf, kClusterVariantMonarch, (int)N, di.max_smem_optin - 1024),
                      cluster_capacity(b, bf, kClusterVariantMonarch, (int)N, kClusterHalfSmem)};
  const int max_parts = Qs / kBatchRows < 1 ? 1 : (Qs / kBatchRows > kClusterMaxParts ? kClusterMaxParts : Qs / kBatchRows);
  int best_m = 0, best_parts = 1, best_two = 0;
  double best = -1.;
  for (int m = 1; m <= b; ++m) {
    if (b % m != 0) continue;
    const int rs = m * per;
    if (rs % 64 != 0 || rs > kClusterMaxSlice) continue;
    const int nsl = b / m;
    for (int two = 0; two < 2; ++two)
      for (int parts = 1; parts <= max_parts && nsl * parts <= cap[two]; ++parts) {
        const int qp = ((Qs + parts - 1) / parts + 15) / 16 * 16;
        const double kb = ((double)rs * P + (double)qp * rs) * 2. / 1024.;
        // beyond about 300 KB of weights per CTA the grid-wide kernel (all SMs, one barrier for Monarch) is as fast
        if (kb > 300.) continue;
        const double cost = kb * (two ? 1.0 : 0.8) + 20. * nsl;
        if (best < 0. || cost < best) { best = cost; best_m = m; best_parts = parts; best_two = two; }
      }
  }
  if (best < 0.) return 1;
  const int rs = best_m * per;
  p.N = (int)N; p.b = b; p.R = rank; p.Q = Qs; p.rs = rs; p.nslices = b / best_m;
  p.qsplit = best_parts;
  p.q_part = ((Qs + best_parts - 1) / best_parts + 15) / 16 * 16;
  p.nchunks1 = rs / 64;
  p.ks0 = p.ks1 = (p.nchunks1 % 2 == 0 && p.ph[0].nchunks % 2 == 0) ? 2 : 1;
  p.monarch = 1; p.mblk = best_m; p.cpb = b / best_m; p.per = per; p.w1_grouped = grouped;
  p.out_blk = interleaved ? 1 : Qs; p.out_q = interleaved ? b : 1;
  p.out = out; p.ldo = ldo; p.out32 = w.out32; p.counters = w.counters + 128; p.status = w.counters + 255;
  p.w_bytes = p.ks0 * kSubBytes;
  p.stage_bytes = p.w_bytes + p.ks0 * p.ph[0].a_boxes * np * 128;
  p.nstages = 2;
  const int extras = (int)cluster_smem_bytes(p, np) - 2 * p.stage_bytes;
  const int budget = best_two ? kClusterHalfSmem : di.max_smem_optin - 1024;
  int nst = (budget - extras) / p.stage_bytes;
  p.nstages = nst > 16 ? 16 : nst;
  if (p.nstages < 2) return 1;
  return launch_blast_cluster(p, bf, stream);
}

static int blast_impl(const void* x, int64_t ldx, int64_t N, int dtype, const void* U, int u_layout, int u_bits,
                      const void* u_scale, const void* V, int v_layout, int v_bits, const void* v_scale, int group, const void* S,
                      int64_t s_i, int64_t s_j, int64_t s_r, int b, int bo, int P, int Q, int R, int flags, void* out,
                      int64_t ldo, void* ws, size_t ws_bytes, cudaStream_t stream, const void* e_ready = nullptr,
                      const void* bias = nullptr, const void* residual = nullptr, int64_t ldr = 0, int out_act = 0) {
  // (bias / residual: added by the last GEMM above 16 tokens; callers with fewer tokens use the two-launch path's own)
  int rc = check_common(x, ldx, N, dtype, out, ldo);
  if (rc) return rc < 0 ? rc : BLR_OK;
  BLR_REQUIRE(U && V && S, BLR_ERR_ARG, "factor pointers must not be null");
  BLR_REQUIRE((reinterpret_cast<uintptr_t>(S) & 15) == 0, BLR_ERR_ALIGN, "S must be 16-byte aligned");
  BLR_REQUIRE(b >= 2, BLR_ERR_SHAPE, "BLAST needs at least 2 blocks per side, got %d (the reference asserts b != 1)", b);
  BLR_REQUIRE(P > 0 && Q > 0 && R > 0, BLR_ERR_SHAPE, "P, Q, R must be positive");
  BLR_REQUIRE(bo >= 1 && bo <= b, BLR_ERR_SHAPE, "output blocks held by this call (%d) must be in 1..%d", bo, b);
  BLR_REQUIRE(ldx >= (int64_t)b * P && ldo >= (int64_t)bo * Q, BLR_ERR_SHAPE, "leading dimensions shorter than a row");
  if ((rc = check_layout(u_layout)) || (rc = check_layout(v_layout))) return rc;
  Workspace w;
  if ((rc = carve(ws, ws_bytes, N, b, R, &w))) return rc;
  const int act8 = (flags & BLR_FLAG_ACT_INT8) ? 1 : 0;

  if (N <= kStreamMaxTokens) {
    rc = split_blast(x, ldx, N, dtype, U, u_layout, u_bits, u_scale, V, v_layout, v_bits, v_scale, group, S, s_i, s_j, s_r, b, bo,
                     P, Q, R, act8, out, ldo, w, stream);
    if (rc <= 0) return rc;  // 0: launched, < 0: error, 1: not applicable -> cluster kernel
    rc = cluster_blast(x, ldx, N, dtype, U, u_layout, u_bits, u_scale, V, v_layout, v_bits, v_scale, group, S, s_i, s_j, s_r, b, bo,
                       P, Q, R, act8, out, ldo, w, stream);
    if (rc <= 0) return rc;  // 1: not applicable -> grid-wide streaming kernel
    StreamParams p = {};
    p.nphases = 2; p.mix = 1; p.b = b; p.b_out = bo; p.R = R; p.round_z = act8;
    p.s_i = s_i; p.s_j = s_j; p.s_r = s_r; p.S = S;
    p.y32 = static_cast<float*>(w.region_a); p.z16 = w.region_b; p.counters = w.counters;
    if ((rc = phase_weights(p.ph[0], dtype, V, v_layout, v_bits, b, R, P))) return rc;
    if ((rc = phase_acts(p.ph[0], dtype, x, P, N, b, ldx, P))) return rc;
    phase_out(p.ph[0], w.region_a, 1, (long long)N * R, R, R, 0, 1, v_scale, act8);
    if ((rc = phase_weights(p.ph[1], dtype, U, u_layout, u_bits, bo, Q, R))) return rc;
    if ((rc = phase_acts(p.ph[1], dtype, w.region_b, R, N, bo, R, (int64_t)N * R))) return rc;
    phase_out(p.ph[1], out, 0, Q, ldo, Q, 0, 1, u_scale, 0);
    p.ph[0].group = p.ph[1].group = group;
    finish_params(p, N);
    return launch_stream(p, dtype == BLR_DTYPE_BF16, stream);
  }
  // quantised factors stay quantised in global memory: the GEMMs widen the tiles they stage
  const BlastQuant quant = {u_bits, v_bits, group, u_scale, v_scale};
  const int64_t per_pass = pass_size(N, b, R);
  for (int64_t n0 = 0; n0 < N; n0 += per_pass) {
    const int64_t n = N - n0 < per_pass ? N - n0 : per_pass;
    rc = pipeline_blast(static_cast<const uint8_t*>(x) + n0 * ldx * 2, ldx, n, dtype, U, u_layout, V, v_layout, S, s_i, s_j, s_r, b,
                        bo, P, Q, R, act8, static_cast<uint8_t*>(out) + n0 * ldo * 2, ldo, w.region_a, w.region_b, w.region_c, stream,
                        e_ready, u_bits != 16 || v_bits != 16 ? &quant : nullptr, bias,
                        residual ? static_cast<const uint8_t*>(residual) + n0 * ldr * 2 : nullptr, ldr, out_act);
    if (rc) return rc;
  }
  return BLR_OK;
}

// ---------------------------------------------------------------------------------- fixed scratch for blr_blast_static
// Scratch of the streaming kernel (control words, fp32 y, 16-bit z) for callers that cannot hand over a
// workspace.  The array lives in every device's copy of this module from load to exit.
static constexpr size_t kStaticScratchBytes = 4u << 20;  // 4 MiB, 2 MiB + 1 KiB of it the fixed head: b * n_tokens * R up to about 349 000
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of the array on the current device.  In host code `g_static_scratch` is only a handle
// for the runtime, not an address a kernel could use, so it is resolved once per device with
// cudaGetSymbolAddress while that device is current.
static int static_scratch_ptr(void** out) {
  static void* ptrs[64] = {};
  static std::mutex mu;
  int dev = 0;
  BLR_CUDA_OK(cudaGetDevice(&dev));
  BLR_REQUIRE(dev >= 0 && dev < 64, BLR_ERR_ARG, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    BLR_CUDA_OK(cudaGetSymbolAddress(&p, g_static_scratch));
    BLR_REQUIRE(p != nullptr, BLR_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return BLR_OK;
}

}  // namespace blr

using namespace blr;

extern "C" {

int blr_version(void) { return 100; }
#ifdef BLR_TIMELINE
int blr_debug_stream_timeline(void* dev_ptr) {  // profiling builds only, not part of the shipped ABI
  set_stream_timeline(static_cast<unsigned long long*>(dev_ptr));
  return BLR_OK;
}
#endif
int blr_debug_decode_path(int which) {
  BLR_REQUIRE(which >= 0 && which <= 2, BLR_ERR_ARG,
              "decode path must be 0 (automatic), 1 (grid-wide kernel) or 2 (cluster kernel before the grid-wide one)");
  g_decode_path.store(which, std::memory_order_relaxed);
  return BLR_OK;
}
const char* blr_last_error(void) { return blr::last_error(); }

size_t blr_workspace_bytes(int64_t n_tokens, int64_t groups, int64_t width) {
  if (n_tokens < 0 || groups < 0 || width < 0) return 0;
  const size_t e = (size_t)groups * (size_t)ws_tokens(n_tokens, groups, width) * (size_t)width;
  return kCtrlBytes + kClusterOut32Bytes + align256(e * 4) + align256(e * 2) + align256(region_c_bytes(n_tokens, groups, width));
}

void* blr_scratch_alloc(size_t bytes) {
  void* p = nullptr;
  const cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) {
    set_last_error("cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    return nullptr;
  }
  return p;
}

int blr_scratch_free(void* p) {
  BLR_CUDA_OK(cudaFree(p));
  return BLR_OK;
}

int blr_workspace_init(void* ws, size_t ws_bytes, void* stream) {
  BLR_REQUIRE(ws != nullptr && ws_bytes >= kCtrlBytes + kClusterOut32Bytes, BLR_ERR_WORKSPACE, "workspace too small");
  BLR_CUDA_OK(cudaMemsetAsync(ws, 0, kCtrlBytes + kClusterOut32Bytes, static_cast<cudaStream_t>(stream)));
  return BLR_OK;
}

int blr_workspace_status(const void* ws, void* stream) {
  BLR_REQUIRE(ws != nullptr, BLR_ERR_WORKSPACE, "workspace is null");
  unsigned words[256] = {};
  BLR_CUDA_OK(cudaMemcpyAsync(words, ws, sizeof(words), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  BLR_CUDA_OK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  if (words[3] != 0 || words[255] != 0) {
    set_last_error("a kernel gave up on a device-side wait (status word %u)", words[3]);
    return BLR_ERR_TIMEOUT;
  }
  return BLR_OK;
}

int blr_blast(const void* x, int64_t ldx, int64_t n_tokens, int dtype, const void* U, int u_layout, const void* V,
              int v_layout, const void* S, int64_t s_i, int64_t s_j, int64_t s_r, int b, int P, int Q, int R, int flags,
              void* out, int64_t ldo, void* ws, size_t ws_bytes, void* stream) {
  return blast_impl(x, ldx, n_tokens, dtype, U, u_layout, 16, nullptr, V, v_layout, 16, nullptr, 0, S, s_i, s_j, s_r, b, b, P,
                    Q, R, flags, out, ldo, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}

int blr_blast_rows(const void* x, int64_t ldx, int64_t n_tokens, int dtype, const void* U, int u_layout, const void* V,
                   int v_layout, const void* S, int64_t s_i, int64_t s_j, int64_t s_r, int b, int b_out, int P, int Q, int R,
                   int flags, void* out, int64_t ldo, void* ws, size_t ws_bytes, void* stream) {
  return blast_impl(x, ldx, n_tokens, dtype, U, u_layout, 16, nullptr, V, v_layout, 16, nullptr, 0, S, s_i, s_j, s_r, b, b_out,
                    P, Q, R, flags, out, ldo, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}

size_t blr_blast_coupling_bytes(int b, int b_out, int R) { return b >= 1 && b_out >= 1 && R > 0 ? pipeline_coupling_bytes(b, b_out, R) : 0; }

int blr_blast_expand_coupling(const void* S, int64_t s_i, int64_t s_j, int64_t s_r, int b, int b_out, int R, int dtype, void* E,
                              size_t E_bytes, void* stream) {
  BLR_REQUIRE(S && E, BLR_ERR_ARG, "null pointer");
  BLR_REQUIRE(dtype == BLR_DTYPE_F16 || dtype == BLR_DTYPE_BF16, BLR_ERR_ARG, "unknown dtype %d", dtype);
  BLR_REQUIRE(b >= 2 && b_out >= 1 && b_out <= b && R > 0, BLR_ERR_SHAPE, "bad dimensions");
  const size_t need = pipeline_coupling_bytes(b, b_out, R);
  BLR_REQUIRE(need > 0, BLR_ERR_UNSUPPORTED, "the coupling of b = %d, R = %d does not use expanded factors", b, R);
  BLR_REQUIRE(E_bytes >= need && (reinterpret_cast<uintptr_t>(E) & 255) == 0, BLR_ERR_WORKSPACE,
              "expanded coupling factors need %zu bytes, 256-byte aligned", need);
  return pipeline_expand_coupling(S, s_i, s_j, s_r, b, b_out, R, dtype, E, static_cast<cudaStream_t>(stream));
}

int blr_blast_rows_prepared(const void* x, int64_t ldx, int64_t n_tokens, int dtype, const void* U, int u_layout, const void* V,
                            int v_layout, const void* S, int64_t s_i, int64_t s_j, int64_t s_r, int b, int b_out, int P, int Q,
                            int R, int flags, void* out, int64_t ldo, void* ws, size_t ws_bytes, void* stream, const void* E) {
  return blast_impl(x, ldx, n_tokens, dtype, U, u_layout, 16, nullptr, V, v_layout, 16, nullptr, 0, S, s_i, s_j, s_r, b, b_out,
                    P, Q, R, flags, out, ldo, ws, ws_bytes, static_cast<cudaStream_t>(stream), E);
}

int blr_blast_static(const void* x, int64_t ldx, int64_t n_tokens, int dtype, const void* U, int u_layout, const void* V,
                     int v_layout, const void* S, int64_t s_i, int64_t s_j, int64_t s_r, int b, int P, int Q, int R,
                     int flags, void* out, int64_t ldo, void* stream) {
  BLR_REQUIRE(n_tokens >= 1 && n_tokens <= kStreamMaxTokens, BLR_ERR_UNSUPPORTED,
              "blr_blast_static handles 1..%d tokens per call, got %lld", kStreamMaxTokens, (long long)n_tokens);
  BLR_REQUIRE(b >= 2 && R > 0, BLR_ERR_SHAPE, "bad dimensions");
  const size_t need = blr_workspace_bytes(n_tokens, b, R);
  BLR_REQUIRE(need <= kStaticScratchBytes, BLR_ERR_WORKSPACE,
              "blr_blast_static: b * n_tokens * R = %lld needs %zu bytes of scratch, the built-in array holds %zu",
              (long long)b * n_tokens * R, need, kStaticScratchBytes);
  void* ws = nullptr;
  int rc = static_scratch_ptr(&ws);  // first call on a device: resolves the array's address
  if (rc) return rc;
  // The array keeps whatever the previous call left.  The control words and the part of the fp32 accumulation
  // area this shape can touch must start at zero; the kernels leave them zero, but a call that gave up on a wait
  // does not, and this entry point has no separate init call.
  // The two status words (3 and 255) are left alone: they keep a time-out until blr_blast_static_status reads it.
  size_t head = (size_t)b * Q * 16 * sizeof(float);
  if (head > (size_t)kClusterOut32Bytes) head = kClusterOut32Bytes;
  uint8_t* wp = static_cast<uint8_t*>(ws);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BLR_CUDA_OK(cudaMemsetAsync(wp, 0, 3 * sizeof(unsigned), st));
  BLR_CUDA_OK(cudaMemsetAsync(wp + 4 * sizeof(unsigned), 0, 251 * sizeof(unsigned), st));
  BLR_CUDA_OK(cudaMemsetAsync(wp + kCtrlBytes, 0, head, st));
  return blast_impl(x, ldx, n_tokens, dtype, U, u_layout, 16, nullptr, V, v_layout, 16, nullptr, 0, S, s_i, s_j, s_r, b, b, P,
                    Q, R, flags, out, ldo, ws, kStaticScratchBytes, static_cast<cudaStream_t>(stream));
}

int blr_blast_static_status(void* stream) {
  void* ws = nullptr;
  int rc = static_scratch_ptr(&ws);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned words[256] = {};
  BLR_CUDA_OK(cudaMemcpyAsync(words, ws, sizeof(words), cudaMemcpyDeviceToHost, st));
  BLR_CUDA_OK(cudaStreamSynchronize(st));
  if (words[3] == 0 && words[255] == 0) return BLR_OK;
  uint8_t* wp = static_cast<uint8_t*>(ws);
  BLR_CUDA_OK(cudaMemsetAsync(wp + 3 * sizeof(unsigned), 0, sizeof(unsigned), st));
  BLR_CUDA_OK(cudaMemsetAsync(wp + 255 * sizeof(unsigned), 0, sizeof(unsigned), st));
  set_last_error("a blr_blast_static call gave up on a device-side wait (status words %u, %u)", words[3], words[255]);
  return BLR_ERR_TIMEOUT;
}

int blr_blast_multi(const void* x, int64_t ldx, const void* x_mul, int act, int64_t n_tokens, int dtype, int n_problems,
                    const blr_blast_problem* problems, int64_t s_i, int64_t s_j, int64_t s_r, int bits, int group, int b, int P,
                    int Q, int R, void* ws, size_t ws_bytes, void* stream) {
  const int64_t N = n_tokens;
  BLR_REQUIRE(N >= 0, BLR_ERR_ARG, "token count must not be negative");
  if (N == 0) return BLR_OK;
  BLR_REQUIRE(x != nullptr && problems != nullptr, BLR_ERR_ARG, "x and problems must not be null");
  BLR_REQUIRE(dtype == BLR_DTYPE_F16 || dtype == BLR_DTYPE_BF16, BLR_ERR_ARG, "unknown dtype %d", dtype);
  BLR_REQUIRE(n_problems >= 1 && n_problems <= kSplitMaxProblems, BLR_ERR_UNSUPPORTED, "1..%d layers per call, got %d",
              kSplitMaxProblems, n_problems);
  BLR_REQUIRE(bits == 16 || bits == 8 || bits == 4, BLR_ERR_ARG, "bits must be 16, 8 or 4, got %d", bits);
  const int out_act = act >> 4;  // BLR_ACT_OUT_*: applied to result + bias, ahead of the residual
  act &= 15;
  BLR_REQUIRE(act == BLR_ACT_NONE || act == BLR_ACT_SILU_MUL, BLR_ERR_ARG, "unknown input transform %d", act);
  BLR_REQUIRE(out_act >= 0 && out_act <= 2, BLR_ERR_ARG, "unknown output activation %d", out_act);
  BLR_REQUIRE(out_act == 0 || n_tokens > kStreamMaxTokens, BLR_ERR_UNSUPPORTED, "output activations are fused above %d tokens only",
              kStreamMaxTokens);
  BLR_REQUIRE(act == BLR_ACT_NONE || x_mul != nullptr, BLR_ERR_ARG, "the silu-mul transform needs x_mul");
  BLR_REQUIRE(b >= 2 && P > 0 && Q > 0 && R > 0 && ldx >= (int64_t)b * P, BLR_ERR_SHAPE, "bad dimensions");
  SplitLayer layers[kSplitMaxProblems];
  for (int i = 0; i < n_problems; ++i) {
    const blr_blast_problem& q = problems[i];
    BLR_REQUIRE(q.U && q.V && q.S && q.out && q.ldo >= (int64_t)b * Q, BLR_ERR_ARG, "layer %d: null factor / output or short row", i);
    BLR_REQUIRE(bits == 16 || (q.u_scale && q.v_scale), BLR_ERR_ARG, "layer %d: quantised factors need scales", i);
    BLR_REQUIRE(q.residual == nullptr || q.ldr >= (int64_t)b * Q, BLR_ERR_SHAPE, "layer %d: residual rows shorter than the output", i);
    layers[i] = {q.U, bits == 16 ? nullptr : q.u_scale, q.V, bits == 16 ? nullptr : q.v_scale, q.S, q.bias, q.residual, q.out, q.ldo, q.ldr};
  }
  if (N > kStreamMaxTokens) {
    // prefill sizes: layer by layer through the tensor-core pipeline, bias and residual added by the last GEMM's epilogue
    BLR_REQUIRE(act == BLR_ACT_NONE, BLR_ERR_UNSUPPORTED, "the silu-mul input transform is fused for 1..%d tokens only", kStreamMaxTokens);
    for (int i = 0; i < n_problems; ++i) {
      const blr_blast_problem& q = problems[i];
      const int rc1 = blast_impl(x, ldx, N, dtype, q.U, BLR_W_KMAJOR, bits, bits == 16 ? nullptr : q.u_scale, q.V, BLR_W_KMAJOR, bits,
                                 bits == 16 ? nullptr : q.v_scale, group, q.S, s_i, s_j, s_r, b, b, P, Q, R, BLR_FLAG_NONE, q.out, q.ldo,
                                 ws, ws_bytes, static_cast<cudaStream_t>(stream), nullptr, q.bias, q.residual, q.ldr, out_act);
      if (rc1) return rc1;
    }
    return BLR_OK;
  }
  Workspace w;
  int rc = carve(ws, ws_bytes, N, (int64_t)n_problems * b, R, &w);
  if (rc) return rc;
  rc = split_blast_multi(x, ldx, x_mul, act == BLR_ACT_SILU_MUL ? kSplitActSiluMul : kSplitActNone, N, dtype, n_problems, layers,
                         BLR_W_KMAJOR, BLR_W_KMAJOR, bits, group, s_i, s_j, s_r, b, b, P, Q, R, 0, w.region_b, w.counters + 255,
                         static_cast<cudaStream_t>(stream), w.region_a,
                         (size_t)(static_cast<uint8_t*>(w.region_b) - static_cast<uint8_t*>(w.region_a)));
  BLR_REQUIRE(rc != 1, BLR_ERR_UNSUPPORTED,
              "the fused call serves 1..16 tokens, contraction-contiguous factors and shapes the two-launch path takes: run "
              "the layers one by one instead");
  return rc;
}

int blr_blast_wq(const void* x, int64_t ldx, int64_t n_tokens, int dtype, const void* Uq, const void* u_scale,
                 const void* Vq, const void* v_scale, const void* S, int64_t s_i, int64_t s_j, int64_t s_r, int bits,
                 int group, int b, int P, int Q, int R, void* out, int64_t ldo, void* ws, size_t ws_bytes, void* stream) {
  BLR_REQUIRE(bits == 8 || bits == 4, BLR_ERR_ARG, "bits must be 8 or 4, got %d", bits);
  BLR_REQUIRE(group == 0 || group == kScaleGroup, BLR_ERR_UNSUPPORTED,
              "scales per output channel (group = 0) or per %d contraction indices are implemented, got group = %d",
              kScaleGroup, group);
  BLR_REQUIRE(group == 0 || (P % kScaleGroup == 0 && R % kScaleGroup == 0), BLR_ERR_SHAPE,
              "with per-group scales P and R must be multiples of %d", kScaleGroup);
  BLR_REQUIRE(u_scale && v_scale, BLR_ERR_ARG, "scale pointers must not be null");
  return blast_impl(x, ldx, n_tokens, dtype, Uq, BLR_W_KMAJOR, bits, u_scale, Vq, BLR_W_KMAJOR, bits, v_scale, group, S, s_i,
                    s_j, s_r, b, b, P, Q, R, BLR_FLAG_NONE, out, ldo, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------- host-buffer entry points
// x and out live in host memory (pinned for truly asynchronous copies); the factors stay resident on the device.
// A call enqueues copy-in, the kernels and copy-out and returns.  The copies run on two streams the library owns
// per (device, caller stream), tied to the caller's stream with events, and the staging buffer is a ring of
// kHostSlots slots: the copy-in of call k+1 and the copy-out of call k-1 overlap the kernel of call k.
// out_host is valid once blr_host_flush has been enqueued on the caller's stream and that stream synchronised.
static constexpr int kHostSlots = 4;

struct HostPipe {
  cudaStream_t s_in = nullptr, s_out = nullptr;
  cudaEvent_t ev_in[kHostSlots] = {}, ev_k[kHostSlots] = {}, ev_out[kHostSlots] = {};
  bool used[kHostSlots] = {};
  unsigned next = 0;
};

static int host_pipe(cudaStream_t user, HostPipe** out) {
  static std::mutex mu;
  static std::unordered_map<unsigned long long, HostPipe*> pipes;
  int dev = 0;
  BLR_CUDA_OK(cudaGetDevice(&dev));
  const unsigned long long key = (unsigned long long)reinterpret_cast<uintptr_t>(user) * 64ull + (unsigned)dev;
  std::lock_guard<std::mutex> lk(mu);
  auto it = pipes.find(key);
  if (it == pipes.end()) {
    HostPipe* hp = new HostPipe();
    BLR_CUDA_OK(cudaStreamCreateWithFlags(&hp->s_in, cudaStreamNonBlocking));
    BLR_CUDA_OK(cudaStreamCreateWithFlags(&hp->s_out, cudaStreamNonBlocking));
    for (int i = 0; i < kHostSlots; ++i) {
      BLR_CUDA_OK(cudaEventCreateWithFlags(&hp->ev_in[i], cudaEventDisableTiming));
      BLR_CUDA_OK(cudaEventCreateWithFlags(&hp->ev_k[i], cudaEventDisableTiming));
      BLR_CUDA_OK(cudaEventCreateWithFlags(&hp->ev_out[i], cudaEventDisableTiming));
    }
    it = pipes.emplace(key, hp).first;
  }
  *out = it->second;
  return BLR_OK;
}

struct HostCall {
  HostPipe* hp;
  int slot;
  void *x_dev, *out_dev;
};

// Copy-in on the library's stream into the next ring slot, after the copy-out that last used the slot; the caller's
// stream then waits for the copy-in.
static int stage_in(const void* x_host, int64_t ldx, int64_t N, int64_t I, int64_t O, void* staging, size_t staging_bytes,
                    cudaStream_t user, HostCall* hc) {
  BLR_REQUIRE(x_host != nullptr && staging != nullptr, BLR_ERR_ARG, "x_host and staging must not be null");
  const size_t need = blr_host_staging_bytes(N, I, O);
  BLR_REQUIRE(staging_bytes >= need, BLR_ERR_WORKSPACE, "staging buffer of %zu bytes needed, got %zu", need, staging_bytes);
  BLR_REQUIRE((reinterpret_cast<uintptr_t>(staging) & 255) == 0, BLR_ERR_ALIGN, "staging buffer must be 256-byte aligned");
  BLR_REQUIRE(ldx >= I, BLR_ERR_SHAPE, "leading dimension shorter than a row");
  int rc = host_pipe(user, &hc->hp);
  if (rc) return rc;
  HostPipe* hp = hc->hp;
  const int slot = hc->slot = (int)(hp->next++ % kHostSlots);
  // slots are cut from the buffer's own size, so calls of different sizes on one buffer agree on where they are
  const size_t per = staging_bytes / kHostSlots / 256 * 256;
  hc->x_dev = static_cast<uint8_t*>(staging) + per * slot;
  hc->out_dev = static_cast<uint8_t*>(hc->x_dev) + align256((size_t)N * I * 2);
  // the copy-out that last used the slot is done, and with it the kernel that read the slot's x (the copy-out waited
  // for that kernel); the caller's stream inherits both through ev_in and so carries one wait per call
  if (hp->used[slot]) BLR_CUDA_OK(cudaStreamWaitEvent(hp->s_in, hp->ev_out[slot], 0));
  if (ldx == I) BLR_CUDA_OK(cudaMemcpyAsync(hc->x_dev, x_host, (size_t)N * I * 2, cudaMemcpyHostToDevice, hp->s_in));
  else BLR_CUDA_OK(cudaMemcpy2DAsync(hc->x_dev, (size_t)I * 2, x_host, (size_t)ldx * 2, (size_t)I * 2, (size_t)N,
                                     cudaMemcpyHostToDevice, hp->s_in));
  BLR_CUDA_OK(cudaEventRecord(hp->ev_in[slot], hp->s_in));
  BLR_CUDA_OK(cudaStreamWaitEvent(user, hp->ev_in[slot], 0));
  return BLR_OK;
}
static int stage_out(void* out_host, int64_t ldo, int64_t N, int64_t O, cudaStream_t user, HostCall* hc) {
  HostPipe* hp = hc->hp;
  const int slot = hc->slot;
  BLR_CUDA_OK(cudaEventRecord(hp->ev_k[slot], user));
  BLR_CUDA_OK(cudaStreamWaitEvent(hp->s_out, hp->ev_k[slot], 0));
  if (ldo == O) BLR_CUDA_OK(cudaMemcpyAsync(out_host, hc->out_dev, (size_t)N * O * 2, cudaMemcpyDeviceToHost, hp->s_out));
  else BLR_CUDA_OK(cudaMemcpy2DAsync(out_host, (size_t)ldo * 2, hc->out_dev, (size_t)O * 2, (size_t)O * 2, (size_t)N,
                                     cudaMemcpyDeviceToHost, hp->s_out));
  BLR_CUDA_OK(cudaEventRecord(hp->ev_out[slot], hp->s_out));
  hp->used[slot] = true;
  return BLR_OK;
}

size_t blr_host_staging_bytes(int64_t n_tokens, int64_t in_features, int64_t out_features) {
  if (n_tokens < 0 || in_features < 0 || out_features < 0) return 0;
  return kHostSlots * (align256((size_t)n_tokens * in_features * 2) + align256((size_t)n_tokens * out_features * 2));
}

int blr_host_flush(void* stream) {
  cudaStream_t user = static_cast<cudaStream_t>(stream);
  HostPipe* hp;
  int rc = host_pipe(user, &hp);
  if (rc) return rc;
  for (int i = 0; i < kHostSlots; ++i)
    if (hp->used[i]) BLR_CUDA_OK(cudaStreamWaitEvent(user, hp->ev_out[i], 0));
  return BLR_OK;
}

int blr_blast_host(const void* x_host, int64_t ldx, int64_t n_tokens, int dtype, const void* U, int u_layout, const void* V,
                   int v_layout, const void* S, int64_t s_i, int64_t s_j, int64_t s_r, int b, int P, int Q, int R, int flags,
                   void* out_host, int64_t ldo, void* staging, size_t staging_bytes, void* ws, size_t ws_bytes, void* stream) {
  if (n_tokens == 0) return BLR_OK;
  BLR_REQUIRE(out_host != nullptr && b >= 1 && P > 0 && Q > 0 && ldo >= (int64_t)b * Q, BLR_ERR_ARG, "bad output arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  HostCall hc;
  int rc = stage_in(x_host, ldx, n_tokens, (int64_t)b * P, (int64_t)b * Q, staging, staging_bytes, st, &hc);
  if (rc) return rc;
  rc = blast_impl(hc.x_dev, (int64_t)b * P, n_tokens, dtype, U, u_layout, 16, nullptr, V, v_layout, 16, nullptr, 0, S, s_i, s_j,
                  s_r, b, b, P, Q, R, flags, hc.out_dev, (int64_t)b * Q, ws, ws_bytes, st);
  if (rc) return rc;
  return stage_out(out_host, ldo, n_tokens, (int64_t)b * Q, st, &hc);
}

int blr_blast_wq_host(const void* x_host, int64_t ldx, int64_t n_tokens, int dtype, const void* Uq, const void* u_scale,
                      const void* Vq, const void* v_scale, const void* S, int64_t s_i, int64_t s_j, int64_t s_r, int bits,
                      int group, int b, int P, int Q, int R, void* out_host, int64_t ldo, void* staging, size_t staging_bytes,
                      void* ws, size_t ws_bytes, void* stream) {
  if (n_tokens == 0) return BLR_OK;
  BLR_REQUIRE(out_host != nullptr && b >= 1 && P > 0 && Q > 0 && ldo >= (int64_t)b * Q, BLR_ERR_ARG, "bad output arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  HostCall hc;
  int rc = stage_in(x_host, ldx, n_tokens, (int64_t)b * P, (int64_t)b * Q, staging, staging_bytes, st, &hc);
  if (rc) return rc;
  t_host_call = true;
  rc = blr_blast_wq(hc.x_dev, (int64_t)b * P, n_tokens, dtype, Uq, u_scale, Vq, v_scale, S, s_i, s_j, s_r, bits, group, b, P, Q, R,
                    hc.out_dev, (int64_t)b * Q, ws, ws_bytes, stream);
  t_host_call = false;
  if (rc) return rc;
  return stage_out(out_host, ldo, n_tokens, (int64_t)b * Q, st, &hc);
}

int blr_monarch(const void* x, int64_t ldx, int64_t n_tokens, int dtype, const void* w1, int w1_layout, int w1_cols,
                const void* w2, int w2_layout, int b, int P, int rank, int Qs, int out_order, void* out, int64_t ldo,
                void* ws, size_t ws_bytes, void* stream) {
  const int64_t N = n_tokens;
  int rc = check_common(x, ldx, N, dtype, out, ldo);
  if (rc) return rc < 0 ? rc : BLR_OK;
  BLR_REQUIRE(w1 && w2, BLR_ERR_ARG, "factor pointers must not be null");
  BLR_REQUIRE(b >= 1 && P > 0 && rank > 0 && Qs > 0, BLR_ERR_SHAPE, "b, P, rank, Qs must be positive");
  BLR_REQUIRE(rank % b == 0, BLR_ERR_SHAPE, "rank %d must be a multiple of the block count %d (wrappers.py:14)", rank, b);
  BLR_REQUIRE(w1_cols == BLR_MONARCH_COLS_TORCH || w1_cols == BLR_MONARCH_COLS_GROUPED, BLR_ERR_ARG, "unknown w1_cols %d", w1_cols);
  BLR_REQUIRE(out_order == BLR_OUT_INTERLEAVED || out_order == BLR_OUT_BLOCKED, BLR_ERR_ARG, "unknown out_order %d", out_order);
  BLR_REQUIRE(ldx >= (int64_t)b * P && ldo >= (int64_t)b * Qs, BLR_ERR_SHAPE, "leading dimensions shorter than a row");
  if ((rc = check_layout(w1_layout)) || (rc = check_layout(w2_layout))) return rc;
  Workspace w;
  if ((rc = carve(ws, ws_bytes, N, b, rank, &w))) return rc;
  const int per = rank / b;
  // intermediate Z[l][n][k*per + jj] lives in region_b (16-bit)
  const long long zplane = (long long)N * rank;
  const int grouped = w1_cols == BLR_MONARCH_COLS_GROUPED;
  if (N <= kStreamMaxTokens) {
    if (w1_layout == BLR_W_KMAJOR && w2_layout == BLR_W_KMAJOR) {
      // the two-launch path of BLAST: the first factor's blocks as V, the second's as U, the permutation in the hand-over
      SplitLayer l = {w2, nullptr, w1, nullptr, nullptr, nullptr, nullptr, out, ldo, 0};
      l.monarch = 1;
      l.mon_torch = grouped ? 0 : 1;
      l.out_interleaved = out_order == BLR_OUT_INTERLEAVED ? 1 : 0;
      rc = split_blast_multi(x, ldx, nullptr, kSplitActNone, N, dtype, 1, &l, BLR_W_KMAJOR, BLR_W_KMAJOR, 16, 0, 0, 0, 0, b, b, P, Qs,
                             rank, 0, w.region_b, w.counters + 255, static_cast<cudaStream_t>(stream), nullptr, 0,
                             /*may_decline=*/true);
      if (rc <= 0) return rc;
    }
    rc = cluster_monarch(x, ldx, N, dtype, w1, w1_layout, grouped, w2, w2_layout, b, P, rank, Qs, out_order == BLR_OUT_INTERLEAVED,
                         out, ldo, w, static_cast<cudaStream_t>(stream));
    if (rc <= 0) return rc;  // 1: not applicable -> grid-wide streaming kernel
    StreamParams p = {};
    p.nphases = 2; p.mix = 0; p.counters = w.counters;
    if ((rc = phase_weights(p.ph[0], dtype, w1, w1_layout, 16, b, rank, P))) return rc;
    if ((rc = phase_acts(p.ph[0], dtype, x, P, N, b, ldx, P))) return rc;
    if (grouped) phase_out(p.ph[0], w.region_b, 0, per, rank, per, zplane, 1, nullptr, 0);
    else phase_out(p.ph[0], w.region_b, 0, per, rank, b, 1, zplane, nullptr, 0);
    if ((rc = phase_weights(p.ph[1], dtype, w2, w2_layout, 16, b, Qs, rank))) return rc;
    if ((rc = phase_acts(p.ph[1], dtype, w.region_b, rank, N, b, rank, zplane))) return rc;
    if (out_order == BLR_OUT_INTERLEAVED) phase_out(p.ph[1], out, 0, 1, ldo, Qs, 0, b, nullptr, 0);
    else phase_out(p.ph[1], out, 0, Qs, ldo, Qs, 0, 1, nullptr, 0);
    finish_params(p, N);
    return launch_stream(p, dtype == BLR_DTYPE_BF16, static_cast<cudaStream_t>(stream));
  }
  const int64_t per_pass = pass_size(N, b, rank);
  for (int64_t n0 = 0; n0 < N; n0 += per_pass) {
    const int64_t n = N - n0 < per_pass ? N - n0 : per_pass;
    rc = pipeline_monarch(static_cast<const uint8_t*>(x) + n0 * ldx * 2, ldx, n, dtype, w1, w1_layout, grouped, w2, w2_layout, b, P,
                          rank, Qs, out_order == BLR_OUT_INTERLEAVED, static_cast<uint8_t*>(out) + n0 * ldo * 2, ldo, w.region_b,
                          w.region_a, static_cast<cudaStream_t>(stream));
    if (rc) return rc;
  }
  return BLR_OK;
}

int blr_low_rank(const void* x, int64_t ldx, int64_t n_tokens, int dtype, const void* V, int v_layout, const void* U,
                 int u_layout, int I, int R, int O, void* out, int64_t ldo, void* ws, size_t ws_bytes, void* stream) {
  const int64_t N = n_tokens;
  int rc = check_common(x, ldx, N, dtype, out, ldo);
  if (rc) return rc < 0 ? rc : BLR_OK;
  BLR_REQUIRE(V && U, BLR_ERR_ARG, "factor pointers must not be null");
  BLR_REQUIRE(I > 0 && R > 0 && O > 0, BLR_ERR_SHAPE, "I, R, O must be positive");
  BLR_REQUIRE(ldx >= I && ldo >= O, BLR_ERR_SHAPE, "leading dimensions shorter than a row");
  if ((rc = check_layout(v_layout)) || (rc = check_layout(u_layout))) return rc;
  Workspace w;
  if ((rc = carve(ws, ws_bytes, N, 1, R, &w))) return rc;
  if (N <= kStreamMaxTokens) {
    // Low rank is BLAST with an all-ones coupling: cut the I columns of V into b blocks (y_j = V[:, block j] x_j,
    // z = sum_j y_j) and the O rows of U into b blocks (out_i = U[block i] z).  That puts it on the cluster kernel,
    // which splits the long contraction of the first stage over b CTAs instead of leaving it to R / 16 of them.
    for (int bb = 16; bb >= 2; bb >>= 1) {
      if (I % (bb * 8) != 0 || O % (bb * 8) != 0) continue;
      const int Pb = I / bb, Qb = O / bb;
      const bool vk = v_layout == BLR_W_KMAJOR, uk = u_layout == BLR_W_KMAJOR;
      if (vk && uk && (int64_t)Pb * 2 % 16 == 0) {
        // the two-launch path: z is the same for every out-block and is kept once (the workspace holds N x R values)
        SplitLayer l = {U, nullptr, V, nullptr, nullptr, nullptr, nullptr, out, ldo, 0};
        l.v_row = I;
        l.v_blk = Pb;
        rc = split_blast_multi(x, ldx, nullptr, kSplitActNone, N, dtype, 1, &l, BLR_W_KMAJOR, BLR_W_KMAJOR, 16, 0, 0, 0, 0, bb, bb,
                               Pb, Qb, R, 0, w.region_b, w.counters + 255, static_cast<cudaStream_t>(stream), nullptr, 0,
                               /*may_decline=*/true);
        if (rc <= 0) return rc;
      }
      rc = cluster_blast(x, ldx, N, dtype, U, u_layout, 16, nullptr, V, v_layout, 16, nullptr, 0, nullptr, 0, 0, 0, bb, bb, Pb,
                         Qb, R, 0, out, ldo, w, static_cast<cudaStream_t>(stream), vk ? I : 0, vk ? Pb : 0, uk ? 0 : O,
                         uk ? 0 : Qb);
      if (rc <= 0) return rc;
      break;  // not applicable: the grid-wide kernel below
    }
    StreamParams p = {};
    p.nphases = 2; p.mix = 0; p.counters = w.counters;
    if ((rc = phase_weights(p.ph[0], dtype, V, v_layout, 16, 1, R, I))) return rc;
    if ((rc = phase_acts(p.ph[0], dtype, x, I, N, 1, ldx, 0))) return rc;
    phase_out(p.ph[0], w.region_b, 0, 0, R, R, 0, 1, nullptr, 0);
    if ((rc = phase_weights(p.ph[1], dtype, U, u_layout, 16, 1, O, R))) return rc;
    if ((rc = phase_acts(p.ph[1], dtype, w.region_b, R, N, 1, R, 0))) return rc;
    phase_out(p.ph[1], out, 0, 0, ldo, O, 0, 1, nullptr, 0);
    finish_params(p, N);
    return launch_stream(p, dtype == BLR_DTYPE_BF16, static_cast<cudaStream_t>(stream));
  }
  const int64_t per_pass = pass_size(N, 1, R);
  for (int64_t n0 = 0; n0 < N; n0 += per_pass) {
    const int64_t n = N - n0 < per_pass ? N - n0 : per_pass;
    rc = pipeline_low_rank(static_cast<const uint8_t*>(x) + n0 * ldx * 2, ldx, n, dtype, V, v_layout, U, u_layout, I, R, O,
                           static_cast<uint8_t*>(out) + n0 * ldo * 2, ldo, w.region_b, w.region_c, region_c_bytes(N, 1, R),
                           static_cast<cudaStream_t>(stream));
    if (rc) return rc;
  }
  return BLR_OK;
}

int blr_dense(const void* x, int64_t ldx, int64_t n_tokens, int dtype, const void* W, int w_layout, int I, int O,
              void* out, int64_t ldo, void* stream) {
  const int64_t N = n_tokens;
  int rc = check_common(x, ldx, N, dtype, out, ldo);
  if (rc) return rc < 0 ? rc : BLR_OK;
  BLR_REQUIRE(W, BLR_ERR_ARG, "weight pointer must not be null");
  BLR_REQUIRE(I > 0 && O > 0, BLR_ERR_SHAPE, "I, O must be positive");
  BLR_REQUIRE(ldx >= I && ldo >= O, BLR_ERR_SHAPE, "leading dimensions shorter than a row");
  if ((rc = check_layout(w_layout))) return rc;
  if (N <= kStreamMaxTokens) {
    StreamParams p = {};
    p.nphases = 1; p.mix = 0; p.counters = nullptr;
    if ((rc = phase_weights(p.ph[0], dtype, W, w_layout, 16, 1, O, I))) return rc;
    if ((rc = phase_acts(p.ph[0], dtype, x, I, N, 1, ldx, 0))) return rc;
    phase_out(p.ph[0], out, 0, 0, ldo, O, 0, 1, nullptr, 0);
    finish_params(p, N);
    return launch_stream(p, dtype == BLR_DTYPE_BF16, static_cast<cudaStream_t>(stream));
  }
  return pipeline_dense(x, ldx, N, dtype, W, w_layout, I, O, out, ldo, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
