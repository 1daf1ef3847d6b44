/* blr_b200.h -- C ABI of the B200 (sm_100a) structured-matmul library.
 *
 * The reference project (pabillam/mem-efficient-blr) has no native interface: its operator API is a
 * set of Python free functions, picked by dotted name from YAML (layer.py:30-38,
 * models/wrappers.py:143-146).  Each entry point below is what a binding for one family of those
 * functions calls; the comment above it names the reference functions it stands in for.
 *
 * Conventions
 *   - All pointers are device pointers unless stated otherwise.  Nothing here allocates device memory;
 *     scratch comes from the caller (`ws`, sized by blr_workspace_bytes).
 *   - `stream` is a cudaStream_t passed as void*.  Calls enqueue work and return; they never
 *     synchronise the host.  Calls that share a workspace must be ordered on one stream.
 *   - `dtype` selects the 16-bit type of x, the 16-bit factors and out.
 *   - x is (N, in_features) with row stride `ldx` elements; out is (N, out_features) with row stride
 *     `ldo` elements.  Input feature j*P+p belongs to input block j; output feature i*Q+q to block i.
 *   - Weight layouts: BLR_W_KMAJOR = [block][out_row][k] (contraction index contiguous, the
 *     reference's torch layouts); BLR_W_MMAJOR = [block][k][out_row] (output index contiguous, the
 *     layouts of the reference's Triton entry points).
 *   - n_tokens = 0 is valid for the 16-bit and quantised entry points: they return 0 without touching a pointer.
 *   - Return value: 0 on success, a negative BLR_ERR_* code otherwise; blr_last_error() has the text.
 *     Token counts up to 16 run weight-streaming kernels (contraction-contiguous factors: a pair of dependent
 *     launches; other layouts: a kernel of thread-block clusters or a grid-wide one); larger counts run the
 *     tensor-core pipeline.
 */
#ifndef BLR_B200_H_
#define BLR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BLR_DTYPE_F16 0
#define BLR_DTYPE_BF16 1

#define BLR_W_KMAJOR 0
#define BLR_W_MMAJOR 1

/* Column order of Monarch's first factor. TORCH: column c of block k feeds out1[c % b][k*per + c / b]
 * (torch_funcs/monarch_funcs.py:41).  GROUPED: column l*per + jj feeds out1[l][k*per + jj]
 * (the regrouping the reference's harness applies for its kernels, layer.py:221-224). */
#define BLR_MONARCH_COLS_TORCH 0
#define BLR_MONARCH_COLS_GROUPED 1

/* Output feature order of Monarch. INTERLEAVED: s*b + l (monarch_funcs.py:44);
 * BLOCKED: l*S + s (triton_monarch_right_ideal, monarch_kernels.py:1004). */
#define BLR_OUT_INTERLEAVED 0
#define BLR_OUT_BLOCKED 1

#define BLR_FLAG_NONE 0
/* Round both BLAST intermediates to the nearest integer in [-128, 127], no scale: the semantics of
 * triton_blast_bmm_int8_fp16 (blast_sym_quant_kernels.py:105-108, 227-230). */
#define BLR_FLAG_ACT_INT8 1

#define BLR_OK 0
#define BLR_ERR_ARG (-1)
#define BLR_ERR_SHAPE (-2)
#define BLR_ERR_ALIGN (-3)
#define BLR_ERR_WORKSPACE (-4)
#define BLR_ERR_CUDA (-5)
#define BLR_ERR_UNSUPPORTED (-6)
#define BLR_ERR_TIMEOUT (-7)

/* Library version (major*10000 + minor*100 + patch). No reference counterpart. */
int blr_version(void);

/* Test aid: which kernel serves 1..16 tokens.  0: automatic (BLAST, low-rank and Monarch with contraction-contiguous
 * factors: the two-launch path; other layouts, and Monarch on up to 8 tokens: the cluster kernel; the rest: the
 * grid-wide streaming kernel).  1: the grid-wide streaming kernel for everything.  2: automatic without the
 * two-launch path.
 * Process-wide (an atomic). No reference counterpart. */
int blr_debug_decode_path(int which);

/* Text of the last error on the calling thread. No reference counterpart (the reference raises
 * Python AssertionError, e.g. blast_kernels.py:1951-1955). */
const char* blr_last_error(void);

/* Bytes of scratch a call needs: `groups` blocks, `width` intermediate features per block, N tokens
 * (BLAST: b, R; Monarch: b, rank; low-rank: 1, R; dense: 0, 0).  The size stops growing with N once the 16-bit
 * intermediates of a call would outgrow the L2 cache (128 MB per intermediate): such a call runs as consecutive passes
 * over equal parts of the tokens on the same scratch.  No reference counterpart: the
 * reference allocates its intermediates with torch.empty per call (blast_kernels.py:1967, 2703). */
size_t blr_workspace_bytes(int64_t n_tokens, int64_t groups, int64_t width);

/* Device memory for a workspace or staging buffer straight from cudaMalloc / back to cudaFree, for host layers whose
 * own allocator is not a safe home for a long-lived scratch buffer (PyTorch routes allocations made while it records a
 * CUDA graph, or warms one up, into that graph's private pool).  Not to be called while a stream capture is under
 * way.  Returns NULL on failure (blr_last_error has the text).  No reference counterpart. */
void* blr_scratch_alloc(size_t bytes);
int blr_scratch_free(void* ptr);

/* Zeroes the fixed head of a workspace: 1 KiB of control words and the 2 MiB fp32 accumulation area of the
 * cluster kernel (the kernels leave both zero again when they finish).  Required once after allocation and
 * after a call reported BLR_ERR_TIMEOUT through blr_workspace_status. No reference counterpart. */
int blr_workspace_init(void* ws, size_t ws_bytes, void* stream);

/* Reads the status word of a workspace (synchronises `stream`): 0, or BLR_ERR_TIMEOUT if a kernel
 * gave up on a device-side wait. No reference counterpart. */
int blr_workspace_status(const void* ws, void* stream);

/* BLAST: y_j = x_j V_j^T ; z_i = sum_j S_ij (.) y_j ; out_i = z_i U_i^T.
 * Replaces torch_blast_baseline / torch_blast_bmm (torch_funcs/blast_funcs.py:3-47, 49-91) and
 * triton_blast_{partial,partial_grouped,partial_grouped_persistent,full,bmm}_fp16
 * (triton_funcs/blast_kernels.py:2666-2707, 2762-2803, 2858-2899, 2955-2995, 3043-3065), and with
 * BLR_FLAG_ACT_INT8 triton_blast_bmm_int8_fp16 (blast_sym_quant_kernels.py:558-580).
 * U: b blocks of Q rows x R; V: b blocks of R rows x P; S element (i, j, r) at i*s_i + j*s_j + r*s_r. */
int blr_blast(const void* x, int64_t ldx, int64_t n_tokens, int dtype,
              const void* U, int u_layout, const void* V, int v_layout,
              const void* S, int64_t s_i, int64_t s_j, int64_t s_r,
              int b, int P, int Q, int R, int flags,
              void* out, int64_t ldo, void* ws, size_t ws_bytes, void* stream);

/* blr_blast on a slice of the output blocks, for sharding a layer over GPUs by output block (no reference
 * counterpart; the reference runs on one GPU): U holds b_out <= b blocks, S element (i, j, r) exists for
 * i < b_out, out is (N, b_out*Q).  The first stage still covers all b input blocks.  The slices of several
 * ranks are joined with an all-gather along the feature axis by the caller. */
int blr_blast_rows(const void* x, int64_t ldx, int64_t n_tokens, int dtype,
                   const void* U, int u_layout, const void* V, int v_layout,
                   const void* S, int64_t s_i, int64_t s_j, int64_t s_r,
                   int b, int b_out, int P, int Q, int R, int flags,
                   void* out, int64_t ldo, void* ws, size_t ws_bytes, void* stream);

/* Above 256 tokens the coupling runs on the tensor cores as a product with expanded coupling factors E (a function of
 * S alone, blr_blast_coupling_bytes bytes; 0 for shapes whose coupling takes another route), which blr_blast rebuilds
 * in its workspace at every call.  A caller whose S does not change between calls builds E once
 * (blr_blast_expand_coupling; E 256-byte aligned) and passes it to blr_blast_rows_prepared, which is blr_blast_rows
 * otherwise (E = NULL: exactly blr_blast_rows; E is ignored at token counts that do not use it).  No reference
 * counterpart (the reference's kernels read S directly, blast_kernels.py:1990-2050). */
size_t blr_blast_coupling_bytes(int b, int b_out, int R);
int blr_blast_expand_coupling(const void* S, int64_t s_i, int64_t s_j, int64_t s_r, int b, int b_out, int R, int dtype,
                              void* E, size_t E_bytes, void* stream);
int blr_blast_rows_prepared(const void* x, int64_t ldx, int64_t n_tokens, int dtype,
                            const void* U, int u_layout, const void* V, int v_layout,
                            const void* S, int64_t s_i, int64_t s_j, int64_t s_r,
                            int b, int b_out, int P, int Q, int R, int flags,
                            void* out, int64_t ldo, void* ws, size_t ws_bytes, void* stream, const void* E);

/* Several BLAST layers that share their input and shapes in one pair of launches, with the element-wise work around
 * them folded in (no counterpart in the reference, whose modules call one operator per layer and add the bias and
 * the activation with separate torch kernels, models/wrappers.py:171-177):
 *   - q / k / v projections of an attention block, or gate / up projections of an MLP: n_problems layers, one x;
 *   - `bias` (b*Q values) and `residual` ((N, b*Q), row stride ldr) are added to a layer's result before it is stored;
 *   - act = BLR_ACT_SILU_MUL: the input is silu(x) * x_mul (x_mul like x, same row stride): a down projection that
 *     takes the gate and up results directly.
 * Factors are contraction-contiguous: U (b,Q,R), V (b,R,P) in the 16-bit dtype (bits = 16: scales ignored) or quantised
 * as for blr_blast_wq (bits = 8 | 4).  S element (i, j, r) of every layer at i*s_i + j*s_j + r*s_r.
 * Scratch: the larger of blr_workspace_bytes(n_tokens, n_problems * b, R) and blr_workspace_bytes(n_tokens, b, R).
 * 1..16 tokens: the two-launch decode path (BLR_ERR_UNSUPPORTED for shapes it does not take - run the layers one by
 * one).  More tokens: the layers run one after the other through the tensor-core pipeline and the last GEMM's
 * epilogue adds bias and residual; BLR_ACT_SILU_MUL is not available there (BLR_ERR_UNSUPPORTED). */
#define BLR_ACT_NONE 0
#define BLR_ACT_SILU_MUL 1
/* Output activations of the fused call above 16 tokens, OR-ed into `act`: applied to result + bias, ahead of the residual
 * (the GELU between the two linears of an encoder / denoiser MLP: models/vit_b_patch16_224.py, DiT/models.py:111-112). */
#define BLR_ACT_OUT_GELU 0x10
#define BLR_ACT_OUT_GELU_TANH 0x20
typedef struct blr_blast_problem {
  const void* U;
  const void* V;
  const void* S;
  const void* u_scale; /* NULL with 16-bit factors */
  const void* v_scale;
  const void* bias;     /* NULL or b*Q values of the 16-bit dtype */
  const void* residual; /* NULL or (N, b*Q) of the 16-bit dtype */
  int64_t ldr;
  void* out;
  int64_t ldo;
} blr_blast_problem;
int blr_blast_multi(const void* x, int64_t ldx, const void* x_mul, int act, int64_t n_tokens, int dtype,
                    int n_problems, const blr_blast_problem* problems,
                    int64_t s_i, int64_t s_j, int64_t s_r, int bits, int group, int b, int P, int Q, int R,
                    void* ws, size_t ws_bytes, void* stream);

/* blr_blast for callers that cannot allocate device memory and have no workspace to pass: plug-ins running
 * inside a host application that owns the device allocator, or latency-critical threads where the implicit
 * synchronisation of cudaMalloc is not acceptable.  This entry point has
 * no counterpart in the reference.  Same arguments and results as blr_blast, minus (ws, ws_bytes); 1..16 tokens
 * only.  Its scratch is a 4 MiB array built into the library's device image, which every GPU that loads the
 * library holds until exit; calls with blr_workspace_bytes(n_tokens, b, R) > 4 MiB (b * n_tokens * R above about 349 000)
 * are rejected with BLR_ERR_WORKSPACE.  The first call on each device looks the array up with
 * cudaGetSymbolAddress (that device must be current) - make that first call before any stream capture.  It calls
 * no cudaMalloc / cudaFree or other allocating routine.  All calls on a device share the one array: it keeps the
 * previous call's contents (the control words and the accumulation area the shape can touch are cleared on the
 * stream at the start of every call), and two
 * calls that overlap on the GPU (different streams) race on it. */
int blr_blast_static(const void* x, int64_t ldx, int64_t n_tokens, int dtype,
                     const void* U, int u_layout, const void* V, int v_layout,
                     const void* S, int64_t s_i, int64_t s_j, int64_t s_r,
                     int b, int P, int Q, int R, int flags,
                     void* out, int64_t ldo, void* stream);
/* Status of the built-in scratch array on the current device (synchronises `stream`, allocates nothing): 0, or
 * BLR_ERR_TIMEOUT if a blr_blast_static call since the last query gave up on a device-side wait, in which case that
 * call's output is not valid.  A time-out stays recorded across later calls until this function has reported it
 * once.  No reference counterpart. */
int blr_blast_static_status(void* stream);

/* BLAST with int8 / packed-int4 factors and fp16 scales.  No reference counterpart (the reference's
 * sym-quant kernels round activations, not weights); the format is: Uq int8 (b,Q,R) or uint8 (b,Q,R/2),
 * Vq int8 (b,R,P) or uint8 (b,R,P/2), contraction index contiguous, two int4 per byte with the even
 * index in the low nibble; weight = q * scale.  `group` = 0: one scale per output channel, u_scale fp16 (b,Q),
 * v_scale fp16 (b,R).  `group` = 128: one scale per 128 consecutive contraction indices, u_scale fp16
 * (b,Q,R/128), v_scale fp16 (b,R,P/128); P and R must then be multiples of 128.  Other widths are rejected
 * with BLR_ERR_UNSUPPORTED.  Any token count; the quantised arrays are the only copy of the factors in device
 * memory: up to 16 tokens the stored bytes are the MMA operands, above that the tensor-core GEMMs stage the stored
 * bytes and widen them (q * scale rounded once to the 16-bit dtype) in shared memory ahead of the MMA.  Above 16
 * tokens a row of P or R weights must be a multiple of 16 bytes (BLR_ERR_UNSUPPORTED otherwise: widen with
 * blr_dequantize_sym and call blr_blast, as the Python layer does). */
int blr_blast_wq(const void* x, int64_t ldx, int64_t n_tokens, int dtype,
                 const void* Uq, const void* u_scale, const void* Vq, const void* v_scale,
                 const void* S, int64_t s_i, int64_t s_j, int64_t s_r,
                 int bits, int group, int b, int P, int Q, int R,
                 void* out, int64_t ldo, void* ws, size_t ws_bytes, void* stream);

/* Host-buffer forms of blr_blast and blr_blast_wq: x_host (N, ldx) and out_host (N, ldo) are host memory (pinned
 * memory makes the copies asynchronous), the factors are device memory.  The call enqueues the copy of x, the
 * kernels and the copy of the result and returns.  The copies run on two streams the library keeps per (device,
 * `stream`), ordered against `stream` with events, and `staging` is used as a ring of four slots, so that
 * consecutive calls overlap: copy-in of the next call and copy-out of the previous one run beside the kernel.
 * out_host is valid after blr_host_flush(stream) has been called and `stream` has been synchronised.
 * `staging` is caller-owned device memory of blr_host_staging_bytes(n_tokens, b*P, b*Q) bytes, 256-byte aligned,
 * used with one stream like the workspace and, from its first use on, always passed with the same size (the
 * slots are cut from that size); size it for the largest call.  Not for use while `stream` is being captured into a
 * CUDA graph: the copy streams are not part of the capture.  No reference counterpart (the reference's operators take device tensors). */
size_t blr_host_staging_bytes(int64_t n_tokens, int64_t in_features, int64_t out_features);
/* Makes `stream` wait for every copy-out that host-buffer calls on it have enqueued so far. */
int blr_host_flush(void* stream);
int blr_blast_host(const void* x_host, int64_t ldx, int64_t n_tokens, int dtype,
                   const void* U, int u_layout, const void* V, int v_layout,
                   const void* S, int64_t s_i, int64_t s_j, int64_t s_r,
                   int b, int P, int Q, int R, int flags,
                   void* out_host, int64_t ldo, void* staging, size_t staging_bytes,
                   void* ws, size_t ws_bytes, void* stream);
int blr_blast_wq_host(const void* x_host, int64_t ldx, int64_t n_tokens, int dtype,
                      const void* Uq, const void* u_scale, const void* Vq, const void* v_scale,
                      const void* S, int64_t s_i, int64_t s_j, int64_t s_r,
                      int bits, int group, int b, int P, int Q, int R,
                      void* out_host, int64_t ldo, void* staging, size_t staging_bytes,
                      void* ws, size_t ws_bytes, void* stream);

/* Monarch: block-diagonal w1, permutation, block-diagonal w2.
 * Replaces torch_monarch_baseline (torch_funcs/monarch_funcs.py:4-45) and
 * triton_monarch_{right,right_ideal,right_left}_fp16 (triton_funcs/monarch_kernels.py:869-909,
 * 961-1005, 1060-1099).  w1: b blocks, `rank` outputs each over P inputs; w2: b blocks, Qs outputs
 * each over `rank` inputs. */
int blr_monarch(const void* x, int64_t ldx, int64_t n_tokens, int dtype,
                const void* w1, int w1_layout, int w1_cols, const void* w2, int w2_layout,
                int b, int P, int rank, int Qs, int out_order,
                void* out, int64_t ldo, void* ws, size_t ws_bytes, void* stream);

/* Low rank: out = (x V^T) U^T.  Replaces torch_low_rank_baseline (torch_funcs/low_rank_funcs.py:4-28)
 * and triton_low_rank_fp16 (triton_funcs/low_rank_kernels.py:410-417).  V: R x I, U: O x R. */
int blr_low_rank(const void* x, int64_t ldx, int64_t n_tokens, int dtype,
                 const void* V, int v_layout, const void* U, int u_layout,
                 int I, int R, int O,
                 void* out, int64_t ldo, void* ws, size_t ws_bytes, void* stream);

/* Dense: out = x W^T.  Replaces torch_dense_baseline (torch_funcs/dense_funcs.py:4-25) and
 * triton_dense_fp16 (triton_funcs/dense_kernels.py:375-381).  W: O x I. */
int blr_dense(const void* x, int64_t ldx, int64_t n_tokens, int dtype,
              const void* W, int w_layout, int I, int O,
              void* out, int64_t ldo, void* stream);

/* fp32 verification variants: exact fp32 FMA arithmetic, intermediates returned.
 * Replace triton_blast_*_fp32 (blast_kernels.py:2614-2664 ... 2998-3041; out, z (b,N,R), y (b,N,R)),
 * triton_monarch_*_fp32 (monarch_kernels.py:823-867, 911-959, 1007-1058; out, out1 (b,N,rank)),
 * triton_low_rank_fp32 (low_rank_kernels.py:394-408; out, z (N,R)) and
 * triton_dense_fp32 (dense_kernels.py:360-373).  All tensors fp32 and dense row-major; the
 * intermediates y, z, out1 are caller-provided outputs and must not be NULL. */
int blr_blast_f32(const float* x, int64_t ldx, int64_t n_tokens,
                  const float* U, int u_layout, const float* V, int v_layout,
                  const float* S, int64_t s_i, int64_t s_j, int64_t s_r,
                  int b, int P, int Q, int R,
                  float* out, int64_t ldo, float* z, float* y, void* stream);
int blr_monarch_f32(const float* x, int64_t ldx, int64_t n_tokens,
                    const float* w1, int w1_layout, int w1_cols, const float* w2, int w2_layout,
                    int b, int P, int rank, int Qs, int out_order,
                    float* out, int64_t ldo, float* out1, void* stream);
int blr_low_rank_f32(const float* x, int64_t ldx, int64_t n_tokens,
                     const float* V, int v_layout, const float* U, int u_layout,
                     int I, int R, int O, float* out, int64_t ldo, float* z, void* stream);
int blr_dense_f32(const float* x, int64_t ldx, int64_t n_tokens,
                  const float* W, int w_layout, int I, int O, float* out, int64_t ldo, void* stream);

/* Symmetric weight quantiser (device): w (rows, K) 16-bit, contraction index contiguous ->
 * q int8 (rows, K) or packed uint8 (rows, K/2) and scale fp16 (rows) = max|w| / (127 | 7).
 * Per-group scales come from the same call on the view (rows * K / group, group): a group is quantised like a
 * row of its own and the layouts coincide.  No reference counterpart. */
int blr_quantize_sym(const void* w, int dtype, int64_t rows, int64_t K, int bits,
                     void* q, void* scale, void* stream);

/* Inverse of blr_quantize_sym: w (rows, K) in the 16-bit `dtype` = q * scale, rounded to that type.
 * `group` = 0 for one scale per row, else the number of consecutive contraction indices per scale.
 * K and the group width must be multiples of 16.  Used for quantised layers on more than 16 tokens, where the
 * tensor-core pipeline takes 16-bit factors.  No reference counterpart. */
int blr_dequantize_sym(const void* q, const void* scale, int64_t rows, int64_t K, int bits, int64_t group,
                       int dtype, void* w, void* stream);

/* Load / store probe: reads the operand arrays a, b, c once (any of them may have 0 bytes) and writes
 * out[n][o] = o / tile (tile > 0) or 0 (tile = 0): the memory traffic of an operator without its arithmetic.
 * Replaces triton_low_rank_load_store_fp16/_fp32 (triton_funcs/low_rank_kernels.py:419-449; kernels :163-236 store
 * the index of the 64-wide output tile) and triton_dense_load_store_fp16/_fp32 (dense_kernels.py:383-411; kernels
 * :190-227 store zeros).  out_kind: 0 fp16, 1 bf16, 2 fp32. */
int blr_load_store_probe(const void* a, size_t a_bytes, const void* b, size_t b_bytes, const void* c, size_t c_bytes,
                         int out_kind, void* out, int64_t n_tokens, int64_t out_features, int64_t ldo, int tile,
                         void* stream);

/* ---- The small kernels of a Llama-style decode step around the structured linears.  No counterpart among the
 * reference's operator files: its network harness runs HuggingFace's modules for them (models/llama7b.py,
 * network.py:60-94).  16-bit tensors of `dtype`, fp32 arithmetic, one rounding on the way out. */

/* out[r][:] = x[r][:] * rsqrt(mean(x[r][:]^2) + eps) * weight[:] for `rows` rows of d values (d, ldx, ldo multiples
 * of 8; pointers 16-byte aligned).  Models LlamaRMSNorm. */
int blr_rmsnorm(const void* x, int64_t ldx, int64_t rows, int d, const void* weight, float eps, int dtype,
                void* out, int64_t ldo, void* stream);
/* LayerNorm over the last dimension with optional weight and bias (NULL: none): out = (x - mean) * rsqrt(var + eps) * w + b,
 * fp32 arithmetic on 16-bit rows, one rounding; d a multiple of 8 and at most 2048 (BLR_ERR_UNSUPPORTED above).  What the
 * encoder and denoiser modules around the linears run between them (HuggingFace ViT's nn.LayerNorm in
 * models/vit_b_patch16_224.py, DiT/models.py:107-109); no counterpart among the reference's operator files. */
int blr_layernorm(const void* x, int64_t ldx, int64_t rows, int d, const void* weight, const void* bias, float eps,
                  int dtype, void* out, int64_t ldo, int64_t rows_per_group, int64_t ldw, int64_t ldb, int weight_plus_one,
                  void* stream);
/* rows_per_group > 0: weight and bias are matrices with one row (ldw / ldb apart) per group of rows_per_group
 * consecutive rows of x, and weight_plus_one uses 1 + weight: the adaLN modulation norm(x) * (1 + scale) + shift of a
 * DiT block (DiT/models.py:19-20, 120-121) in the norm's own pass.  rows_per_group = 0: one weight / bias for all rows.
 *
 * out = x + gate * y with gate one row per group of rows_per_group rows (the gated residual of the same block,
 * DiT/models.py:120-121): 16-byte accesses.  No counterpart among the reference's operator files. */
int blr_gated_add(const void* x, int64_t ldx, const void* y, int64_t ldy, const void* gate, int64_t ldg, int64_t rows,
                  int64_t rows_per_group, int d, int dtype, void* out, int64_t ldo, void* stream);

/* Rotary embedding and append to a static KV cache.  q, k, v: n_seq * n_tok rows (sequence-major) of heads * head_dim
 * values, row strides ldq / ldk / ldv.  Token t takes cache slot pos[t] (device int64) and the rotation angle of that
 * slot from cos_table / sin_table ((slots, head_dim / 2) fp32; pairs (i, i + head_dim / 2) rotate, as in HF's Llama).
 * q is rotated in place; rotated k and v are written to k_cache / v_cache [seq][head][pos[t]][:] (caches of
 * (n_seq, heads, slots, head_dim)). */
int blr_rope_append(void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                    const float* cos_table, const float* sin_table, const int64_t* pos,
                    int64_t n_seq, int n_tok, int heads, int head_dim, int slots, int dtype,
                    void* k_cache, void* v_cache, void* stream);

/* Attention of one query token per sequence over the first n_keys slots of the cache:
 * out[seq][head*head_dim + :] = softmax(scale * q . K^T) V, q (n_seq, heads * head_dim) with row stride ldq
 * (a multiple of 8, q 16-byte aligned); head_dim a power of two from 8 to 256.
 * The keys of a head are split over up to 8 CTAs whose partial results a second kernel merges; `scratch` holds the
 * partials (blr_attention_decode_scratch_bytes). */
size_t blr_attention_decode_scratch_bytes(int64_t n_seq, int heads, int head_dim, int n_keys);
int blr_attention_decode(const void* q, int64_t ldq, const void* k_cache, const void* v_cache,
                         int64_t n_seq, int heads, int head_dim, int slots, int n_keys, float scale, int dtype,
                         void* out, int64_t ldo, void* scratch, size_t scratch_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BLR_B200_H_ */
