// Thin PyTorch C++ extension over the C ABI of libblr_b200.so: the operators as TORCH_LIBRARY ops (CUDA + Meta
// kernels), so that an eager call costs a dispatcher hop instead of a ctypes conversion per argument, and a compiled
// graph calls straight into C++.  No arithmetic lives here: tensors in, pointers and sizes to the C entry points,
// tensors out.  The signatures are those of the Python layer's operators (ops.py), which mirror the reference's
// operator functions one level up (triton_funcs/*.py entry points; models/wrappers.py:143-146 resolves them by name).
//
// Scratch: one workspace per (device, stream), from cudaMalloc through the library (PyTorch's CUDA-graph memory pools
// are no home for a long-lived buffer); while a stream capture is under way the buffer comes from the capture's pool.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime_api.h>
#include <torch/library.h>

#include <map>
#include <mutex>
#include <utility>
#include <vector>

#include "blr_b200.h"

namespace {

struct Scratch {
  void* ptr = nullptr;
  size_t bytes = 0;
  at::Tensor holder;  // set when the buffer had to come from torch's allocator (stream capture under way)
};

std::mutex g_mu;
std::map<std::pair<int, cudaStream_t>, Scratch> g_ws, g_staging;
std::vector<Scratch> g_retired;

void check_rc(int rc) { TORCH_CHECK(rc == 0, "blr_b200 error ", rc, ": ", blr_last_error()); }

bool capturing(cudaStream_t st) {
  cudaStreamCaptureStatus s = cudaStreamCaptureStatusNone;
  return cudaStreamIsCapturing(st, &s) == cudaSuccess && s != cudaStreamCaptureStatusNone;
}

// Grows geometrically.
Scratch& scratch(std::map<std::pair<int, cudaStream_t>, Scratch>& reg, int dev, cudaStream_t st, size_t need, bool is_ws) {
  std::lock_guard<std::mutex> lock(g_mu);
  Scratch& s = reg[{dev, st}];
  if (s.bytes >= need) return s;
  size_t cap = need < (size_t(1) << 20) ? (size_t(1) << 20) : need;
  if (cap < 2 * s.bytes) cap = 2 * s.bytes;
  if (s.ptr != nullptr) {
    // A replaced buffer stays allocated: CUDA graphs captured earlier hold its address, work in flight may still use
    // it, and nothing may synchronise or free while a capture is under way.  Growth is geometric, so the retired
    // buffers of a stream add up to less than its current one.
    g_retired.push_back(s);
    s = Scratch();
  }
  if (capturing(st)) {
    s.holder = at::empty({(int64_t)cap}, at::TensorOptions().dtype(at::kByte).device(at::kCUDA, dev));
    s.ptr = s.holder.data_ptr();
  } else {
    s.ptr = blr_scratch_alloc(cap);
    TORCH_CHECK(s.ptr != nullptr, "blr_b200: ", blr_last_error());
  }
  s.bytes = cap;
  if (is_ws) check_rc(blr_workspace_init(s.ptr, s.bytes, st));
  return s;
}

int dtype_code(const at::Tensor& x) {
  if (x.scalar_type() == at::kHalf) return BLR_DTYPE_F16;
  TORCH_CHECK(x.scalar_type() == at::kBFloat16, "expected float16 or bfloat16 tensors, got ", x.scalar_type());
  return BLR_DTYPE_BF16;
}

// (N, I) activations as the TMA rules want them: unit inner stride, row stride a multiple of 8 elements, 16-byte
// aligned base; copies only if the input forces it.
at::Tensor rows(const at::Tensor& x) {
  TORCH_CHECK(x.dim() == 2, "x must be (tokens, features)");
  at::Tensor r = x;
  if (r.stride(1) != 1 || (r.size(0) > 1 && r.stride(0) % 8 != 0) || reinterpret_cast<uintptr_t>(r.data_ptr()) % 16 != 0) {
    r = r.contiguous();
    if (reinterpret_cast<uintptr_t>(r.data_ptr()) % 16 != 0) r = r.clone();
  }
  return r;
}

void need_factors(const at::Tensor& x, std::initializer_list<const at::Tensor*> factors) {
  TORCH_CHECK(x.is_cuda(), "blr_b200 operators need CUDA tensors: there is no CPU implementation in this package");
  for (const at::Tensor* t : factors) {
    TORCH_CHECK(t->is_cuda() && t->device() == x.device(), "x and the factors must live on one CUDA device");
    TORCH_CHECK(t->is_contiguous(), "factor tensors must be contiguous");
  }
}

struct Call {
  c10::cuda::CUDAGuard guard;
  cudaStream_t st;
  int dev;
  explicit Call(const at::Tensor& x) : guard(x.device()), st(at::cuda::getCurrentCUDAStream(x.device().index()).stream()), dev(x.device().index()) {}
  Scratch& ws(int64_t n, int64_t groups, int64_t width) { return scratch(g_ws, dev, st, blr_workspace_bytes(n, groups, width), true); }
};

// ----------------------------------------------------------------------------------------------- operators
at::Tensor blast(const at::Tensor& x_in, const at::Tensor& U, const at::Tensor& V, const at::Tensor& S, int64_t u_layout,
                 int64_t v_layout, int64_t s_i, int64_t s_j, int64_t s_r, int64_t b, int64_t P, int64_t Q, int64_t R, int64_t flags,
                 int64_t b_out, const c10::optional<at::Tensor>& E) {
  need_factors(x_in, {&U, &V, &S});
  const int64_t bo = b_out < 0 ? b : b_out;
  if (x_in.size(0) == 0) return at::empty({0, bo * Q}, x_in.options());
  const at::Tensor x = rows(x_in);
  TORCH_CHECK(U.scalar_type() == x.scalar_type() && V.scalar_type() == x.scalar_type() && S.scalar_type() == x.scalar_type(),
              "x, U, V, S must share one 16-bit dtype");
  Call c(x);
  const int64_t n = x.size(0);
  at::Tensor out = at::empty({n, bo * Q}, x.options());
  Scratch& w = c.ws(n, b, R);
  const void* e_ready = nullptr;  // expanded coupling factors built once by the caller (prefill sizes)
  if (E.has_value() && E->defined()) {
    TORCH_CHECK(E->is_cuda() && E->device() == x.device() && E->is_contiguous() &&
                    (size_t)E->nbytes() >= blr_blast_coupling_bytes((int)b, (int)bo, (int)R),
                "E must hold blr_blast_coupling_bytes bytes on x's device");
    e_ready = E->data_ptr();
  }
  check_rc(blr_blast_rows_prepared(x.data_ptr(), x.stride(0), n, dtype_code(x), U.data_ptr(), (int)u_layout, V.data_ptr(),
                                   (int)v_layout, S.data_ptr(), s_i, s_j, s_r, (int)b, (int)bo, (int)P, (int)Q, (int)R, (int)flags,
                                   out.data_ptr(), out.stride(0), w.ptr, w.bytes, c.st, e_ready));
  return out;
}

at::Tensor blast_wq(const at::Tensor& x_in, const at::Tensor& Uq, const at::Tensor& u_scale, const at::Tensor& Vq,
                    const at::Tensor& v_scale, const at::Tensor& S, int64_t s_i, int64_t s_j, int64_t s_r, int64_t bits,
                    int64_t group, int64_t b, int64_t P, int64_t Q, int64_t R) {
  need_factors(x_in, {&Uq, &u_scale, &Vq, &v_scale, &S});
  if (x_in.size(0) == 0) return at::empty({0, b * Q}, x_in.options());
  const at::Tensor x = rows(x_in);
  TORCH_CHECK(u_scale.scalar_type() == at::kHalf && v_scale.scalar_type() == at::kHalf, "scales are fp16");
  TORCH_CHECK(S.scalar_type() == x.scalar_type(), "x and S must share one 16-bit dtype");
  Call c(x);
  const int64_t n = x.size(0);
  at::Tensor out = at::empty({n, b * Q}, x.options());
  Scratch& w = c.ws(n, b, R);
  check_rc(blr_blast_wq(x.data_ptr(), x.stride(0), n, dtype_code(x), Uq.data_ptr(), u_scale.data_ptr(), Vq.data_ptr(),
                        v_scale.data_ptr(), S.data_ptr(), s_i, s_j, s_r, (int)bits, (int)group, (int)b, (int)P, (int)Q, (int)R,
                        out.data_ptr(), out.stride(0), w.ptr, w.bytes, c.st));
  return out;
}

at::Tensor monarch(const at::Tensor& x_in, const at::Tensor& w1, const at::Tensor& w2, int64_t w1_layout, int64_t w1_cols,
                   int64_t w2_layout, int64_t b, int64_t P, int64_t rank, int64_t Qs, int64_t out_order) {
  need_factors(x_in, {&w1, &w2});
  if (x_in.size(0) == 0) return at::empty({0, b * Qs}, x_in.options());
  const at::Tensor x = rows(x_in);
  TORCH_CHECK(w1.scalar_type() == x.scalar_type() && w2.scalar_type() == x.scalar_type(), "x and the factors must share one 16-bit dtype");
  Call c(x);
  const int64_t n = x.size(0);
  at::Tensor out = at::empty({n, b * Qs}, x.options());
  Scratch& w = c.ws(n, b, rank);
  check_rc(blr_monarch(x.data_ptr(), x.stride(0), n, dtype_code(x), w1.data_ptr(), (int)w1_layout, (int)w1_cols, w2.data_ptr(),
                       (int)w2_layout, (int)b, (int)P, (int)rank, (int)Qs, (int)out_order, out.data_ptr(), out.stride(0), w.ptr,
                       w.bytes, c.st));
  return out;
}

at::Tensor low_rank(const at::Tensor& x_in, const at::Tensor& V, const at::Tensor& U, int64_t v_layout, int64_t u_layout, int64_t I,
                    int64_t R, int64_t O) {
  need_factors(x_in, {&V, &U});
  if (x_in.size(0) == 0) return at::empty({0, O}, x_in.options());
  const at::Tensor x = rows(x_in);
  TORCH_CHECK(V.scalar_type() == x.scalar_type() && U.scalar_type() == x.scalar_type(), "x and the factors must share one 16-bit dtype");
  Call c(x);
  const int64_t n = x.size(0);
  at::Tensor out = at::empty({n, O}, x.options());
  Scratch& w = c.ws(n, 1, R);
  check_rc(blr_low_rank(x.data_ptr(), x.stride(0), n, dtype_code(x), V.data_ptr(), (int)v_layout, U.data_ptr(), (int)u_layout, (int)I,
                        (int)R, (int)O, out.data_ptr(), out.stride(0), w.ptr, w.bytes, c.st));
  return out;
}

at::Tensor dense(const at::Tensor& x_in, const at::Tensor& W, int64_t w_layout, int64_t I, int64_t O) {
  need_factors(x_in, {&W});
  if (x_in.size(0) == 0) return at::empty({0, O}, x_in.options());
  const at::Tensor x = rows(x_in);
  TORCH_CHECK(W.scalar_type() == x.scalar_type(), "x and W must share one 16-bit dtype");
  Call c(x);
  const int64_t n = x.size(0);
  at::Tensor out = at::empty({n, O}, x.options());
  check_rc(blr_dense(x.data_ptr(), x.stride(0), n, dtype_code(x), W.data_ptr(), (int)w_layout, (int)I, (int)O, out.data_ptr(),
                     out.stride(0), c.st));
  return out;
}

// Host-buffer call (x_host and out_host pinned, N <= 16): copy-in, kernels and copy-out of consecutive calls overlap on
// the library's copy streams; out_host is valid after host_flush() and a synchronisation of the current stream.
void blast_wq_host(const at::Tensor& x_host, at::Tensor& out_host, const at::Tensor& Uq, const at::Tensor& u_scale,
                   const at::Tensor& Vq, const at::Tensor& v_scale, const at::Tensor& S, int64_t bits, int64_t group) {
  TORCH_CHECK(!x_host.is_cuda() && !out_host.is_cuda(), "x_host and out_host are host tensors");
  need_factors(S, {&Uq, &u_scale, &Vq, &v_scale});
  const int64_t per = bits == 8 ? 1 : 2;
  const int64_t b = u_scale.size(0), Q = u_scale.size(1), R = v_scale.size(1), P = Vq.size(-1) * per, n = x_host.size(0);
  TORCH_CHECK(x_host.dim() == 2 && out_host.dim() == 2 && n <= 16 && x_host.size(1) == b * P && out_host.size(0) == n &&
                  out_host.size(1) == b * Q && x_host.scalar_type() == S.scalar_type() && out_host.scalar_type() == S.scalar_type() &&
                  x_host.stride(1) == 1 && out_host.stride(1) == 1,
              "x_host (N <= 16, b*P) and out_host (N, b*Q) must be 16-bit host tensors of the factors' dtype");
  Call c(S);
  Scratch& w = scratch(g_ws, c.dev, c.st, blr_workspace_bytes(16, b, R), true);
  Scratch& sg = scratch(g_staging, c.dev, c.st, blr_host_staging_bytes(16, b * P, b * Q), false);
  check_rc(blr_blast_wq_host(x_host.data_ptr(), x_host.stride(0), n, dtype_code(S), Uq.data_ptr(), u_scale.data_ptr(), Vq.data_ptr(),
                             v_scale.data_ptr(), S.data_ptr(), b * R, R, 1, (int)bits, (int)group, (int)b, (int)P, (int)Q, (int)R,
                             out_host.data_ptr(), out_host.stride(0), sg.ptr, sg.bytes, w.ptr, w.bytes, c.st));
}

void host_flush(int64_t device) {
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  check_rc(blr_host_flush(at::cuda::getCurrentCUDAStream((c10::DeviceIndex)device).stream()));
}

// The workspace of (device, stream), grown to at least nbytes: (pointer, bytes).  For the parts of the Python layer that
// still call the C ABI through ctypes, and for tests that look into the scratch.
std::vector<int64_t> workspace(int64_t device, int64_t stream, int64_t nbytes) {
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  Scratch& w = scratch(g_ws, (int)device, reinterpret_cast<cudaStream_t>(stream), (size_t)nbytes, true);
  return {(int64_t)reinterpret_cast<uintptr_t>(w.ptr), (int64_t)w.bytes};
}

// The staging buffer of the host-buffer calls of (device, stream), likewise.
std::vector<int64_t> staging(int64_t device, int64_t stream, int64_t nbytes) {
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  Scratch& w = scratch(g_staging, (int)device, reinterpret_cast<cudaStream_t>(stream), (size_t)nbytes, false);
  return {(int64_t)reinterpret_cast<uintptr_t>(w.ptr), (int64_t)w.bytes};
}

// Status of the workspace of (device, stream) (synchronises the stream): 0, or a BLR_ERR_* code after which the
// workspace has been re-initialised.
int64_t workspace_status(int64_t device, int64_t stream) {
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  Scratch s;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_ws.find({(int)device, reinterpret_cast<cudaStream_t>(stream)});
    if (it == g_ws.end()) return 0;
    s = it->second;
  }
  const int rc = blr_workspace_status(s.ptr, reinterpret_cast<void*>(stream));
  if (rc != 0) blr_workspace_init(s.ptr, s.bytes, reinterpret_cast<void*>(stream));
  return rc;
}

// ----------------------------------------------------------------------------------------------- shapes only
at::Tensor blast_meta(const at::Tensor& x, const at::Tensor&, const at::Tensor&, const at::Tensor&, int64_t, int64_t, int64_t, int64_t,
                      int64_t, int64_t b, int64_t, int64_t Q, int64_t, int64_t, int64_t b_out, const c10::optional<at::Tensor>&) {
  return at::empty_symint({x.sym_size(0), c10::SymInt((b_out < 0 ? b : b_out) * Q)}, x.options());
}
at::Tensor blast_wq_meta(const at::Tensor& x, const at::Tensor&, const at::Tensor&, const at::Tensor&, const at::Tensor&,
                         const at::Tensor&, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t b, int64_t, int64_t Q, int64_t) {
  return at::empty_symint({x.sym_size(0), c10::SymInt(b * Q)}, x.options());
}
at::Tensor monarch_meta(const at::Tensor& x, const at::Tensor&, const at::Tensor&, int64_t, int64_t, int64_t, int64_t b, int64_t, int64_t,
                        int64_t Qs, int64_t) {
  return at::empty_symint({x.sym_size(0), c10::SymInt(b * Qs)}, x.options());
}
at::Tensor low_rank_meta(const at::Tensor& x, const at::Tensor&, const at::Tensor&, int64_t, int64_t, int64_t, int64_t, int64_t O) {
  return at::empty_symint({x.sym_size(0), c10::SymInt(O)}, x.options());
}
at::Tensor dense_meta(const at::Tensor& x, const at::Tensor&, int64_t, int64_t, int64_t O) {
  return at::empty_symint({x.sym_size(0), c10::SymInt(O)}, x.options());
}

}  // namespace

TORCH_LIBRARY(blr_b200_ext, m) {
  m.def("blast(Tensor x, Tensor U, Tensor V, Tensor S, int u_layout, int v_layout, int s_i, int s_j, int s_r, int b, int P, int Q, "
        "int R, int flags, int b_out=-1, Tensor? E=None) -> Tensor");
  m.def("blast_wq(Tensor x, Tensor Uq, Tensor u_scale, Tensor Vq, Tensor v_scale, Tensor S, int s_i, int s_j, int s_r, int bits, "
        "int group, int b, int P, int Q, int R) -> Tensor");
  m.def("monarch(Tensor x, Tensor w1, Tensor w2, int w1_layout, int w1_cols, int w2_layout, int b, int P, int rank, int Qs, "
        "int out_order) -> Tensor");
  m.def("low_rank(Tensor x, Tensor V, Tensor U, int v_layout, int u_layout, int I, int R, int O) -> Tensor");
  m.def("dense(Tensor x, Tensor W, int w_layout, int I, int O) -> Tensor");
  m.def("blast_wq_host(Tensor x_host, Tensor(a!) out_host, Tensor Uq, Tensor u_scale, Tensor Vq, Tensor v_scale, Tensor S, int bits, "
        "int group) -> ()");
  m.def("host_flush(int device) -> ()", &host_flush);
  m.def("workspace(int device, int stream, int nbytes) -> int[]", &workspace);
  m.def("staging(int device, int stream, int nbytes) -> int[]", &staging);
  m.def("workspace_status(int device, int stream) -> int", &workspace_status);
}

TORCH_LIBRARY_IMPL(blr_b200_ext, CUDA, m) {
  m.impl("blast", &blast);
  m.impl("blast_wq", &blast_wq);
  m.impl("monarch", &monarch);
  m.impl("low_rank", &low_rank);
  m.impl("dense", &dense);
}

// CPU tensors: the same refusal as everywhere else in this package (the device functions check is_cuda first)
TORCH_LIBRARY_IMPL(blr_b200_ext, CPU, m) {
  m.impl("blast", &blast);
  m.impl("blast_wq", &blast_wq);
  m.impl("monarch", &monarch);
  m.impl("low_rank", &low_rank);
  m.impl("dense", &dense);
}

// the host-buffer call mixes host tensors (x, out) with device tensors (factors): one kernel for every backend key
TORCH_LIBRARY_IMPL(blr_b200_ext, CompositeExplicitAutograd, m) { m.impl("blast_wq_host", &blast_wq_host); }

TORCH_LIBRARY_IMPL(blr_b200_ext, Meta, m) {
  m.impl("blast", &blast_meta);
  m.impl("blast_wq", &blast_wq_meta);
  m.impl("monarch", &monarch_meta);
  m.impl("low_rank", &low_rank_meta);
  m.impl("dense", &dense_meta);
}
