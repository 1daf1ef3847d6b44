"""Loads libblr_b200.so (the C ABI in include/blr_b200.h): the ctypes binding, the thin PyTorch C++ extension
_blr_torch.so over the same ABI (TORCH_LIBRARY ops `blr_b200_ext::*`, the route of the hot operators), and the
workspace handling they share."""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libblr_b200.so")
EXT_PATH = os.path.join(HERE, "_blr_torch.so")

F16, BF16 = 0, 1
KMAJOR, MMAJOR = 0, 1
COLS_TORCH, COLS_GROUPED = 0, 1
OUT_INTERLEAVED, OUT_BLOCKED = 0, 1
FLAG_NONE, FLAG_ACT_INT8 = 0, 1
STREAM_MAX_TOKENS = 16

_i64, _int, _vp, _sz = C.c_int64, C.c_int, C.c_void_p, C.c_size_t


class BlastProblem(C.Structure):
    """blr_blast_problem of include/blr_b200.h."""
    _fields_ = [("U", _vp), ("V", _vp), ("S", _vp), ("u_scale", _vp), ("v_scale", _vp), ("bias", _vp), ("residual", _vp),
                ("ldr", _i64), ("out", _vp), ("ldo", _i64)]


ACT_NONE, ACT_SILU_MUL = 0, 1
ACT_OUT = {None: 0, "gelu": 0x10, "gelu_tanh": 0x20}   # output activations of the fused call above 16 tokens

# name -> (restype, argtypes); must list every symbol include/blr_b200.h declares
SIGNATURES = {
    "blr_version": (_int, []),
    "blr_debug_decode_path": (_int, [_int]),
    "blr_last_error": (C.c_char_p, []),
    "blr_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "blr_load_store_probe": (_int, [_vp, _sz, _vp, _sz, _vp, _sz, _int, _vp, _i64, _i64, _i64, _int, _vp]),
    "blr_scratch_alloc": (_vp, [_sz]),
    "blr_scratch_free": (_int, [_vp]),
    "blr_workspace_init": (_int, [_vp, _sz, _vp]),
    "blr_workspace_status": (_int, [_vp, _vp]),
    "blr_blast": (_int, [_vp, _i64, _i64, _int, _vp, _int, _vp, _int, _vp, _i64, _i64, _i64,
                         _int, _int, _int, _int, _int, _vp, _i64, _vp, _sz, _vp]),
    "blr_blast_rows": (_int, [_vp, _i64, _i64, _int, _vp, _int, _vp, _int, _vp, _i64, _i64, _i64,
                              _int, _int, _int, _int, _int, _int, _vp, _i64, _vp, _sz, _vp]),
    "blr_blast_coupling_bytes": (_sz, [_int, _int, _int]),
    "blr_blast_expand_coupling": (_int, [_vp, _i64, _i64, _i64, _int, _int, _int, _int, _vp, _sz, _vp]),
    "blr_blast_rows_prepared": (_int, [_vp, _i64, _i64, _int, _vp, _int, _vp, _int, _vp, _i64, _i64, _i64,
                                       _int, _int, _int, _int, _int, _int, _vp, _i64, _vp, _sz, _vp, _vp]),
    "blr_blast_multi": (_int, [_vp, _i64, _vp, _int, _i64, _int, _int, C.POINTER(BlastProblem), _i64, _i64, _i64,
                               _int, _int, _int, _int, _int, _int, _vp, _sz, _vp]),
    "blr_blast_static": (_int, [_vp, _i64, _i64, _int, _vp, _int, _vp, _int, _vp, _i64, _i64, _i64,
                                _int, _int, _int, _int, _int, _vp, _i64, _vp]),
    "blr_blast_static_status": (_int, [_vp]),
    "blr_blast_wq": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64,
                            _int, _int, _int, _int, _int, _int, _vp, _i64, _vp, _sz, _vp]),
    "blr_monarch": (_int, [_vp, _i64, _i64, _int, _vp, _int, _int, _vp, _int,
                           _int, _int, _int, _int, _int, _vp, _i64, _vp, _sz, _vp]),
    "blr_low_rank": (_int, [_vp, _i64, _i64, _int, _vp, _int, _vp, _int, _int, _int, _int,
                            _vp, _i64, _vp, _sz, _vp]),
    "blr_dense": (_int, [_vp, _i64, _i64, _int, _vp, _int, _int, _int, _vp, _i64, _vp]),
    "blr_blast_f32": (_int, [_vp, _i64, _i64, _vp, _int, _vp, _int, _vp, _i64, _i64, _i64,
                             _int, _int, _int, _int, _vp, _i64, _vp, _vp, _vp]),
    "blr_monarch_f32": (_int, [_vp, _i64, _i64, _vp, _int, _int, _vp, _int,
                               _int, _int, _int, _int, _int, _vp, _i64, _vp, _vp]),
    "blr_low_rank_f32": (_int, [_vp, _i64, _i64, _vp, _int, _vp, _int, _int, _int, _int, _vp, _i64, _vp, _vp]),
    "blr_dense_f32": (_int, [_vp, _i64, _i64, _vp, _int, _int, _int, _vp, _i64, _vp]),
    "blr_host_staging_bytes": (_sz, [_i64, _i64, _i64]),
    "blr_host_flush": (_int, [_vp]),
    "blr_blast_host": (_int, [_vp, _i64, _i64, _int, _vp, _int, _vp, _int, _vp, _i64, _i64, _i64,
                              _int, _int, _int, _int, _int, _vp, _i64, _vp, _sz, _vp, _sz, _vp]),
    "blr_blast_wq_host": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64,
                                 _int, _int, _int, _int, _int, _int, _vp, _i64, _vp, _sz, _vp, _sz, _vp]),
    "blr_rmsnorm": (_int, [_vp, _i64, _i64, _int, _vp, C.c_float, _int, _vp, _i64, _vp]),
    "blr_layernorm": (_int, [_vp, _i64, _i64, _int, _vp, _vp, C.c_float, _int, _vp, _i64, _i64, _i64, _i64, _int, _vp]),
    "blr_gated_add": (_int, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _int, _int, _vp, _i64, _vp]),
    "blr_rope_append": (_int, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64, _int, _int, _int, _int, _int, _vp, _vp, _vp]),
    "blr_attention_decode_scratch_bytes": (_sz, [_i64, _int, _int, _int]),
    "blr_attention_decode": (_int, [_vp, _i64, _vp, _vp, _i64, _int, _int, _int, _int, C.c_float, _int, _vp, _i64, _vp, _sz, _vp]),
    "blr_quantize_sym": (_int, [_vp, _int, _i64, _i64, _int, _vp, _vp, _vp]),
    "blr_dequantize_sym": (_int, [_vp, _vp, _i64, _i64, _int, _i64, _int, _vp, _vp]),
}

_lib = None
_lock = threading.RLock()


def load() -> C.CDLL:
    """Loads the shared library; raises if it has not been built (there is no fallback path)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with `python -m mem_efficient_blr_b200.build` "
                    "(needs nvcc); this package has no CPU or Triton fallback")
            lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)  # (the torch extension links against it by soname)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype, fn.argtypes = res, args
            _lib = lib
    return _lib


_ext = None
_ext_tried = False


def _ext_registered() -> bool:
    """True when a copy of the extension is already loaded: its operators resolve.  Loading a second copy would
    register the operator namespace twice, which torch answers by aborting the process."""
    try:
        torch.ops.blr_b200_ext.blast
        return True
    except (AttributeError, RuntimeError):
        return False


def ext():
    """torch.ops.blr_b200_ext once _blr_torch.so is loaded, None where it has not been built (the operators then go
    through ctypes: same kernels, more host time per call).  Setting BLR_B200_NO_TORCH_EXT=1 keeps it unloaded."""
    global _ext, _ext_tried
    if _ext_tried:
        return _ext
    with _lock:
        if not _ext_tried:
            if os.path.exists(EXT_PATH) and LIB_PATH.endswith("libblr_b200.so") and not os.environ.get("BLR_B200_NO_TORCH_EXT"):
                load()
                if not _ext_registered():  # (a process that has just built the extension has it loaded from the build folder)
                    torch.ops.load_library(EXT_PATH)
                _ext = torch.ops.blr_b200_ext
            _ext_tried = True
    return _ext


def check(rc: int) -> None:
    if rc != 0:
        msg = load().blr_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"blr_b200 error {rc}: {msg}")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float16:
        return F16
    if dt == torch.bfloat16:
        return BF16
    raise AssertionError(f"expected float16 or bfloat16 tensors, got {dt}")


def stream_ptr(device: torch.device) -> int:
    """The current stream of `device` as an integer handle."""
    idx = device.index
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device() if idx is None else idx)


# ----------------------------------------------------------------------------- workspaces
# One scratch buffer per (device, stream): calls that share a workspace must be ordered on one stream.
_workspaces: dict = {}


class _RawBuffer:
    """Device memory from blr_scratch_alloc, exposed through the CUDA array interface so that torch can view it."""

    def __init__(self, nbytes: int):
        self.ptr = load().blr_scratch_alloc(nbytes)
        if not self.ptr:
            raise RuntimeError("blr_b200: " + load().blr_last_error().decode("utf-8", "replace"))
        self.nbytes = nbytes
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (self.ptr, False), "version": 3}

    def __del__(self):
        try:
            if self.ptr:
                load().blr_scratch_free(self.ptr)
        except Exception:
            pass


def _alloc_outside_graph_pools(nbytes: int, device: torch.device) -> torch.Tensor:
    """A long-lived scratch buffer must not come from a CUDA-graph memory pool: torch.compile's CUDA-graph trees
    (mode='reduce-overhead', what the reference's network harness uses, models/llama7b.py:65) route every allocation
    of the thread that warms up or records a graph into the graph's private pool and then insist that nothing but
    the graph's outputs lives there.  So the buffer comes from cudaMalloc through the library and torch only views
    it.  While a capture is under way cudaMalloc is not allowed: the buffer then comes from the capture's pool (a
    caller that captures without a warm-up call owns that choice)."""
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(nbytes, dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        raw = _RawBuffer(nbytes)
        t = torch.as_tensor(raw, device=device)
    t._blr_owner = raw  # the view keeps the allocation alive
    return t


class _RawView:
    """Device memory owned elsewhere (the torch extension's workspace registry), viewable by torch."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


_ext_views: dict = {}


def workspace(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    e = ext()
    if e is not None:
        # one registry for both routes: the extension owns the buffers, this layer views them
        ptr, cap = e.workspace(key[0], stream, nbytes)
        v = _ext_views.get(key)
        if v is None or v.data_ptr() != ptr or v.numel() != cap:
            with torch.cuda.device(key[0]):
                v = _ext_views[key] = torch.as_tensor(_RawView(ptr, cap), device=torch.device("cuda", key[0]))
        return v
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        cap = max(nbytes, 1 << 20)
        if ws is not None:
            cap = max(cap, 2 * ws.numel())
        ws = _alloc_outside_graph_pools(cap, device)
        check(load().blr_workspace_init(ws.data_ptr(), ws.numel(), stream))
        _workspaces[key] = ws
    return ws


_stagings: dict = {}
_ext_staging_views: dict = {}


def staging(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    """Device buffer that the host-buffer entry points copy x into and the result out of; one per (device, stream)."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    e = ext()
    if e is not None:
        ptr, cap = e.staging(key[0], stream, nbytes)
        v = _ext_staging_views.get(key)
        if v is None or v.data_ptr() != ptr or v.numel() != cap:
            with torch.cuda.device(key[0]):
                v = _ext_staging_views[key] = torch.as_tensor(_RawView(ptr, cap), device=torch.device("cuda", key[0]))
        return v
    st = _stagings.get(key)
    if st is None or st.numel() < nbytes:
        if st is not None:
            # the ring's slots are cut from the buffer's size: drain the copies in flight before it changes
            torch.cuda.synchronize(device)
        st = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _stagings[key] = st
    return st


def workspace_status(device: torch.device) -> None:
    """Raises if a kernel that used this device's current-stream workspace reported a timed-out wait."""
    st = stream_ptr(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(), st)
    e = ext()
    if e is not None:
        check(e.workspace_status(key[0], st))  # (re-initialises the workspace after an error)
        return
    ws = _workspaces.get(key)
    if ws is not None:
        rc = load().blr_workspace_status(ws.data_ptr(), st)
        if rc != 0:
            load().blr_workspace_init(ws.data_ptr(), ws.numel(), st)
            check(rc)
