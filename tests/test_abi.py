"""CPU-side checks of the boundary: the shared library loads, exports every symbol the header declares,
and the Python operator modules keep the reference's names.  No compute calls (there is no GPU here)."""
import ctypes
import importlib
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from mem_efficient_blr_b200 import build as b
    b.build()  # no-op when the library is newer than its sources
    from mem_efficient_blr_b200 import _lib
    return _lib.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "blr_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(blr_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    from mem_efficient_blr_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/blr_b200.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_host_only_entry_points(lib):
    assert lib.blr_version() >= 100
    # groups * tokens * width elements: 4-byte + 2-byte regions, after the fixed part
    fixed = 1024 + (2 << 20)   # control words + the fp32 accumulation area of the cluster kernel
    assert lib.blr_workspace_bytes(16, 16, 1024) == fixed + 16 * 16 * 1024 * 6
    assert lib.blr_workspace_bytes(1, 0, 0) == fixed
    big = lib.blr_workspace_bytes(2048, 16, 1024)
    assert big >= 256 + 2048 * 16 * 1024 * 6 + 16 * 16 * 1024 * 32


def test_null_arguments_are_rejected_without_touching_a_device(lib):
    rc = lib.blr_dense(None, 8, 1, 0, None, 0, 8, 8, None, 8, None)
    assert rc == -1
    assert b"null" in lib.blr_last_error()
    rc = lib.blr_blast_wq(ctypes.c_void_p(16), 64, 1, 0, ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16),
                          ctypes.c_void_p(16), ctypes.c_void_p(16), 1, 1, 1, 3, 0, 4, 16, 16, 16, ctypes.c_void_p(16), 64,
                          None, 0, None)
    assert rc == -1 and b"bits" in lib.blr_last_error()


def test_reference_probe_names_exist():
    import mem_efficient_blr_b200.dense_kernels as dk
    import mem_efficient_blr_b200.low_rank_kernels as lk
    for m, names in ((lk, ("triton_low_rank_load_store_fp16", "triton_low_rank_load_store_fp32")),
                     (dk, ("triton_dense_load_store_fp16", "triton_dense_load_store_fp32"))):
        for n in names:
            assert callable(getattr(m, n))


REFERENCE_NAMES = {
    "blast_kernels": ["triton_blast_partial_fp16", "triton_blast_partial_fp32", "triton_blast_partial_grouped_fp16",
                      "triton_blast_partial_grouped_fp32", "triton_blast_partial_grouped_persistent_fp16",
                      "triton_blast_partial_grouped_persistent_fp32", "triton_blast_full_fp16", "triton_blast_full_fp32",
                      "triton_blast_bmm_fp16", "triton_blast_bmm_fp32", "get_triton_blast_partial_fp16_config",
                      "get_triton_blast_partial_grouped_fp16_config", "get_triton_blast_partial_grouped_persistent_fp16_config",
                      "get_triton_blast_full_fp16_config", "get_triton_blast_bmm_xv_fp16_config",
                      "get_triton_blast_bmm_sxv_fp16_config", "get_triton_blast_bmm_usxv_fp16_config"],
    "blast_sym_quant_kernels": ["triton_blast_bmm_int8_fp16", "get_triton_blast_bmm_xv_int8_fp16_config",
                                "get_triton_blast_bmm_sxv_int8_fp16_config", "get_triton_blast_bmm_usxv_int8_fp16_config"],
    "monarch_kernels": ["triton_monarch_right_fp16", "triton_monarch_right_fp32", "triton_monarch_right_ideal_fp16",
                        "triton_monarch_right_ideal_fp32", "triton_monarch_right_left_fp16", "triton_monarch_right_left_fp32",
                        "get_triton_monarch_right_fp16_config", "get_triton_monarch_right_ideal_fp16_config",
                        "get_triton_monarch_right_left_fp16_config"],
    "low_rank_kernels": ["triton_low_rank_fp16", "triton_low_rank_fp32", "get_triton_low_rank_fp16_config"],
    "dense_kernels": ["triton_dense_fp16", "triton_dense_fp32", "get_triton_dense_fp16_config"],
}


@pytest.mark.parametrize("module", sorted(REFERENCE_NAMES))
def test_reference_function_names_exist(module):
    m = importlib.import_module(f"mem_efficient_blr_b200.{module}")
    for name in REFERENCE_NAMES[module]:
        assert callable(getattr(m, name)), name
        if name.startswith("get_"):
            import pickle
            pickle.dumps(getattr(m, name)())  # the reference's harness pickles these (layer.py:310-326)


def test_operators_refuse_cpu_tensors():
    import torch
    import mem_efficient_blr_b200.dense_kernels as dk
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        dk.dense_torch_layout(torch.zeros(2, 8, dtype=torch.float16), torch.zeros(8, 8, dtype=torch.float16))


def test_torch_extension_loads_and_declares_the_operators():
    """The thin C++ extension over the C ABI: built in-tree, loads without a GPU, declares every hot operator with a
    Meta kernel (shape inference for torch.compile) and refuses CPU tensors like the rest of the package."""
    import torch
    from mem_efficient_blr_b200 import _lib
    e = _lib.ext()
    assert e is not None, "mem_efficient_blr_b200/_blr_torch.so is missing: python -m mem_efficient_blr_b200.build"
    for name in ("blast", "blast_wq", "monarch", "low_rank", "dense", "blast_wq_host", "host_flush", "workspace",
                 "staging", "workspace_status"):
        assert hasattr(e, name), name
    x = torch.empty(5, 64, device="meta", dtype=torch.bfloat16)
    w = torch.empty(48, 64, device="meta", dtype=torch.bfloat16)
    assert e.dense(x, w, _lib.KMAJOR, 64, 48).shape == (5, 48)
    u = torch.empty(4, 12, 32, device="meta", dtype=torch.bfloat16)
    v = torch.empty(4, 32, 16, device="meta", dtype=torch.bfloat16)
    s_ = torch.empty(4, 4, 32, device="meta", dtype=torch.bfloat16)
    assert e.blast(x, u, v, s_, _lib.KMAJOR, _lib.KMAJOR, 128, 32, 1, 4, 16, 12, 32, 0).shape == (5, 48)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        e.dense(torch.zeros(2, 8, dtype=torch.float16), torch.zeros(8, 8, dtype=torch.float16), _lib.KMAJOR, 8, 8)


def test_extension_built_and_used_in_one_process():
    """A process that builds the extension has it loaded from the build folder already; taking it into use afterwards
    must not load the in-tree copy on top (torch aborts the process on a second registration of the namespace)."""
    import subprocess
    import sys
    code = ("from mem_efficient_blr_b200 import build as b, _lib\n"
            "b.build()\n"
            "b.build_torch_ext(force=True)\n"
            "e = _lib.ext()\n"
            "assert e is not None and hasattr(e, 'blast_wq')\n"
            "print('ok')\n")
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stderr[-2000:]
