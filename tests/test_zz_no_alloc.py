"""The entry point with built-in scratch (blr_blast_static) must give what blr_blast gives.

Some callers cannot allocate device memory or carry a workspace around (a plug-in inside a host that owns the
allocator, a thread that must not hit cudaMalloc's implicit synchronisation).  For them the library keeps 4 MiB
of scratch in its own device image.  This test calls the entry point through the C ABI twice in a row - the
second call finds the first call's leftovers in the scratch - and compares both results with the ordinary entry
point on the same inputs.  It also checks that a problem whose scratch would not fit is refused.
The file name sorts last on purpose, so a run that stops at the first failure has already run every other test.
"""
import pytest
import torch

from oracle import blr_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 1e-2  # the bound every GPU parity test here uses (relative Frobenius error)


def _call_static(lib, L, x2, U, Vt, S, b, P, Q, R):
    out = torch.empty((x2.shape[0], b * Q), dtype=x2.dtype, device=x2.device)
    rc = lib.blr_blast_static(x2.data_ptr(), x2.stride(0), x2.shape[0], L.dtype_code(x2.dtype), U.data_ptr(), L.KMAJOR,
                              Vt.data_ptr(), L.KMAJOR, S.data_ptr(), b * R, R, 1, b, P, Q, R, L.FLAG_NONE,
                              out.data_ptr(), out.stride(0), L.stream_ptr(x2.device))
    return rc, out


@pytest.mark.parametrize("shape", [(16, 4096, 11008, 16, 1024), (3, 512, 768, 4, 128)])
def test_static_scratch_entry_matches_workspace_entry_twice(shape):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from mem_efficient_blr_b200 import _lib as L
    import mem_efficient_blr_b200.blast_kernels as bk
    lib = L.load()
    N, I, O, b, R = shape
    P, Q = I // b, O // b
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, torch.float16, seed=11)
    xd, Ud, Vd, Sd = (t.to(DEV) for t in (x, U, Vt, S))
    want = bk.blast_torch_layout(xd, Ud, Vd, Sd).reshape(N, O).float()
    ref, _, _ = orc.blast(x, U, Vt, S)
    x2 = xd.reshape(N, I)
    # every decode kernel on the built-in array in turn: the two-launch path (0), the grid-wide kernel (1), the cluster
    # kernel (2); the second call of each finds the leftovers of the call before it
    try:
        for path in (0, 1, 2):
            assert lib.blr_debug_decode_path(path) == 0
            for attempt in range(2):
                rc, got = _call_static(lib, L, x2, Ud, Vd, Sd, b, P, Q, R)
                assert rc == 0, lib.blr_last_error()
                assert lib.blr_blast_static_status(L.stream_ptr(xd.device)) == 0, lib.blr_last_error()
                assert orc.rel_fro(got.float().cpu(), want.cpu()) < TOL, f"path {path} call {attempt}"
                assert orc.rel_fro(got.float().cpu(), ref.reshape(N, O)) < TOL, f"path {path} call {attempt}"
    finally:
        assert lib.blr_debug_decode_path(0) == 0


def test_static_scratch_entry_rejects_oversized_problems():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from mem_efficient_blr_b200 import _lib as L
    lib = L.load()
    N, b, P, Q, R = 16, 16, 64, 64, 4096      # 16 * 16 * 4096 elements of scratch: more than 4 MiB
    x2 = torch.zeros(N, b * P, dtype=torch.float16, device=DEV)
    U = torch.zeros(b, Q, R, dtype=torch.float16, device=DEV)
    Vt = torch.zeros(b, R, P, dtype=torch.float16, device=DEV)
    S = torch.zeros(b, b, R, dtype=torch.float16, device=DEV)
    rc, _ = _call_static(lib, L, x2, U, Vt, S, b, P, Q, R)
    assert rc == -4 and b"built-in array" in lib.blr_last_error()
    x17 = torch.zeros(17, b * P, dtype=torch.float16, device=DEV)
    rc, _ = _call_static(lib, L, x17, U, Vt, S, b, P, Q, R)
    assert rc == -6
