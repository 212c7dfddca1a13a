"""The no-allocation skinny GEMM entry point, called through the C ABI (collected last: the file name sorts after
every other test file, so it runs both alone and after the rest of the GPU suite has used the library).

spgt_batched_skinny_gemm_noalloc keeps its scratch (the partial tiles of the split k range and the tickets that count
them) in a fixed array inside the library instead of a caller-provided workspace.  It launches the same kernels on the
same plan as spgt_batched_skinny_gemm, so the results must be bit-identical, on the first call (which also does the
per-device set-up) and on a second call that finds the array dirty from the first one.
"""
import ctypes as C

import pytest
import torch

from oracle import gt_oracle as O
from tests.helpers import rel_l2

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _with_workspace(lib, A, Bm, alpha):
    batch, M, K = A.shape
    N = Bm.shape[2]
    need = lib.spgt_skinny_gemm_workspace_bytes(M, N, K, batch)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=A.device)
    out = torch.full((batch, M, N), float('nan'), device=A.device)
    rc = lib.spgt_batched_skinny_gemm(_ptr(A), _ptr(Bm), _ptr(out), C.c_float(alpha), M, N, K, batch, _ptr(ws), need, _stream())
    assert rc == 0, lib.spgt_error_string(rc)
    return out, need


def _no_alloc(lib, A, Bm, alpha):
    batch, M, K = A.shape
    N = Bm.shape[2]
    out = torch.full((batch, M, N), float('nan'), device=A.device)
    rc = lib.spgt_batched_skinny_gemm_noalloc(_ptr(A), _ptr(Bm), _ptr(out), C.c_float(alpha), M, N, K, batch, _stream())
    assert rc == 0, lib.spgt_error_string(rc)
    return out


def test_no_alloc_matches_workspace_entry_point_twice_in_a_row():
    from spgt_b200._lib import lib
    dev = torch.device('cuda:0')
    torch.cuda.set_device(dev)
    assert lib.spgt_skinny_gemm_noalloc_max_bytes() == 8 << 20
    g = torch.Generator().manual_seed(20)
    # second problem is smaller and differently shaped, so it reads a scratch array left dirty by the first
    # (one-launch kernel, then the two-pass kernels: N = 34 is not a multiple of 4, then the one-launch kernel on the dirty array)
    for call, (batch, M, N, K) in enumerate([(64, 32, 32, 1849), (3, 40, 34, 5000), (5, 40, 36, 7001)]):
        A = torch.randn(batch, M, K, generator=g).to(dev)
        Bm = torch.randn(batch, K, N, generator=g).to(dev)
        alpha = 1.0 / K
        want, need = _with_workspace(lib, A, Bm, alpha)
        assert 0 < need <= lib.spgt_skinny_gemm_noalloc_max_bytes()
        got = _no_alloc(lib, A, Bm, alpha)
        torch.cuda.synchronize()
        assert torch.equal(got, want), (call, rel_l2(got, want))
        again = _no_alloc(lib, A, Bm, alpha)
        torch.cuda.synchronize()
        assert torch.equal(again, want), call
        ref = O.batched_skinny_gemm(A.cpu().double(), Bm.cpu().double(), alpha)
        assert rel_l2(got, ref) < 5e-5


def test_no_alloc_rejects_what_does_not_fit_and_bad_arguments():
    from spgt_b200._lib import lib
    dev = torch.device('cuda:0')
    torch.cuda.set_device(dev)
    batch, M, N, K = 4096, 64, 66, 64          # two-pass kernels (N % 4 != 0): 6 tiles x 4096 batches x 4 KiB = 96 MiB of partial tiles
    assert lib.spgt_skinny_gemm_workspace_bytes(M, N, K, batch) > lib.spgt_skinny_gemm_noalloc_max_bytes()
    A = torch.zeros(batch, M, K, device=dev)
    Bm = torch.zeros(batch, K, N, device=dev)
    out = torch.full((batch, M, N), 7.0, device=dev)
    rc = lib.spgt_batched_skinny_gemm_noalloc(_ptr(A), _ptr(Bm), _ptr(out), C.c_float(1.0), M, N, K, batch, _stream())
    assert rc == -6
    assert b'no-allocation' in lib.spgt_error_string(rc)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())            # nothing was launched
    assert lib.spgt_batched_skinny_gemm_noalloc(None, _ptr(Bm), _ptr(out), C.c_float(1.0), M, N, K, batch, _stream()) == -1
    assert lib.spgt_batched_skinny_gemm_noalloc(_ptr(A), _ptr(Bm), _ptr(out), C.c_float(1.0), 0, N, K, batch, _stream()) == -2
