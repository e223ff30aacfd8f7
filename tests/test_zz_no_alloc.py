"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some users of the library run where device memory cannot be allocated (inside another framework's stream
callback, in a real-time loop, under a host that owns the whole memory pool), so they cannot supply the
workspace the regular entry point needs.  ``llmq_rmsnorm_backward_noalloc`` keeps that workspace inside the
library.  This test checks that it gives the same answer as the regular entry point, twice in a row (the
second call finds the first call's leftovers in the shared workspace), and that it refuses sizes beyond its
documented maximum.  The file name sorts last so that a failure here cannot hide other tests under ``-x``.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, dinp, dw, dout, x, w, rstd, absmax, accumulate, dtype=0):
    rows, C = x.shape
    fn = lib.llmq_rmsnorm_backward_noalloc
    fn.restype = ctypes.c_int
    return fn(ctypes.c_void_p(dinp.data_ptr()), ctypes.c_void_p(dw.data_ptr()), ctypes.c_void_p(dout.data_ptr()),
              ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(rstd.data_ptr()),
              ctypes.c_int(rows), ctypes.c_int(C), ctypes.c_int(dtype), ctypes.c_void_p(absmax.data_ptr()),
              ctypes.c_int(int(accumulate)), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("C", [896, 3584])
def test_noalloc_matches_regular_entry_point_twice(C):
    from llmq_b200.ops import kernels as K
    from llmq_b200.ops import lib as L

    lib = L.kernels()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    for call in range(2):                       # second call reuses the workspace the first one left behind
        rows = 777 + 64 * call
        x = torch.randn(rows, C, device=dev).bfloat16()
        dy = torch.randn(rows, C, device=dev).bfloat16()
        w = (1 + 0.1 * torch.randn(C, device=dev)).bfloat16()
        dres = torch.randn(rows, C, device=dev).bfloat16()
        dw0 = torch.randn(C, device=dev).bfloat16()
        rstd = torch.zeros(rows, device=dev)
        K.rmsnorm_forward(None, rstd, x, w, 1e-6)
        # regular entry point (caller-provided scratch)
        dinp_a, dw_a, am_a = dres.clone(), dw0.clone(), torch.zeros(1, device=dev)
        scratch = torch.zeros(K.rmsnorm_backward_scratch_elems(C, dev), device=dev)
        K.rmsnorm_backward(dinp_a, dw_a, scratch, dy, x, w, rstd, absmax=am_a, accumulate_dweight=True)
        # allocation-free entry point
        dinp_b, dw_b, am_b = dres.clone(), dw0.clone(), torch.zeros(1, device=dev)
        rc = _call_noalloc(lib, dinp_b, dw_b, dy, x, w, rstd, am_b, True)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert torch.equal(dinp_a, dinp_b)      # the input gradient does not depend on the workspace at all
        assert am_a.item() == am_b.item()
        err = (dw_a.float() - dw_b.float()).abs().max().item()
        assert err <= 2e-2 + 2e-2 * dw_a.float().abs().max().item(), err


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_noalloc_at_the_documented_maximum_row_length(dt):
    """C = 8192 is the longest row the built-in workspace serves: bf16 (4 values per thread in registers) and fp32
    (dtype code 3, where the partial rows fill the workspace exactly), each against the regular entry point."""
    from llmq_b200.ops import kernels as K
    from llmq_b200.ops import lib as L

    lib = L.kernels()
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    rows, C = 301, 8192
    x = torch.randn(rows, C, device=dev).to(dt)
    dy = torch.randn(rows, C, device=dev).to(dt)
    w = (1 + 0.1 * torch.randn(C, device=dev)).to(dt)
    dres = torch.randn(rows, C, device=dev).to(dt)
    dw0 = torch.randn(C, device=dev).to(dt)
    rstd = torch.zeros(rows, device=dev)
    K.rmsnorm_forward(None, rstd, x, w, 1e-6)
    dinp_a, dw_a, am_a = dres.clone(), dw0.clone(), torch.zeros(1, device=dev)
    scratch = torch.zeros(K.rmsnorm_backward_scratch_elems(C, dev), device=dev)
    K.rmsnorm_backward(dinp_a, dw_a, scratch, dy, x, w, rstd, absmax=am_a, accumulate_dweight=True)
    for _ in range(2):
        dinp_b, dw_b, am_b = dres.clone(), dw0.clone(), torch.zeros(1, device=dev)
        rc = _call_noalloc(lib, dinp_b, dw_b, dy, x, w, rstd, am_b, True, dtype=0 if dt == torch.bfloat16 else 3)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert torch.equal(dinp_a, dinp_b) and am_a.item() == am_b.item()
        err = (dw_a.float() - dw_b.float()).abs().max().item()
        assert err <= 2e-2 + 2e-2 * dw_a.float().abs().max().item(), err


def test_noalloc_refuses_fp32_rows_that_are_not_a_multiple_of_four():
    """fp32 rows are read as 16-byte vectors: a row length like 1002 is refused before anything is launched, like the
    regular entry point refuses it."""
    from llmq_b200.ops import lib as L

    lib = L.kernels()
    dev = torch.device("cuda", 0)
    C = 1002
    x = torch.ones(4, C, device=dev)
    w = torch.ones(C, device=dev)
    rstd = torch.ones(4, device=dev)
    am = torch.zeros(1, device=dev)
    dinp = torch.full((4, C), 3.0, device=dev)
    rc = _call_noalloc(lib, dinp, w.clone(), x.clone(), x, w, rstd, am, False, dtype=3)
    torch.cuda.synchronize()
    assert rc != 0
    assert (dinp == 3.0).all()


def test_noalloc_rejects_oversized_rows():
    from llmq_b200.ops import lib as L

    lib = L.kernels()
    dev = torch.device("cuda", 0)
    C = 8192 + 8
    x = torch.zeros(4, C, device=dev, dtype=torch.bfloat16)
    w = torch.ones(C, device=dev, dtype=torch.bfloat16)
    rstd = torch.ones(4, device=dev)
    am = torch.zeros(1, device=dev)
    before = x.clone()
    rc = _call_noalloc(lib, x, w.clone(), x.clone(), x.clone(), w, rstd, am, False)
    torch.cuda.synchronize()
    assert rc == -20
    assert torch.equal(x, before)
