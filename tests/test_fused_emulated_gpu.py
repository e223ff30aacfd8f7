"""The kernels that carry a collective, on ONE GPU: rank 0 of an emulated group runs, the peer tables point at local
buffers and the peers' arrivals are booked before the launch, so every code path of the kernel executes (peer stores,
counter bumps, the summing tail, the producer's flag polls) without a second device.  The multi-GPU versions of these
checks live in test_y_multi_gpu_collectives.py and need two or more GPUs."""
import ctypes

import pytest
import torch

from llmq_b200.ops import kernels as K
from llmq_b200.ops import lib as L

pytestmark = pytest.mark.gpu


def _arr(ptrs):
    return (ctypes.c_void_p * 8)(*(list(ptrs) + [0] * (8 - len(ptrs))))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float8_e4m3fn])
@pytest.mark.parametrize("world", [2, 4])
def test_gemm_reduce_scatter_one_gpu(dtype, world):
    dev = torch.device("cuda", 0)
    st, k = K._dev_state(dev), L.kernels()
    M, N, Kd = 1024, 640, 768
    g = torch.Generator(device="cuda").manual_seed(world)
    At = (torch.randn(Kd, M, device=dev, generator=g) * 0.5).to(dtype)            # both operands MN-major, as in dW = dY^T X
    Bt = (torch.randn(Kd, N, device=dev, generator=g) * 0.5).to(dtype)
    ref = At.float().t() @ Bt.float()
    rows = M // world
    landing = [(torch.randn(world, rows, N, device=dev, generator=g)).to(torch.bfloat16) for _ in range(world)]
    before = [t.clone() for t in landing]
    counters = torch.zeros(world, 64, dtype=torch.int32, device=dev)
    shard = torch.zeros(rows, N, dtype=torch.bfloat16, device=dev)
    parts = torch.zeros(K.NORM_PARTIALS, device=dev)
    arrivals = int(k.llmq_gemm_rs_arrivals(M, N, world))
    assert arrivals % world == 0
    counters[0, 0] = arrivals - arrivals // world                                     # the peers "delivered" already
    ones = torch.ones(1, device=dev)
    rc = k.llmq_gemm_rs(L.ptr(At), L.ptr(Bt), L.ptr(landing[0]), M, N, Kd, L.dtype_code(dtype), L.dtype_code(dtype), 1, 1,
                        ctypes.c_longlong(M), ctypes.c_longlong(N), 0, L.ptr(ones), L.ptr(ones), ctypes.c_float(1.0), L.ptr(st["status"]),
                        st["sms"], _arr([t.data_ptr() for t in landing]), _arr([counters[i].data_ptr() for i in range(world)]), 0, world,
                        ctypes.c_uint(arrivals), L.ptr(shard), 0, ctypes.c_float(1.0 / world), L.ptr(parts), K.NORM_PARTIALS,
                        ctypes.c_uint(11), ctypes.c_double(2.0), L.stream_ptr())
    L.check(rc, "gemm_rs")
    torch.cuda.synchronize()
    K.check_status(dev)
    tol = 2e-2 * ref.abs().max().item()
    for owner in range(world):
        # slot 0 (= the running rank) of every owner's landing buffer holds that owner's rows of the product
        got = landing[owner][0].float()
        assert (got - ref[owner * rows:(owner + 1) * rows]).abs().max().item() <= tol, owner
        for s in range(1, world):
            assert torch.equal(landing[owner][s], before[owner][s])                 # other ranks' slots are untouched
        assert int(counters[owner, 0]) == (arrivals if owner == 0 else arrivals // world)
    want = (landing[0].float().sum(0)) / world
    assert (shard.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    assert abs(parts.sum().item() - (shard.float() ** 2).sum().item()) <= 2e-2 * (shard.float() ** 2).sum().item()


def test_gemm_polls_arrival_flags_one_gpu():
    dev = torch.device("cuda", 0)
    M, N, Kd, world = 512, 1024, 512, 4
    g = torch.Generator(device="cuda").manual_seed(5)
    X = torch.randn(M, Kd, device=dev, generator=g).to(torch.bfloat16)
    W = torch.randn(N, Kd, device=dev, generator=g).to(torch.bfloat16)
    plain, polled = torch.empty(M, N, dtype=torch.bfloat16, device=dev), torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    K.gemm(plain, X, W)
    flags = torch.full((8,), 9, dtype=torch.int32, device=dev)                        # every source arrived at generation 9
    K.gemm(polled, X, W, ready=(flags.data_ptr(), 9, N // world, 2.0))
    torch.cuda.synchronize()
    K.check_status(dev)
    tol = 4e-3 * plain.float().abs().max().item()           # the two calls may take different tile shapes
    assert (plain.float() - polled.float()).abs().max().item() <= tol


def test_wait_on_a_flag_nobody_sets_runs_out():
    """The bounded device-side wait: the limit passes, the kernel reports it in the status word and returns; the
    context stays usable."""
    dev = torch.device("cuda", 0)
    st = K._dev_state(dev)
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    flags[:3] = 1                                                                     # "rank" 3 never signals generation 1
    L.check(L.kernels().llmq_p2p_wait(L.ptr(flags), 4, ctypes.c_uint(1), L.ptr(st["status"]), ctypes.c_double(0.2), L.stream_ptr()), "p2p_wait")
    torch.cuda.synchronize()
    with pytest.raises(L.KernelError):
        K.check_status(dev)
    flags[3] = 1
    L.check(L.kernels().llmq_p2p_wait(L.ptr(flags), 4, ctypes.c_uint(1), L.ptr(st["status"]), ctypes.c_double(0.2), L.stream_ptr()), "p2p_wait")
    torch.cuda.synchronize()
    K.check_status(dev)
    assert torch.ones(4, device=dev).sum().item() == 4


@pytest.mark.parametrize("world", [2, 8])
def test_quant_allgather_and_reduce_scatter_one_gpu(world):
    dev = torch.device("cuda", 0)
    k = L.kernels()
    sms = K.num_sms(dev)
    g = torch.Generator(device="cuda").manual_seed(world)
    n_shard = 256 * 1024
    shard = torch.randn(n_shard, device=dev, generator=g).to(torch.bfloat16)
    gathers = [torch.zeros(n_shard * world, dtype=torch.float8_e4m3fn, device=dev) for _ in range(world)]
    am = shard.float().abs().max().reshape(1)
    sc = torch.zeros(1, device=dev)
    L.check(k.llmq_p2p_quant_allgather(_arr([t.data_ptr() for t in gathers]), ctypes.c_longlong(0), L.ptr(shard), ctypes.c_longlong(n_shard), 0,
                                       world, L.ptr(am), L.ptr(sc), 1, sms, L.stream_ptr()), "p2p_quant_allgather")
    torch.cuda.synchronize()
    q = torch.empty(n_shard, dtype=torch.float8_e4m3fn, device=dev)
    sc2 = torch.zeros(1, device=dev)
    K.quantize(q, sc2, shard, am)
    assert torch.equal(sc, sc2)
    for t in gathers:                                                                  # every "rank" received rank 0's slice
        assert torch.equal(t[:n_shard].view(torch.uint8), q.view(torch.uint8))
        assert int(t[n_shard:].view(torch.uint8).max()) == 0
    grads = [torch.randn(n_shard * world, device=dev, generator=g).to(torch.bfloat16) for _ in range(world)]
    dst = torch.zeros(n_shard, dtype=torch.bfloat16, device=dev)
    parts = torch.zeros(K.NORM_PARTIALS, device=dev)
    L.check(k.llmq_p2p_reduce_scatter(_arr([t.data_ptr() for t in grads]), None, ctypes.c_longlong(0), ctypes.c_longlong(n_shard), 0, world,
                                      L.ptr(dst), 0, ctypes.c_float(1.0 / world), L.ptr(parts), K.NORM_PARTIALS, ctypes.c_uint(3), sms,
                                      L.stream_ptr()), "p2p_reduce_scatter")
    torch.cuda.synchronize()
    K.check_status(dev)
    want = sum(t[:n_shard].float() for t in grads) / world
    assert (dst.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item()
    assert abs(parts.sum().item() - (dst.float() ** 2).sum().item()) <= 1e-2 * (dst.float() ** 2).sum().item()
