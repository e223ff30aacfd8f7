"""Peer-memory collectives on 2+ GPUs against NCCL on the same data (skipped with fewer than two devices)."""
import os
import socket
import traceback

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, multimem, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                          LLMQ_P2P_MULTIMEM="1" if multimem else "0")
        os.environ["NCCL_NVLS_ENABLE"] = "0"                 # NCCL is only the comparison here; our kernels own the multicast objects
        import torch.distributed as dist
        from llmq_b200.ops import kernels as K
        from llmq_b200.parallel.comm import TorchDistComm
        from llmq_b200.parallel.fused import FusedCollectives
        dev = torch.device("cuda", rank)
        torch.cuda.set_device(dev)
        comm = TorchDistComm(dev, timeout_s=30)
        fc = FusedCollectives(comm, dev, wait_limit_s=5.0)
        g = torch.Generator(device="cpu").manual_seed(100 + rank)
        rows, cols = 512, 384
        # ---- quantise + all-gather
        shard = (torch.randn(rows // world, cols, generator=g) * 3).bfloat16().to(dev)
        am = torch.zeros(1, device=dev)
        K.abs_max(am, shard)
        fc.all_reduce_small(am, "max")
        ref_am = am.clone()
        dist.all_reduce(ref_am, op=dist.ReduceOp.MAX)
        assert torch.equal(am, ref_am)
        full = fc.heap.empty((rows, cols), torch.float8_e4m3fn)
        scale = torch.zeros(1, device=dev)
        for it in range(3):                                    # generations advance, buffers are reused
            fc.quant_allgather(full, shard, am, scale)
            gen = fc.signal(1)
            fc.wait(1, gen)
            q_local = torch.empty_like(shard, dtype=torch.float8_e4m3fn)
            K.quantize(q_local, None, shard, am)
            ref = torch.empty(rows, cols, dtype=torch.uint8, device=dev)
            dist.all_gather_into_tensor(ref.view(-1), q_local.view(torch.uint8).view(-1))
            torch.cuda.synchronize()
            assert torch.equal(full.view(torch.uint8), ref), f"all-gather mismatch it={it}"
            assert abs(scale.item() - am.item() / 448.0) <= 2e-7 * scale.item()            # fp32 division on the device
            g2 = fc.signal(2)                                   # everybody finished checking before the next overwrite
            fc.wait(2, g2)
            shard.mul_(0.5)
        vec = fc.heap.empty((world * 64,), torch.bfloat16)
        mine = torch.full((64,), float(rank + 1), dtype=torch.bfloat16, device=dev)
        fc.quant_allgather(vec, mine)
        gen = fc.signal(1)
        fc.wait(1, gen)
        torch.cuda.synchronize()
        assert torch.equal(vec.float().view(world, 64)[:, 0].cpu(), torch.arange(1, world + 1).float())
        # ---- reduce-scatter (mean), with accumulation and the fused norm
        grad = fc.heap.empty((rows, cols), torch.bfloat16)
        grad.copy_(torch.randn(rows, cols, generator=g).bfloat16())
        ref_full = grad.clone().float()
        dist.all_reduce(ref_full)
        ref_shard = (ref_full / world)[rank * rows // world:(rank + 1) * rows // world]
        gen = fc.signal(3)
        fc.wait(3, gen)
        dst = torch.zeros(rows // world, cols, dtype=torch.bfloat16, device=dev)
        partials = torch.zeros(K.NORM_PARTIALS, device=dev)
        fc.reduce_scatter(grad, dst, accumulate=False, scale=1.0 / world, norm_partials=partials)
        torch.cuda.synchronize()
        err = (dst.float() - ref_shard).abs().max().item()
        assert err <= 2e-2 * ref_shard.abs().max().item() + 1e-3, err
        assert abs(partials.sum().item() - dst.float().pow(2).sum().item()) < 1e-2 * dst.float().pow(2).sum().item()
        fc.reduce_scatter(grad, dst, accumulate=True, scale=1.0 / world, seed=7)
        torch.cuda.synchronize()
        err = (dst.float() - 2 * ref_shard).abs().max().item()
        assert err <= 3e-2 * ref_shard.abs().max().item() + 1e-2, err
        # ---- GEMM with the reduce-scatter inside: dW = dout^T @ inp per rank, mean over ranks, own rows
        M, N, Kd = 1024, 640, 512
        landing = fc.heap.empty((world, M // world, N), torch.bfloat16)
        shard_dst = torch.zeros(M // world, N, dtype=torch.bfloat16, device=dev)
        partials.zero_()
        assert fc.gemm_rs_supported(M, N)
        for it in range(3):
            a_t = torch.randn(Kd, M, generator=g).bfloat16().to(dev)          # stored [K, M]
            b_t = torch.randn(Kd, N, generator=g).bfloat16().to(dev)          # stored [K, N]
            prev = torch.randn(M, N, generator=g).bfloat16().to(dev) if it == 2 else None
            local = a_t.float().t() @ b_t.float()
            if prev is not None:
                local = local + prev.float()
            tot = local.bfloat16().float()                                    # each rank's contribution is rounded to bf16
            dist.all_reduce(tot)
            want = (tot / world)[rank * M // world:(rank + 1) * M // world]
            before = shard_dst.float().clone()
            fc.gemm_rs(landing, 0, shard_dst, a_t, b_t, a_mn=True, b_mn=True, prev=prev, shard_accumulate=it > 0, shard_scale=1.0 / world,
                       norm_partials=partials if it == 0 else None, seed=11 + it)
            gen = fc.signal(4)                                                # nobody overwrites a landing buffer that is still being summed
            fc.wait(4, gen)
            torch.cuda.synchronize()
            K.check_status(dev)
            expect = want + (before if it > 0 else 0)
            err = (shard_dst.float() - expect).abs().max().item()
            assert err <= 2e-2 * expect.abs().max().item() + 1e-2, (it, err)
            if it == 0:
                ssq = shard_dst.float().pow(2).sum().item()
                assert abs(partials.sum().item() - ssq) < 1e-3 * ssq
        # ---- a wait on a flag nobody sets runs out and is reported, the context stays usable
        fc.wait_limit_s = 0.5
        fc.wait(9, 1)
        torch.cuda.synchronize()
        try:
            K.check_status(dev)
            raise AssertionError("time-out was not reported")
        except Exception as e:
            assert "timed out" in str(e)
        assert torch.ones(4, device=dev).sum().item() == 4
        used_multimem = bool(fc.use_multimem)
        fc.close()                                          # every rank is done with the peers' memory before anything is unmapped
        q.put((rank, "ok", used_multimem))
        comm.shutdown()
    except Exception as e:
        q.put((rank, "error", repr(e) + "\n" + traceback.format_exc()))


@pytest.mark.parametrize("multimem", [False, True], ids=["peer-loads", "multimem"])
def test_fused_collectives_match_nccl(multimem):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, multimem, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = []
    try:
        for _ in range(world):
            res.append(q.get(timeout=100))
    except Exception:                                   # a rank that never answered: report what the others said
        pass
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.kill()
    assert len(res) == world and all(r[1] == "ok" for r in res), res
