"""End-to-end steps on the GPU: bf16 and e4m3 runs against the fp32 autograd oracle, recompute equality."""
import pytest
import torch

from llmq_b200.config import TransformerConfig
from llmq_b200.models.llama import LlamaModel
from llmq_b200.models.reference import loss_ref
from llmq_b200.ops import kernels as K
from llmq_b200.options import LLamaOptions

pytestmark = pytest.mark.gpu
B, T = 2, 256


def cfg_small(tied=True, hs=64):
    return TransformerConfig("qwen2", 0, 0, None, 4 * hs, 512, 1024, 4, 2, 2, 2048, 1e6, 1e-6, tied, True, torch.bfloat16)


def data(n=1, seed=0):
    g = torch.Generator().manual_seed(seed)
    t = torch.randint(0, 1024, (n, B, T + 1), generator=g, dtype=torch.int32)
    return t[:, :, :-1].contiguous(), t[:, :, 1:].contiguous()


def run(opts, tied=True, hs=64, steps=2, ga=2, lr=1e-3):
    cfg = cfg_small(tied, hs)
    m = LlamaModel(cfg, opts, device="cuda:0", batch_size=B, seq_len=T)
    m.init_weights(0)
    x, y = data(ga, 1)
    out = []
    for s in range(1, steps + 1):
        for j in range(ga):
            m.forward(x[j], j)
            m.backward(x[j], y[j], 0.0, ga, j)
        if s == 1:
            grads = {n: g.float().cpu().clone() for n, g in m.get_gradients().items()}
        r = m.update(lr=lr, step=s, grad_accum=ga)
        out.append((r["loss"], r["norm"]))
    torch.cuda.synchronize()
    K.check_status(torch.device("cuda:0"))
    return cfg, m, out, grads


@pytest.mark.parametrize("mm,hs,tied,gdt", [(None, 64, True, None), ("e4m3", 64, True, None), ("e4m3", 128, False, None), (None, 128, False, None),
                                            ("e4m3", 64, True, "e5m2"), ("e4m3", 128, False, "e5m2")])
def test_step_matches_oracle(mm, hs, tied, gdt):
    """bf16, e4m3 and e4m3 with e5m2 activation gradients (--matmul-dtype e4m3 --gradient-dtype e5m2, the reference's third
    pinned configuration) against the fp32 autograd model."""
    opts = LLamaOptions(matmul_type=mm, gradient_type=gdt)
    cfg = cfg_small(tied, hs)
    m = LlamaModel(cfg, opts, device="cuda:0", batch_size=B, seq_len=T)
    m.init_weights(0)
    ref_p = {n: t.detach().float().cpu().clone().requires_grad_(True) for n, t, _, _ in m.weights.master_items()}
    x, y = data(1, 1)
    loss, ce = loss_ref(cfg, ref_p, x[0], y[0])
    loss.backward()
    m.forward(x[0])
    m.backward(x[0], y[0], 0.0, 1, 0)
    got = m.get_gradients()
    r = m.update(lr=0.0, step=1)
    K.check_status(torch.device("cuda:0"))
    assert abs(r["loss"] - ce.item()) < (3e-2 if mm else 2e-2), (r, ce.item())
    cos, rel = [], []
    for n, g in got.items():
        a, b = g.float().cpu().flatten(), ref_p[n].grad.flatten()
        if b.norm() > 0:
            cos.append((torch.dot(a, b) / (a.norm() * b.norm() + 1e-12)).item())
            rel.append(((a.norm() - b.norm()).abs() / b.norm()).item())
    assert min(cos) > (0.9 if mm else 0.97), (min(cos), cos)
    assert sum(cos) / len(cos) > (0.97 if mm else 0.99)
    assert sum(rel) / len(rel) < 0.05


@pytest.mark.parametrize("mm", [None, "bf16"])
def test_fp32_model_matches_oracle(mm):
    """--model-dtype fp32 on the GPU: tf32 tensor-core GEMMs on fp32 operands (or bf16 GEMM operands with ``matmul_type=bf16``,
    the mixed-precision variant), bf16 copies inside attention, everything else in fp32."""
    cfg = cfg_small(True, 64).replace(dtype=torch.float32)
    m = LlamaModel(cfg, LLamaOptions(matmul_type=mm), device="cuda:0", batch_size=B, seq_len=T)
    assert m.dtype == torch.float32 and m.quant == (mm == "bf16")
    m.init_weights(0)
    ref_p = {n: t.detach().float().cpu().clone().requires_grad_(True) for n, t, _, _ in m.weights.master_items()}
    x, y = data(1, 1)
    loss, ce = loss_ref(cfg, ref_p, x[0], y[0])
    loss.backward()
    m.forward(x[0])
    m.backward(x[0], y[0], 0.0, 1, 0)
    got = m.get_gradients()
    r = m.update(lr=0.0, step=1)
    K.check_status(torch.device("cuda:0"))
    assert abs(r["loss"] - ce.item()) < 5e-3, (r, ce.item())
    cos = []
    for n, g in got.items():
        assert g.dtype == torch.float32
        a, b = g.float().cpu().flatten(), ref_p[n].grad.flatten()
        if b.norm() > 0:
            cos.append((torch.dot(a, b) / (a.norm() * b.norm() + 1e-12)).item())
    assert min(cos) > 0.99 and sum(cos) / len(cos) > 0.999, cos
    # and it trains
    first = r["loss"]
    for s in range(2, 5):
        m.forward(x[0])
        m.backward(x[0], y[0], 0.0, 1, 0)
        r = m.update(lr=1e-3, step=s)
    assert r["loss"] < first


@pytest.mark.parametrize("mm", [None, "e4m3"])
@pytest.mark.parametrize("kw", [dict(recompute_swiglu=True), dict(recompute_block=True), dict(recompute_att=True, recompute_ffn=True),
                                dict(recompute_rms_norm=True, recompute_qkv=True), dict(shard_weights=True, shard_gradients=True),
                                dict(offload_master=True, offload_opt_m=True, offload_opt_v=True),
                                dict(offload_master=True, offload_opt_m=True, offload_opt_v=True, use_zero_copy=True),
                                dict(offload_master=True, offload_opt_m=True, offload_opt_v=True, use_write_combined=True),
                                dict(offload_residual=True, recompute_block=True),
                                dict(shard_weights=True, persistent_quants=True, offload_quants=True, offload_master=True)],
                         ids=lambda d: "+".join(d))
def test_variants_bit_identical_on_gpu(kw, mm):
    base = run(LLamaOptions(matmul_type=mm))[2]
    var = run(LLamaOptions(matmul_type=mm, **kw))[2]
    if kw.get("shard_gradients"):
        # sharded gradients accumulate micro-steps in fp32 with stochastic rounding instead of the GEMM's
        # bf16 read-modify-write, so the runs agree to rounding only
        for (l0, n0), (l1, n1) in zip(base, var):
            assert abs(l0 - l1) < 2e-3 and abs(n0 - n1) < 2e-3 * max(1.0, n0)
        return
    assert base == var


def test_loss_goes_down_fp8():
    _, _, out, _ = run(LLamaOptions(matmul_type="e4m3", momentum_type="bf16", variance_type="bf16"), steps=8, ga=1, lr=3e-3)
    assert out[-1][0] < out[0][0] - 0.3, out


@pytest.mark.parametrize("mm", [None, "e4m3"])
def test_cuda_graphs_reproduce_eager_steps(mm):
    """Per-block CUDA graphs (captured on the second step, replayed afterwards) give the same steps as plain launches."""
    from llmq_b200.ops import lib as L
    base = run(LLamaOptions(matmul_type=mm), steps=4, ga=2)[2]
    n0 = L.launch_count
    cfg, m, out, _ = run(LLamaOptions(matmul_type=mm, use_cuda_graphs=True), steps=4, ga=2)
    assert m.graphs is not None and len(m.graphs.graphs) >= 2 * cfg.num_hidden_layers     # fwd + bwd of every layer
    assert out == base, (out, base)
    # replays are still counted as kernel launches
    n1 = L.launch_count
    run(LLamaOptions(matmul_type=mm), steps=4, ga=2)
    assert n1 - n0 == L.launch_count - n1


def test_time_breakdown_reports_phases():
    opts = LLamaOptions(matmul_type="e4m3", trigger_timing_events=True)
    m = LlamaModel(cfg_small(), opts, device="cuda:0", batch_size=B, seq_len=T)
    m.init_weights(0)
    x, y = data(2, 1)
    for j in range(2):
        m.forward(x[j], j)
        m.backward(x[j], y[j], 0.0, 2, j)
    r = m.update(lr=1e-3, step=1, grad_accum=2)
    tb = r["time_breakdown"]
    assert set(tb) == {"forward", "lm-head", "backward", "optimizer"} and all(v > 0 for v in tb.values()), tb
    am = m.abs_maxes()
    assert len(am) == 2 and max(am["layer0"]) > 0


@pytest.mark.parametrize("mm", [None, "e4m3"])
def test_swiglu_in_gemm_epilogues_is_bit_identical(mm):
    """SwiGLU forward / backward inside the GEMM epilogues round exactly like the separate kernels."""
    base = run(LLamaOptions(matmul_type=mm, fuse_swiglu=0), steps=3, ga=2)
    fused = run(LLamaOptions(matmul_type=mm, fuse_swiglu=3), steps=3, ga=2)
    assert fused[1]._fuse_swiglu and not base[1]._fuse_swiglu
    assert fused[2] == base[2], (fused[2], base[2])
    for n in base[3]:
        assert torch.equal(base[3][n], fused[3][n]), n


@pytest.mark.parametrize("kw", [dict(), dict(recompute_swiglu=True), dict(recompute_block=True), dict(overlap_dw=True)], ids=lambda d: "+".join(d) or "plain")
def test_swiglu_backward_two_pass_is_bit_identical(kw):
    """The SwiGLU gradient as abs-max pass + quantising pass (its bf16 form never stored, the first pass doubling as the
    SwiGLU recompute) gives the bytes of the separate kernels: same losses, norms and gradients."""
    base = run(LLamaOptions(matmul_type="e4m3", swiglu_backward_two_pass=False, **kw), steps=3, ga=2)
    two = run(LLamaOptions(matmul_type="e4m3", swiglu_backward_two_pass=True, **kw), steps=3, ga=2)
    assert two[1]._kmajor and two[1].opts.swiglu_backward_two_pass
    assert two[2] == base[2], (two[2], base[2])
    for n in base[3]:
        assert torch.equal(base[3][n], two[3][n]), n


def test_lmhead_transposed_operands_match():
    base = run(LLamaOptions(matmul_type="e4m3", lmhead_transposed_operands=False), steps=3, ga=2)
    tr = run(LLamaOptions(matmul_type="e4m3", lmhead_transposed_operands=True), steps=3, ga=2)
    for (l0, n0), (l1, n1) in zip(base[2], tr[2]):
        assert abs(l0 - l1) < 2e-3 and abs(n0 - n1) < 2e-2 * max(1.0, n0)


@pytest.mark.parametrize("mm", [None, "e4m3"])
@pytest.mark.parametrize("graphs", [False, True])
def test_dw_side_stream_is_bit_identical(mm, graphs):
    """Weight-gradient GEMMs on the second stream (with and without CUDA graphs) change nothing but the schedule."""
    base = run(LLamaOptions(matmul_type=mm, overlap_dw=False), steps=4, ga=2)
    side = run(LLamaOptions(matmul_type=mm, overlap_dw=True, use_cuda_graphs=graphs), steps=4, ga=2)
    assert side[1]._dw_stream is not None and base[1]._dw_stream is None
    assert side[2] == base[2], (side[2], base[2])
    for n in base[3]:
        assert torch.equal(base[3][n], side[3][n]), n
