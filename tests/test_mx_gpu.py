"""Block-scaled (MX) e4m3 on the GPU: the quantiser kernels bit for bit against the PyTorch implementation, and the
tcgen05 block-scaled GEMM against an fp32 matmul of the dequantised operands."""
import pytest
import torch

from llmq_b200.ops import kernels as K

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _blocky(rows, cols, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    x = x * torch.exp2(torch.randint(-6, 7, (rows, 1), generator=g).float()) * torch.exp2(torch.randint(-6, 7, (1, cols), generator=g).float())
    return x.to(torch.bfloat16)


@pytest.fixture(autouse=True)
def _check_status():
    yield
    torch.cuda.synchronize()
    K.check_status(torch.device(DEV, 0))


@pytest.mark.parametrize("R,C", [(128, 128), (384, 200 * 8), (1000, 512)])
@pytest.mark.parametrize("transpose", [False, True])
@pytest.mark.parametrize("operand", ["a", "b"])
def test_quantize_mx_matches_reference(R, C, transpose, operand):
    if (R if transpose else C) % 128:
        pytest.skip("contraction length must be a multiple of 128")
    x = _blocky(R, C, 3)
    q_ref, sf_ref = K.quantize_mx(x, transpose=transpose, operand=operand)
    q, sf = K.quantize_mx(x.to(DEV), transpose=transpose, operand=operand)
    assert torch.equal(sf.cpu(), sf_ref)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))


@pytest.mark.parametrize("M,N,Kd", [(128, 224, 128), (256, 448, 512), (200, 300, 384), (1024, 3584, 1024)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_mx(M, N, Kd, out_dtype):
    a, b = _blocky(M, Kd, 4), _blocky(N, Kd, 5)
    aq, asf = K.quantize_mx(a.to(DEV), operand="a")
    bq, bsf = K.quantize_mx(b.to(DEV), operand="b")
    ref = K.dequantize_mx(aq.cpu(), asf.cpu(), "a") @ K.dequantize_mx(bq.cpu(), bsf.cpu(), "b").t()
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    K.gemm_mx(out, aq, asf, bq, bsf)
    err = (out.float().cpu() - ref).abs().max().item()
    tol = (1e-4 if out_dtype == torch.float32 else 1e-2) * ref.abs().max().item()
    assert err <= tol, (err, tol)


def test_gemm_mx_bias_accumulate_absmax():
    M, N, Kd = 256, 448, 256
    a, b = _blocky(M, Kd, 6), _blocky(N, Kd, 7)
    aq, asf = K.quantize_mx(a.to(DEV), operand="a")
    bq, bsf = K.quantize_mx(b.to(DEV), operand="b")
    bias = torch.randn(N).to(torch.bfloat16)
    prev = torch.randn(M, N)
    ref = K.dequantize_mx(aq.cpu(), asf.cpu(), "a") @ K.dequantize_mx(bq.cpu(), bsf.cpu(), "b").t() + bias.float() + prev
    out = prev.to(DEV)
    am = torch.zeros(1, device=DEV)
    K.gemm_mx(out, aq, asf, bq, bsf, bias=bias.to(DEV), accumulate=True, absmax=am)
    assert (out.cpu() - ref).abs().max().item() <= 1e-4 * ref.abs().max().item()
    assert abs(am.item() - out.abs().max().item()) <= 1e-6 * am.item()


def test_block_scaled_model_step_matches_cpu_path():
    """One training step of a small block-scaled model: the CUDA kernels against the PyTorch implementation of the same recipe."""
    from test_mx_cpu import _grad_cosines, _tiny_model
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, 512, (2, 129), generator=g, dtype=torch.int32)
    x, y = toks[:, :-1].contiguous(), toks[:, 1:].contiguous()
    kw = dict(heads=(4, 2), hidden=256, ffn=512, B=2, T=128)
    models = [_tiny_model(True, "cpu", **kw), _tiny_model(True, DEV, **kw)]
    # the normal-init streams of the two devices differ: give both models the same weights
    for (n0, w0, _, _), (n1, w1, _, _) in zip(models[0].weights.master_items(), models[1].weights.master_items()):
        assert n0 == n1
        w0.copy_(w1.cpu())
    models[0].on_weights_changed()
    res = []
    for m in models:
        m.forward(x)
        m.backward(x, y, 0.0, 1, 0)
        res.append(m.update(lr=0.0, step=1))
    assert abs(res[0]["loss"] - res[1]["loss"]) < 4e-2, res         # bf16 activations: attention / norms round differently on the two paths
    cos = _grad_cosines(*models)
    assert min(cos) > 0.97 and sum(cos) / len(cos) > 0.99, cos


def test_quantize_mx_both_equals_the_two_single_passes():
    x = _blocky(384, 256, 9).to(DEV)
    qr, sr, qc, sc = K.quantize_mx_both(x, row_operand="a", col_operand="b")
    qr1, sr1 = K.quantize_mx(x, operand="a")
    qc1, sc1 = K.quantize_mx(x, transpose=True, operand="b")
    assert torch.equal(qr.view(torch.uint8), qr1.view(torch.uint8)) and torch.equal(sr, sr1)
    assert torch.equal(qc.view(torch.uint8), qc1.view(torch.uint8)) and torch.equal(sc, sc1)
