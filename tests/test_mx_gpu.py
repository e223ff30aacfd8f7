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
