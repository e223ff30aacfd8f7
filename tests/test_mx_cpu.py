"""Block-scaled (MX) e4m3 operands: the PyTorch reference path of the quantiser, the scale-factor tiling and the GEMM."""
import pytest
import torch

from llmq_b200.ops import kernels as K


def _blocky(rows, cols, seed):
    """bf16 matrix whose 32-element blocks (both ways) differ in magnitude by up to 2^12."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    x = x * torch.exp2(torch.randint(-6, 7, (rows, 1), generator=g).float()) * torch.exp2(torch.randint(-6, 7, (1, cols), generator=g).float())
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("tile", [K.MX_TILE_A, K.MX_TILE_B])
def test_scale_offsets_are_a_bijection(tile):
    rows, Kdim = 300, 384
    off = K.mx_sf_offsets(rows, Kdim, tile).reshape(-1)
    assert off.unique().numel() == off.numel()
    assert int(off.max()) < K.mx_sf_bytes(rows, Kdim, tile)


@pytest.mark.parametrize("transpose", [False, True])
def test_quantize_roundtrip(transpose):
    x = _blocky(256, 384, 0)
    q, sf = K.quantize_mx(x, transpose=transpose, operand="b")
    ref = (x.t() if transpose else x).float()
    back = K.dequantize_mx(q, sf, "b")
    # e4m3 has 3 mantissa bits; a block is scaled so its abs-max lands in (224, 448], so the error of an element is at most
    # half a step (2^-4 relative) of the block's top binade
    blk_max = ref.reshape(ref.shape[0], -1, 32).abs().amax(-1, keepdim=True).expand(-1, -1, 32).reshape(ref.shape)
    assert ((back - ref).abs() <= blk_max * 2.0 ** -3 + 1e-30).all()
    assert (back.abs() <= 448 * torch.exp2(torch.ceil(torch.log2(blk_max / 448)))).all()


def test_gemm_matches_fp32_matmul_of_dequantised_operands():
    a, b = _blocky(128, 256, 1), _blocky(224, 256, 2)
    aq, asf = K.quantize_mx(a, operand="a")
    bq, bsf = K.quantize_mx(b, operand="b")
    out = torch.empty(128, 224, dtype=torch.float32)
    K.gemm_mx(out, aq, asf, bq, bsf)
    ref = a.float() @ b.float().t()
    rel = (out - ref).norm() / ref.norm()
    assert rel < 0.05, rel
