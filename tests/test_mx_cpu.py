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


def _tiny_model(block_scaled, device="cpu", heads=(4, 2), hidden=128, ffn=256, B=2, T=64):
    from llmq_b200.config import create_config_from_name
    from llmq_b200.models.llama import LlamaModel
    from llmq_b200.options import LLamaOptions
    cfg = create_config_from_name("tiny-qwen2", torch.bfloat16).replace(hidden_size=hidden, intermediate_size=ffn, num_attention_heads=heads[0],
                                                                        num_key_value_heads=heads[1])
    m = LlamaModel(cfg, LLamaOptions(matmul_type="mxe4m3" if block_scaled else None), device=device, batch_size=B, seq_len=T)
    m.init_weights(0)
    return m


def _grad_cosines(ma, mb):
    ga, gb = ma.get_gradients(), mb.get_gradients()
    cos = []
    for n in ga:
        a, b = ga[n].flatten().float().cpu(), gb[n].flatten().float().cpu()
        if a.norm() > 0:
            cos.append(float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-12)))
    return cos


def test_block_scaled_training_step_tracks_bf16():
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, 512, (2, 65), generator=g, dtype=torch.int32)
    x, y = toks[:, :-1].contiguous(), toks[:, 1:].contiguous()
    res = []
    models = [_tiny_model(False), _tiny_model(True)]
    assert models[1].mx and not models[1].quant
    for m in models:
        m.forward(x)
        m.backward(x, y, 0.0, 1, 0)
        res.append(m.update(lr=0.0, step=1))
    assert abs(res[0]["loss"] - res[1]["loss"]) < 2e-2
    cos = _grad_cosines(*models)
    assert min(cos) > 0.95 and sum(cos) / len(cos) > 0.99, cos


def test_block_scaled_rejects_unaligned_shapes():
    with pytest.raises(ValueError, match="multiples of 128"):
        _tiny_model(True, hidden=64, ffn=172)
