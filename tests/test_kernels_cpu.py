"""PyTorch paths of the kernel wrappers that have no model-level CPU coverage: they are what the CPU tests of the model run
and what the GPU kernels are compared with, so they are checked against the formulas directly."""
import pytest
import torch

from llmq_b200.ops import kernels as K

F8 = torch.float8_e4m3fn


def _swiglu_grad(dout, inp):
    D = inp.shape[-1] // 2
    x = inp.float()
    up, gate = x[:, :D], x[:, D:]
    s = torch.sigmoid(gate)
    d = dout.float()
    return torch.cat([d * gate * s, d * up * s * (1 + gate * (1 - s))], -1)


def test_swiglu_backward_two_pass_fallbacks_match_the_separate_kernels():
    torch.manual_seed(0)
    rows, D = 48, 80
    inp = (torch.randn(rows, 2 * D) * 1.5).bfloat16()
    dout = (torch.randn(rows, D) * 0.7).bfloat16()
    want = _swiglu_grad(dout, inp).bfloat16()
    # pass 1: abs-max of the gradient as it would be stored
    am = torch.zeros(1)
    K.swiglu_backward_stats(am, dout, inp)
    assert am.item() == want.float().abs().max().item()
    # ... and, on request, the transposed e4m3 SwiGLU output under a known abs-max
    act = torch.empty(rows, D, dtype=torch.bfloat16)
    act_am = torch.zeros(1)
    K.swiglu_forward(act, inp, absmax=act_am)
    act_t, act_sc = torch.zeros(D, rows, dtype=F8), torch.zeros(1)
    am2 = torch.zeros(1)
    K.swiglu_backward_stats(am2, dout, inp, act_t=act_t, act_absmax=act_am, act_scale=act_sc)
    assert am2.item() == am.item()
    assert act_sc.item() == pytest.approx(act_am.item() / 448.0, rel=1e-6)
    back = act_t.float().t() * act_sc
    assert (back - act.float()).abs().max().item() <= 0.07 * act_am.item()          # e4m3: 3 mantissa bits
    # pass 2: e4m3 rows and their transpose, same bytes as quantising the stored gradient
    q, qt, sc = torch.zeros(rows, 2 * D, dtype=F8), torch.zeros(2 * D, rows, dtype=F8), torch.zeros(1)
    K.swiglu_backward_quant(q, qt, sc, dout, inp, am)
    q_ref, qt_ref, sc_ref = torch.zeros(rows, 2 * D, dtype=F8), torch.zeros(2 * D, rows, dtype=F8), torch.zeros(1)
    K.quantize_transpose(q_ref, qt_ref, sc_ref, want, am)
    assert sc.item() == sc_ref.item() == pytest.approx(am.item() / 448.0, rel=1e-6)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(qt.view(torch.uint8), q.view(torch.uint8).t())


def test_quantize_transpose_fallback_is_quantise_then_transpose():
    torch.manual_seed(1)
    x = torch.randn(32, 48).bfloat16()
    am = x.float().abs().max().reshape(1)
    q, qt, sc = torch.zeros(32, 48, dtype=F8), torch.zeros(48, 32, dtype=F8), torch.zeros(1)
    K.quantize_transpose(q, qt, sc, x, am)
    assert torch.equal(qt.view(torch.uint8), q.view(torch.uint8).t())
    assert (q.float() * sc - x.float()).abs().max().item() <= 0.07 * am.item()
    # 1-byte input: a plain transpose
    qt2 = torch.zeros(48, 32, dtype=F8)
    K.quantize_transpose(None, qt2, None, q, None)
    assert torch.equal(qt2.view(torch.uint8), q.view(torch.uint8).t())
