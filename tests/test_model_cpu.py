"""The hand-scheduled model on CPU (fp32) against the autograd oracle: tiny Qwen2 config, one
forward/backward with gradient accumulation, one AdamW step, recompute variants, fp8 plumbing."""
import copy

import pytest
import torch

from llmq_b200.config import create_config_from_name
from llmq_b200.models.llama import LlamaModel
from llmq_b200.models.reference import adamw_ref, loss_ref
from llmq_b200.options import LLamaOptions

B, T = 2, 64


def make(opts=None, dtype=torch.float32, tied=True, seed=0):
    cfg = create_config_from_name("tiny-qwen2", dtype).replace(tie_word_embeddings=tied)
    opts = opts or LLamaOptions()
    m = LlamaModel(cfg, opts, device="cpu", batch_size=B, seq_len=T)
    m.init_weights(seed)
    return cfg, m


def data(seed=0, n=1):
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(0, 512, (n, B, T + 1), generator=g, dtype=torch.int32)
    return toks[:, :, :-1].contiguous(), toks[:, :, 1:].contiguous()


def params_of(m):
    return {name: master.detach().clone().float().requires_grad_(True) for name, master, _, _ in m.weights.master_items()}


@pytest.mark.parametrize("tied", [True, False])
@pytest.mark.parametrize("ga", [1, 2])
def test_forward_backward_matches_autograd(tied, ga):
    cfg, m = make(tied=tied)
    x, y = data(1, ga)
    y[0, 0, 5] = -100
    ref_p = params_of(m)
    total = 0
    for j in range(ga):
        loss, ce = loss_ref(cfg, ref_p, x[j], y[j], positions=B * T * ga)
        loss.backward()
        total += ce.item()
    for j in range(ga):
        m.forward(x[j], j)
        m.backward(x[j], y[j], 0.0, ga, j)
    grads = m.get_gradients()
    for name, g in grads.items():
        ref = ref_p[name].grad
        err = (g.float() - ref).abs().max().item()
        assert err <= 1e-5 + 1e-3 * ref.abs().max().item(), (name, err, ref.abs().max().item())
    res = m.update(lr=0.0, step=1, grad_accum=ga)
    assert abs(res["loss"] - total) < 1e-4
    ref_norm = torch.sqrt(sum(p.grad.pow(2).sum() for p in ref_p.values())).item()
    assert abs(res["norm"] - ref_norm) < 1e-4 * max(1, ref_norm)


def test_zloss_gradient():
    cfg, m = make()
    x, y = data(2)
    ref_p = params_of(m)
    loss, _ = loss_ref(cfg, ref_p, x[0], y[0], z_loss=1e-2)
    loss.backward()
    m.forward(x[0])
    m.backward(x[0], y[0], 1e-2, 1, 0)
    for name, g in m.get_gradients().items():
        ref = ref_p[name].grad
        assert (g.float() - ref).abs().max().item() <= 1e-5 + 1e-3 * ref.abs().max().item(), name


def test_adamw_step_matches_reference():
    cfg, m = make()
    x, y = data(3)
    before = {n: t.clone() for n, t in params_of(m).items()}
    m.forward(x[0])
    m.backward(x[0], y[0], 0.0, 1, 0)
    grads = {n: g.clone().float() for n, g in m.get_gradients().items()}
    norm = torch.sqrt(sum(g.pow(2).sum() for g in grads.values())).item()
    clip = 0.5 * norm                       # force clipping
    m.update(lr=1e-2, beta1=0.9, beta2=0.95, step=1, eps=1e-8, weight_decay=0.1, grad_clip=clip)
    for name, master, spec, _ in m.weights.master_items():
        g = grads[name] * (clip / norm)
        p, _, _ = adamw_ref(before[name].detach(), g, torch.zeros_like(g), torch.zeros_like(g), 1e-2, 0.9, 0.95, 1, 1e-8,
                            0.1 if spec.matrix else 0.0)
        assert (master.float() - p).abs().max().item() < 2e-5, name


RECOMPUTE = [dict(recompute_swiglu=True), dict(recompute_rms_norm=True), dict(recompute_ffn=True), dict(recompute_qkv=True),
             dict(recompute_att=True), dict(recompute_block=True), dict(recompute_swiglu=True, recompute_rms_norm=True),
             dict(lmhead_chunks=4), dict(shard_weights=True), dict(shard_gradients=True),
             dict(shard_weights=True, shard_gradients=True, recompute_block=True)]


@pytest.mark.parametrize("mm", ["fp32", "e4m3"])
@pytest.mark.parametrize("kw", RECOMPUTE, ids=lambda d: "+".join(d))
def test_variants_are_bit_identical(kw, mm):
    """Recompute / chunking / sharding variants must reproduce the plain run exactly (losses, norms, weights)."""
    def run(**o):
        mt = None if mm == "fp32" else "e4m3"
        _, m = make(LLamaOptions(matmul_type=mt, **o))
        x, y = data(4, 2)
        out = []
        for step in range(1, 3):
            for j in range(2):
                m.forward(x[j], j)
                m.backward(x[j], y[j], 0.0, 2, j)
            r = m.update(lr=1e-3, step=step, grad_accum=2)
            out.append((r["loss"], r["norm"]))
        return out, [t.clone() for _, t, _, _ in m.weights.master_items()]
    base, wb = run()
    var, wv = run(**kw)
    if "lmhead_chunks" in kw:
        # chunking changes the summation order of the head's weight gradient: equal up to rounding only
        for (l0, n0), (l1, n1) in zip(base, var):
            assert abs(l0 - l1) < 1e-5 and abs(n0 - n1) < 1e-4
        return
    assert base == var
    for a, b in zip(wb, wv):
        assert torch.equal(a, b)


def test_fp8_matmuls_track_fp32():
    cfg, m32 = make()
    _, m8 = make(LLamaOptions(matmul_type="e4m3"))
    x, y = data(5)
    for m in (m32, m8):
        m.forward(x[0])
        m.backward(x[0], y[0], 0.0, 1, 0)
    r32, r8 = m32.update(lr=0.0, step=1), m8.update(lr=0.0, step=1)
    assert abs(r32["loss"] - r8["loss"]) < 2e-2
    g32, g8 = m32.get_gradients(), m8.get_gradients()
    cos = []
    for n in g32:
        a, b = g32[n].flatten().float(), g8[n].flatten().float()
        if a.norm() > 0:
            cos.append(torch.dot(a, b) / (a.norm() * b.norm() + 1e-12))
    assert min(cos) > 0.9 and sum(cos) / len(cos) > 0.97


def test_validate_and_bf16():
    cfg, m = make(dtype=torch.bfloat16)
    x, y = data(6)
    loss, loss1k = m.validate(x[0], y[0])
    assert abs(loss - 6.24) < 0.3 and abs(loss - loss1k) < 1e-5      # ~ln(512) at init
    m.forward(x[0])
    m.backward(x[0], y[0], 0.0, 1, 0)
    r = m.update(lr=1e-3, step=1)
    assert abs(r["loss"] - loss) < 5e-2 and r["norm"] > 0


def test_fp32_model_with_bf16_matmuls_tracks_fp32():
    """Mixed precision: fp32 weights / activations, GEMM operands rounded to bf16 (``--model-dtype fp32 --matmul-dtype bf16``)."""
    _, m32 = make()
    _, mx = make(LLamaOptions(matmul_type="bf16"))
    assert mx.quant and mx.qdtype == torch.bfloat16 and mx.dtype == torch.float32
    x, y = data(7)
    for m in (m32, mx):
        m.forward(x[0])
        m.backward(x[0], y[0], 0.0, 1, 0)
    r32, rx = m32.update(lr=0.0, step=1), mx.update(lr=0.0, step=1)
    assert abs(r32["loss"] - rx["loss"]) < 2e-3
    g32, gx = m32.get_gradients(), mx.get_gradients()
    for n in g32:
        a, b = g32[n].flatten().float(), gx[n].flatten().float()
        if a.norm() > 0:
            assert torch.dot(a, b) / (a.norm() * b.norm() + 1e-12) > 0.999, n


def test_temporaries_live_on_the_stack_and_phases_share_addresses():
    """The step's temporaries are views of one stack buffer sized by a dry run; LM-head buffers and block-backward buffers
    are pushed and popped per phase, so they overlap, while the buffers that live for the whole step do not."""
    from llmq_b200.config import create_config_from_name
    from llmq_b200.models.llama import LlamaModel
    from llmq_b200.options import LLamaOptions
    from llmq_b200.utils.memory import allocator_report

    cfg = create_config_from_name("tiny-qwen2", "fp32")
    m = LlamaModel(cfg, LLamaOptions(lmhead_chunks=2), batch_size=2, seq_len=64)
    t, back = m.tmp, m.stack.backing
    lo, hi = back.data_ptr(), back.data_ptr() + back.numel()
    span = lambda x: (x.data_ptr(), x.data_ptr() + x.numel() * x.element_size())
    for name in ("proj", "d_res", "d_ln", "logits", "d_sw", "d_qkv", "att_scratch"):
        a, b = span(getattr(t, name))
        assert lo <= a and b <= hi, name
    overlap = lambda x, y: span(x)[0] < span(y)[1] and span(y)[0] < span(x)[1]
    assert overlap(t.logits, t.d_sw)                                 # different phases: same addresses
    assert not overlap(t.proj, t.logits) and not overlap(t.d_res, t.d_sw) and not overlap(t.d_sw, t.d_qkv)
    rep = m.stack_report
    assert rep["capacity"] == rep["high_water"] == back.numel() and rep["breakdown"]
    assert allocator_report(m)["_stack"]["high_water"] == rep["high_water"]
