"""The pyllmq-compatible import package and the torch custom-op kernel API, on CPU tensors (PyTorch reference paths)."""
import numpy as np
import pytest
import torch

import llmq_b200.kernels_api as ops
import pyllmq


def test_pyllmq_surface():
    cfg = pyllmq.Config.from_name("Qwen2.5-0.5B")
    assert cfg.hidden_size == 896 and cfg.num_hidden_layers == 24 and cfg.vocab_size == 151936
    for name in ("LLMQTrainer", "LLamaOptions", "DataLoader", "TrainingRunLogger", "TrainingConfig", "CosineLRSchedule", "get_num_gpus"):
        assert hasattr(pyllmq, name) or hasattr(pyllmq.training, name), name
    tc = pyllmq.training.TrainingConfig()
    assert tc.matmul_dtype in (None, "", "bf16", "e4m3") or isinstance(tc.matmul_dtype, str)


def test_tiny_trainer_through_pyllmq():
    cfg = pyllmq.Config(hidden_size=64, intermediate_size=128, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2,
                        vocab_size=256, max_position_embeddings=128, tie_word_embeddings=True)
    tr = pyllmq.LLMQTrainer(ngpu=1, config=cfg, options=pyllmq.LLamaOptions(), batch_size=2, seq_len=32, grad_accum=1, device="cpu")
    tr.init_weights()
    rng = np.random.default_rng(0)
    tok = rng.integers(0, 256, size=(2, 33), dtype=np.int32)
    first = None
    for step in range(3):
        tr.step(np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:]))
        r = tr.update(1e-2, 0.9, 0.95, step + 1, 0.0, 1.0)
        first = first if first is not None else r["loss"]
    assert r["loss"] < first and np.isfinite(r["norm"])


def test_custom_ops_on_cpu_tensors():
    torch.manual_seed(0)
    x, w = torch.randn(6, 64).bfloat16(), (1 + 0.1 * torch.randn(64)).bfloat16()
    out, rms = torch.zeros_like(x), torch.zeros(6)
    torch.ops.llmq_b200.rmsnorm_forward(out, rms, x, w, None, 1e-6)
    ref = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)).bfloat16().float() * w.float()
    assert torch.allclose(out.float(), ref, atol=2e-2)
    a, b = torch.randn(8, 32).bfloat16(), torch.randn(16, 32).bfloat16()
    c = torch.zeros(8, 16, dtype=torch.bfloat16)
    ops.matmul(c, a, b, None, None, None, None, "TN", False)
    assert torch.allclose(c.float(), a.float() @ b.float().t(), atol=0.25, rtol=2e-2)
    up = torch.randn(4, 2 * 16).bfloat16()
    sw, am = torch.zeros(4, 16, dtype=torch.bfloat16), torch.zeros(1)
    torch.ops.llmq_b200.swiglu_forward(sw, up, am)
    u, g = up[:, :16].float(), up[:, 16:].float()
    assert torch.allclose(sw.float(), u * g * torch.sigmoid(g), atol=3e-2) and am.item() > 0
    q, scale = torch.zeros(6, 64, dtype=torch.float8_e4m3fn), torch.zeros(1)
    amx = x.float().abs().max().reshape(1)
    torch.ops.llmq_b200.quantize_with_abs_max(q, scale, x, amx)
    assert torch.allclose(q.float() * scale, x.float(), atol=0.07 * amx.item())
    p_, g_, m_, v_ = torch.randn(64).bfloat16(), torch.randn(64).bfloat16(), torch.zeros(64), torch.zeros(64)
    before = p_.clone()
    ops.adamw_update(p_, g_, m_, v_, 1e-2, 0.9, 0.95, 1, 1e-8, 0.0)
    assert not torch.equal(before, p_) and m_.abs().sum() > 0


def test_block_scaled_custom_ops():
    torch.manual_seed(1)
    a, b = torch.randn(128, 256).bfloat16(), torch.randn(224, 256).bfloat16()
    aq, bq = torch.zeros(128, 256, dtype=torch.float8_e4m3fn), torch.zeros(224, 256, dtype=torch.float8_e4m3fn)
    asf = torch.zeros(ops.mx_scale_bytes(128, 256, "a"), dtype=torch.uint8)
    bsf = torch.zeros(ops.mx_scale_bytes(224, 256, "b"), dtype=torch.uint8)
    torch.ops.llmq_b200.quantize_mx(aq, asf, a, False, "a")
    torch.ops.llmq_b200.quantize_mx(bq, bsf, b, False, "b")
    c = torch.zeros(128, 224)
    torch.ops.llmq_b200.matmul_mx(c, aq, asf, bq, bsf, None, None, False)
    ref = a.float() @ b.float().t()
    assert (c - ref).norm() / ref.norm() < 0.05


def test_reference_matmul_signature():
    """``pyllmq.kernels.matmul`` with the reference's argument list (handle, workspace, integer transpose mode)."""
    import pyllmq.kernels as pk
    h = pk.create_cublas_handle()
    g = torch.Generator().manual_seed(0)
    A, Bm = torch.randn(6, 10, generator=g), torch.randn(10, 4, generator=g)     # c = A @ Bm
    bias, ws = torch.randn(4, generator=g), torch.empty(16)
    forms = {pk.MM_NN: (A, Bm), pk.MM_TN: (A.t().contiguous(), Bm), pk.MM_NT: (A, Bm.t().contiguous()),
             pk.MM_TT: (A.t().contiguous(), Bm.t().contiguous())}
    for mode, (a, b) in forms.items():
        c = torch.zeros(6, 4)
        pk.matmul(c, a, b, bias, None, None, h, ws, mode)
        assert torch.allclose(c, A @ Bm + bias, atol=1e-5), mode
        pk.matmul(c, a, b, None, None, None, h, ws, mode, True)
        assert torch.allclose(c, 2 * (A @ Bm) + bias, atol=1e-5), mode
    with pytest.raises(ValueError):
        pk.matmul(torch.zeros(6, 4), A, Bm, None, None, None, h, ws, 7)
    pk.destroy_cublas_handle(h)


def test_reference_argument_lists():
    """The calls of ``pyllmq.kernels`` that take the reference's extra arguments (handles, workspaces, bucket tables)
    give what the plain ops give."""
    import pyllmq.kernels as pk
    g = torch.Generator().manual_seed(3)
    B, T, C, V, Hq, Hkv, HS = 2, 16, 32, 50, 4, 2, 8
    tok = torch.randint(0, V, (B, T), generator=g, dtype=torch.int32)
    wte, wpe = torch.randn(V, C, generator=g), torch.randn(T, C, generator=g)
    out = torch.empty(B, T, C)
    pk.encoder_forward(out, tok, wte, wpe)
    assert torch.allclose(out, wte[tok.long()] + wpe)
    dout = torch.randn(B, T, C, generator=g)
    d1, d2 = torch.zeros(V, C), torch.zeros(V, C)
    pk.encoder_backward(d1, None, None, None, dout, tok, tok.clone(), 5)
    ops.encoder_backward(d2, dout, tok)
    assert torch.equal(d1, d2) and d1.abs().sum() > 0
    # RMSNorm backward with a separate residual gradient
    x, w = torch.randn(B, T, C, generator=g), torch.randn(C, generator=g)
    y, rstd = torch.empty_like(x), torch.empty(B * T)
    ops.rmsnorm_forward(y, rstd, x, w, None, 1e-6)
    dres = torch.randn(B, T, C, generator=g)
    scratch = torch.empty(ops.get_rmsnorm_backward_scratch_size(C, "cpu") // 4)
    a, dwa = torch.full_like(x, 7.0), torch.zeros(C)
    pk.rmsnorm_backward(a, dwa, scratch, dres, dout, x, w, rstd, None)
    b, dwb = dres.clone(), torch.zeros(C)
    ops.rmsnorm_backward(b, dwb, scratch, dout, x, w, rstd, None)
    assert torch.equal(a, b) and torch.equal(dwa, dwb)
    # attention with workspace / handle arguments
    qkv = torch.randn(B, T, Hq + 2 * Hkv, HS, generator=g)
    o1, s1, o2, s2 = torch.empty(B, T, Hq, HS), torch.empty(B, Hq, T), torch.empty(B, T, Hq, HS), torch.empty(B, Hq, T)
    ws = torch.empty(4 * B * Hq * T, dtype=torch.uint8)
    pk.attention_forward(o1, s1, qkv, ws, 0, Hq, Hkv)
    ops.attention_forward(o2, s2, qkv, Hq, Hkv)
    assert torch.equal(o1, o2) and torch.equal(s1, s2)
    do = torch.randn(B, T, Hq, HS, generator=g)
    g1, g2 = torch.empty_like(qkv), torch.empty_like(qkv)
    pk.attention_backward(g1, s1, o1, do, qkv, ws, 0, Hq, Hkv)
    ops.attention_backward(g2, torch.empty(B * Hq * T), s2, o2, do, qkv, Hq, Hkv)
    assert torch.equal(g1, g2)
    pk.attention_backward(g1, s1, o1, do, qkv, None, 0, Hq, Hkv)                 # no workspace: scratch is allocated
    assert torch.equal(g1, g2)


def test_fixed_reference_ten_steps():
    """Regression guard in the manner of the reference's fixed-reference runs (``scripts/modal_test_app.py:101-143``
    there): ten optimizer steps of the tiny Qwen2 model on seeded tokens against stored loss / gradient-norm values.
    The stored numbers are CPU fp32, so the comparison has a small tolerance instead of exact equality; two runs in
    one process must agree exactly."""
    from llmq_b200.config import create_config_from_name
    want = [(6.257861, 0.812518), (6.236615, 0.778743), (6.267263, 0.797388), (6.280034, 0.81367), (6.263968, 0.810399),
            (6.239417, 0.801177), (6.256784, 0.792924), (6.239585, 0.784477), (6.253052, 0.783787), (6.251751, 0.805303)]

    def run():
        tr = pyllmq.LLMQTrainer(ngpu=1, config=create_config_from_name("tiny-qwen2", torch.float32), options=pyllmq.LLamaOptions(),
                                batch_size=2, seq_len=64, grad_accum=2, device="cpu")
        tr.init_weights()
        rng = np.random.default_rng(42)
        out = []
        for step in range(10):
            for _ in range(2):
                tok = rng.integers(0, 512, size=(2, 65), dtype=np.int32)
                tr.step(np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:]))
            r = tr.update(1e-3, 0.9, 0.95, step + 1, 0.1, 1.0)
            out.append((r["loss"], r["norm"]))
        return out

    a, b = run(), run()
    assert a == b
    for (l, n), (wl, wn) in zip(a, want):
        assert abs(l - wl) < 5e-4 and abs(n - wn) < 5e-4, (a, want)


def test_script_modules_under_reference_paths():
    import pyllmq.scripts.tokenize_data as tk
    import pyllmq.scripts.train as tr
    from pyllmq.scripts import demo, export_wandb, plot_training_run
    assert all(callable(m.main) for m in (tk, tr, demo, export_wandb, plot_training_run))
