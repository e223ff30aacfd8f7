"""Every CUDA kernel against the plain PyTorch fp32 implementation of the same operation (the CPU path
of llmq_b200.ops.kernels), at small and odd shapes."""
import math

import pytest
import torch

from llmq_b200.ops import kernels as K

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16
F8 = torch.float8_e4m3fn


def close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float().cpu(), b.float().cpu()
    assert a.shape == b.shape
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert err <= atol + rtol * ref, f"max err {err} vs ref scale {ref}"


@pytest.fixture(autouse=True)
def _check_status():
    yield
    torch.cuda.synchronize()
    K.check_status(torch.device(DEV, 0))


@pytest.mark.parametrize("M,N,Kd", [(128, 256, 32), (384, 272, 200), (1008, 896, 1024)])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1), (1, 0)])
@pytest.mark.parametrize("accumulate", [False, True])
def test_gemm_fp32_operands_tf32(M, N, Kd, a_mn, b_mn, accumulate):
    """fp32 operands go through the tf32 MMA kind: products carry a 10-bit mantissa, accumulation is fp32."""
    torch.manual_seed(2)
    A, Bm, bias = torch.randn(M, Kd), torch.randn(N, Kd), torch.randn(N)
    prev = torch.randn(M, N)
    ref = A.double() @ Bm.double().t() + bias.double() + (prev.double() if accumulate else 0)
    As = A.t().contiguous() if a_mn else A
    Bs = Bm.t().contiguous() if b_mn else Bm
    out = prev.clone().to(DEV)
    K.gemm(out, As.to(DEV), Bs.to(DEV), a_mn=bool(a_mn), b_mn=bool(b_mn), bias=bias.to(DEV), accumulate=accumulate)
    err = (out.cpu().double() - ref).abs().max().item()
    assert err <= 2e-3 * (A.abs().max() * Bm.abs().max()).item() * Kd ** 0.5, err


@pytest.mark.parametrize("M,N,Kd", [(128, 256, 64), (384, 272, 192), (1008, 896, 1024)])
@pytest.mark.parametrize("dt", ["bf16", "fp8"])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1), (1, 0)])
def test_gemm(M, N, Kd, dt, a_mn, b_mn):
    torch.manual_seed(1)
    A = torch.randn(M, Kd)
    B = torch.randn(N, Kd)
    A, B = (A.to(BF), B.to(BF)) if dt == "bf16" else (A.to(F8), B.to(F8))
    As = A.float().t().contiguous().to(A.dtype) if a_mn else A
    Bs = B.float().t().contiguous().to(B.dtype) if b_mn else B
    out = torch.zeros(M, N, dtype=BF, device=DEV)
    K.gemm(out, As.to(DEV), Bs.to(DEV), a_mn=bool(a_mn), b_mn=bool(b_mn))
    close(out, A.float() @ B.float().t(), rtol=1e-2, atol=1e-2)


def test_gemm_epilogue():
    torch.manual_seed(2)
    M, N, Kd = 256, 512, 256
    A, B = torch.randn(M, Kd).to(BF), torch.randn(N, Kd).to(BF)
    bias = torch.randn(N).to(BF)
    C0 = torch.randn(M, N).to(BF)
    sa, sb = torch.tensor([0.5]), torch.tensor([0.25])
    ref = C0.clone()
    am_ref = torch.zeros(1)
    K.gemm(ref, A, B, bias=bias, accumulate=True, scale_a=sa, scale_b=sb, alpha=2.0, absmax=am_ref)
    out = C0.to(DEV)
    am = torch.zeros(1, device=DEV)
    K.gemm(out, A.to(DEV), B.to(DEV), bias=bias.to(DEV), accumulate=True, scale_a=sa.to(DEV), scale_b=sb.to(DEV), alpha=2.0, absmax=am)
    close(out, ref)
    close(am, am_ref)
    outf = torch.zeros(M, N, device=DEV)
    K.gemm(outf, A.to(DEV), B.to(DEV))
    close(outf, A.float() @ B.float().t(), rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("dt", ["bf16", "fp8"])
@pytest.mark.parametrize("M,N,Kd,a_mn,b_mn", [(256, 256, 8192, 0, 0), (896, 1152, 4096, 1, 1), (200, 304, 2560, 0, 1)])
def test_gemm_split_k(M, N, Kd, a_mn, b_mn, dt):
    """Few output tiles and a long K: the K loop is split over several CTAs and summed by a second kernel."""
    torch.manual_seed(21)
    A, B = torch.randn(M, Kd) * 0.5, torch.randn(N, Kd) * 0.5
    A, B = (A.to(BF), B.to(BF)) if dt == "bf16" else (A.to(F8), B.to(F8))
    As = A.float().t().contiguous().to(A.dtype) if a_mn else A
    Bs = B.float().t().contiguous().to(B.dtype) if b_mn else B
    bias, C0 = torch.randn(N).to(BF), torch.randn(M, N).to(BF)
    sa = torch.tensor([0.5])
    ref = (A.float() @ B.float().t()) * 0.5 + bias.float() + C0.float()
    out = C0.to(DEV)
    am = torch.zeros(1, device=DEV)
    K.gemm(out, As.to(DEV), Bs.to(DEV), a_mn=bool(a_mn), b_mn=bool(b_mn), bias=bias.to(DEV), accumulate=True, scale_a=sa.to(DEV), absmax=am)
    K.check_status(torch.device(DEV))
    close(out, ref, rtol=1e-2, atol=0.3)
    assert abs(am.item() - out.float().abs().max().item()) < 8e-3 * am.item()          # abs-max is taken before the bf16 rounding
    outf = torch.zeros(M, N, device=DEV)
    K.gemm(outf, As.to(DEV), Bs.to(DEV), a_mn=bool(a_mn), b_mn=bool(b_mn))
    close(outf, A.float() @ B.float().t(), rtol=1e-3, atol=2e-2)


@pytest.mark.parametrize("C", [64, 896, 3584])
@pytest.mark.parametrize("fused", [False, True])
def test_rmsnorm_forward(C, fused):
    torch.manual_seed(3)
    rows = 37
    a, b, w = torch.randn(rows, C).to(BF), torch.randn(rows, C).to(BF), (1 + 0.1 * torch.randn(C)).to(BF)
    outs = []
    for dev in ("cpu", DEV):
        y = torch.zeros(rows, C, dtype=BF, device=dev)
        res = torch.zeros(rows, C, dtype=BF, device=dev)
        rstd = torch.zeros(rows, device=dev)
        am = torch.zeros(1, device=dev)
        K.rmsnorm_forward(y, rstd, a.to(dev), w.to(dev), 1e-6, residual_out=res if fused else None,
                          inp2=b.to(dev) if fused else None, absmax=am)
        q = torch.zeros(rows, C, dtype=F8, device=dev)
        qs = torch.zeros(1, device=dev)
        K.rmsnorm_forward(None, None, a.to(dev), w.to(dev), 1e-6, residual_out=res if fused else None,
                          inp2=b.to(dev) if fused else None, q_out=q, known_absmax=am, q_scale=qs)
        outs.append((y, res, rstd, am, q, qs))
    for g, r in zip(outs[1], outs[0]):
        close(g, r, rtol=1e-2, atol=1e-2 if g.dtype != F8 else 0.07 * 448)


@pytest.mark.parametrize("C", [64, 896, 3584])
def test_rmsnorm_backward(C):
    torch.manual_seed(4)
    rows = 300
    x, dy, w = torch.randn(rows, C).to(BF), torch.randn(rows, C).to(BF), (1 + 0.1 * torch.randn(C)).to(BF)
    dres = torch.randn(rows, C).to(BF)
    dw0 = torch.randn(C).to(BF)
    res = []
    for dev in ("cpu", DEV):
        rstd = torch.zeros(rows, device=dev)
        K.rmsnorm_forward(None, rstd, x.to(dev), w.to(dev), 1e-6)
        dinp = dres.clone().to(dev)
        dw = dw0.clone().to(dev)
        am = torch.zeros(1, device=dev)
        scratch = torch.zeros(K.rmsnorm_backward_scratch_elems(C, dev), device=dev)
        K.rmsnorm_backward(dinp, dw, scratch, dy.to(dev), x.to(dev), w.to(dev), rstd, absmax=am, accumulate_dweight=True)
        res.append((dinp, dw, am))
    close(res[1][0], res[0][0])
    close(res[1][1], res[0][1], rtol=2e-2, atol=0.3)
    close(res[1][2], res[0][2])


@pytest.mark.parametrize("D", [8, 172 * 2, 4864])
def test_swiglu(D):
    torch.manual_seed(5)
    rows = 33
    x = torch.randn(rows, 2 * D).to(BF)
    dy = torch.randn(rows, D).to(BF)
    res = []
    for dev in ("cpu", DEV):
        out = torch.zeros(rows, D, dtype=BF, device=dev)
        am = torch.zeros(1, device=dev)
        K.swiglu_forward(out, x.to(dev), absmax=am)
        q = torch.zeros(rows, D, dtype=F8, device=dev)
        qs = torch.zeros(1, device=dev)
        K.swiglu_forward(None, x.to(dev), q_out=q, known_absmax=am, q_scale=qs)
        dx = x.clone().to(dev)
        am2 = torch.zeros(1, device=dev)
        K.swiglu_backward(dx, dy.to(dev), dx, absmax=am2)
        res.append((out, am, q, qs, dx, am2))
    for g, r in zip(res[1], res[0]):
        close(g, r, rtol=1e-2, atol=1e-2 if g.dtype != F8 else 0.07 * 448)


@pytest.mark.parametrize("HS", [16, 64, 128])
def test_rope(HS):
    torch.manual_seed(6)
    B, T, Hq, Hkv = 2, 48, 4, 2
    x = torch.randn(B, T, Hq + 2 * Hkv, HS).to(BF)
    res = []
    for dev in ("cpu", DEV):
        f = K.rope_table(T, HS, 1e6, dev)
        y = x.clone().to(dev)
        K.rope(y, y, f, Hq, Hkv)
        z = torch.zeros_like(y)
        am = torch.zeros(1, device=dev)
        K.rope(z, y, f, Hq, Hkv, backward=True, absmax=am)
        res.append((f, y, z, am))
    for g, r in zip(res[1], res[0]):
        close(g, r, rtol=1e-2, atol=1e-2)
    close(res[1][2], x, rtol=2e-2, atol=3e-2)          # backward(forward(x)) == x


def test_quant_transpose_convert_fill():
    torch.manual_seed(7)
    x = (torch.randn(130, 72) * 3).to(BF)
    for dev in (DEV,):
        xd = x.to(dev)
        am = torch.zeros(1, device=dev)
        K.abs_max(am, xd)
        assert am.item() == x.float().abs().max().item()
        for qdt in (F8, torch.float8_e5m2):
            q = torch.zeros(130, 72, dtype=qdt, device=dev)
            sc = torch.zeros(1, device=dev)
            K.quantize(q, sc, xd, am)
            qr = torch.zeros(130, 72, dtype=qdt)
            scr = torch.zeros(1)
            K.quantize(qr, scr, x, am.cpu())
            close(q.float() * sc, qr.float() * scr, rtol=0.13, atol=0)
            close(q.float() * sc, x, rtol=0.13, atol=0)
            qt = torch.zeros(72, 130, dtype=qdt, device=dev)
            K.transpose(qt, xd, absmax=am, scale_out=sc)
            assert torch.equal(qt.float().t().cpu(), q.float().cpu())
        t = torch.zeros(72, 130, dtype=BF, device=dev)
        K.transpose(t, xd)
        assert torch.equal(t.cpu(), x.t())
        f = torch.zeros(130, 72, device=dev)
        K.convert(f, xd)
        assert torch.equal(f.cpu(), x.float())
        K.fill(f, 1.5)
        assert (f == 1.5).all()
        n = torch.zeros(1 << 20, dtype=BF, device=dev)
        K.fill_normal(n, 0.5, 0.02, seed=42, subsequence=3)
        assert abs(n.float().mean().item() - 0.5) < 1e-3 and abs(n.float().std().item() - 0.02) < 1e-3
        part = torch.zeros(1 << 10, dtype=BF, device=dev)
        K.fill_normal(part, 0.5, 0.02, seed=42, subsequence=3, offset=4096)
        assert torch.equal(part, n[4096:4096 + 1024])
        other = torch.zeros(1 << 10, dtype=BF, device=dev)
        K.fill_normal(other, 0.5, 0.02, seed=42, subsequence=4)
        assert not torch.equal(other, n[:1024])


@pytest.mark.parametrize("rows,cols", [(128, 128), (400, 208), (1024, 3584), (16, 4864)])
@pytest.mark.parametrize("src", ["bf16", "fp32", "e4m3", "e5m2"])
def test_quantize_transpose_tiles(rows, cols, src):
    """The 128 x 128 tile kernel: row-major fp8 copy equals the plain quantiser bit for bit, the transposed copy is its
    exact transpose; 1-byte inputs are copied.  Shapes cover full tiles, ragged tiles and a single 16-row strip."""
    torch.manual_seed(rows + cols)
    x = torch.randn(rows, cols) * 2.5
    for qdt in ((F8, torch.float8_e5m2) if src in ("bf16", "fp32") else ((F8,) if src == "e4m3" else (torch.float8_e5m2,))):
        if src in ("bf16", "fp32"):
            xd = x.to(BF if src == "bf16" else torch.float32).to(DEV)
            am = torch.zeros(1, device=DEV)
            K.abs_max(am, xd)
            ref_rows = torch.zeros(rows, cols, dtype=qdt, device=DEV)
            sc_ref = torch.zeros(1, device=DEV)
            K.quantize(ref_rows, sc_ref, xd, am)
            out_rows = torch.zeros(rows, cols, dtype=qdt, device=DEV)
            out_t = torch.zeros(cols, rows, dtype=qdt, device=DEV)
            sc = torch.zeros(1, device=DEV)
            K.quantize_transpose(out_rows, out_t, sc, xd, am)
            assert sc.item() == sc_ref.item()
            assert torch.equal(out_rows.view(torch.uint8), ref_rows.view(torch.uint8))
            assert torch.equal(out_t.view(torch.uint8), ref_rows.view(torch.uint8).t())
            only_t = torch.zeros(cols, rows, dtype=qdt, device=DEV)
            K.quantize_transpose(None, only_t, None, xd, am)
            assert torch.equal(only_t.view(torch.uint8), out_t.view(torch.uint8))
        else:
            xq = x.to(qdt).to(DEV)
            out_t = torch.zeros(cols, rows, dtype=qdt, device=DEV)
            K.transpose(out_t, xq)
            assert torch.equal(out_t.view(torch.uint8), xq.view(torch.uint8).t())


@pytest.mark.parametrize("rows,cols", [(64, 8), (256, 136), (1000, 3584), (72, 4104)])
def test_transpose_bf16_tiles(rows, cols):
    """The 64 x 64 tile transpose of 2-byte elements (full and ragged tiles) is exact."""
    torch.manual_seed(rows)
    x = torch.randn(rows, cols).to(BF).to(DEV)
    out = torch.zeros(cols, rows, dtype=BF, device=DEV)
    K.transpose(out, x)
    assert torch.equal(out, x.t())


@pytest.mark.parametrize("rows,D", [(256, 128), (400, 4864), (1024, 176)])
def test_swiglu_forward_transposed(rows, D):
    """The recompute kernel that writes only the transposed e4m3 activation: same bytes as quantise-then-transpose."""
    torch.manual_seed(5)
    inp = (torch.randn(rows, 2 * D) * 1.5).to(BF).to(DEV)
    out = torch.zeros(rows, D, dtype=BF, device=DEV)
    am = torch.zeros(1, device=DEV)
    K.swiglu_forward(out, inp, absmax=am)
    q = torch.zeros(rows, D, dtype=F8, device=DEV)
    sc = torch.zeros(1, device=DEV)
    K.swiglu_forward(None, inp, q_out=q, known_absmax=am, q_scale=sc)
    qt = torch.zeros(D, rows, dtype=F8, device=DEV)
    sc2 = torch.zeros(1, device=DEV)
    K.swiglu_forward_transposed(qt, inp, known_absmax=am, q_scale=sc2)
    assert sc.item() == sc2.item()
    assert torch.equal(qt.view(torch.uint8), q.view(torch.uint8).t())


@pytest.mark.parametrize("rows,D", [(256, 384), (272, 208), (1040, 1168)])
@pytest.mark.parametrize("with_act", [False, True])
def test_swiglu_backward_two_pass(rows, D, with_act):
    """Abs-max pass + quantising pass against swiglu_backward followed by quantize_transpose: same abs-max, same scale, same
    bytes in both copies; the first pass's optional transposed activation equals swiglu_forward_transposed's."""
    torch.manual_seed(6)
    inp = (torch.randn(rows, 2 * D) * 1.5).to(BF).to(DEV)
    dout = (torch.randn(rows, D) * 0.7).to(BF).to(DEV)
    # the separate kernels
    d_ref = torch.zeros(rows, 2 * D, dtype=BF, device=DEV)
    am_ref = torch.zeros(1, device=DEV)
    K.swiglu_backward(d_ref, dout, inp, absmax=am_ref)
    q_ref = torch.zeros(rows, 2 * D, dtype=F8, device=DEV)
    qt_ref = torch.zeros(2 * D, rows, dtype=F8, device=DEV)
    sc_ref = torch.zeros(1, device=DEV)
    K.quantize_transpose(q_ref, qt_ref, sc_ref, d_ref, am_ref)
    # fp32 oracle of the gradient itself
    x = inp.float()
    up, gate = x[:, :D], x[:, D:]
    s_ = torch.sigmoid(gate)
    want = torch.cat([dout.float() * gate * s_, dout.float() * up * s_ * (1 + gate * (1 - s_))], -1)
    assert (d_ref.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    # the two passes
    am = torch.zeros(1, device=DEV)
    act_am = torch.zeros(1, device=DEV)
    act_t = act_t_ref = None
    if with_act:
        K.swiglu_forward(torch.zeros(rows, D, dtype=BF, device=DEV), inp, absmax=act_am)
        act_t_ref = torch.zeros(D, rows, dtype=F8, device=DEV)
        K.swiglu_forward_transposed(act_t_ref, inp, known_absmax=act_am)
        act_t = torch.zeros(D, rows, dtype=F8, device=DEV)
    act_sc = torch.zeros(1, device=DEV)
    K.swiglu_backward_stats(am, dout, inp, act_t=act_t, act_absmax=act_am if with_act else None, act_scale=act_sc if with_act else None)
    assert am.item() == am_ref.item()
    q = torch.zeros(rows, 2 * D, dtype=F8, device=DEV)
    qt = torch.zeros(2 * D, rows, dtype=F8, device=DEV)
    sc = torch.zeros(1, device=DEV)
    K.swiglu_backward_quant(q, qt, sc, dout, inp, am)
    assert sc.item() == sc_ref.item()
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(qt.view(torch.uint8), qt_ref.view(torch.uint8))
    if with_act:
        assert act_sc.item() == pytest.approx(act_am.item() / 448.0, rel=1e-6)
        assert torch.equal(act_t.view(torch.uint8), act_t_ref.view(torch.uint8))


# Shapes with M >= 256 and M * N >= 2 Mi select the CTA-pair kernel (256 x 256 tiles, cta_group::2), the kernel that carries
# the training step; the smaller shapes above all run the one-CTA kernel.
PAIR_SHAPES = [(2048, 1536, 512), (1104, 2000, 208), (2304, 4608, 3584)]      # every extent a multiple of 16 bytes in fp8 (TMA rows)


@pytest.mark.parametrize("M,N,Kd", PAIR_SHAPES)
@pytest.mark.parametrize("dt", ["bf16", "e4m3", "e5m2"])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1), (1, 0)])
def test_gemm_pair_kernel(M, N, Kd, dt, a_mn, b_mn):
    """Plain product on the CTA-pair kernel against fp32 A @ B^T, every operand layout, ragged M / N / K edges."""
    torch.manual_seed(11)
    tdt = {"bf16": BF, "e4m3": F8, "e5m2": torch.float8_e5m2}[dt]
    A, B = (torch.randn(M, Kd) * 0.5).to(tdt), (torch.randn(N, Kd) * 0.5).to(tdt)
    As = A.float().t().contiguous().to(tdt) if a_mn else A
    Bs = B.float().t().contiguous().to(tdt) if b_mn else B
    out = torch.zeros(M, N, dtype=BF, device=DEV)
    K.gemm(out, As.to(DEV), Bs.to(DEV), a_mn=bool(a_mn), b_mn=bool(b_mn))
    ref = A.float().to(DEV) @ B.float().to(DEV).t()
    close(out, ref.cpu(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("M,N,Kd", PAIR_SHAPES)
@pytest.mark.parametrize("dt", ["bf16", "e4m3"])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (1, 1)])
@pytest.mark.parametrize("out_dt", [BF, torch.float32])
def test_gemm_pair_kernel_epilogue(M, N, Kd, dt, a_mn, b_mn, out_dt):
    """Bias, accumulation into the existing output (the gradient-accumulation path), per-tensor scales, alpha and the
    abs-max output of the CTA-pair kernel against fp32 arithmetic."""
    torch.manual_seed(12)
    tdt = BF if dt == "bf16" else F8
    A, B = (torch.randn(M, Kd) * 0.5).to(tdt), (torch.randn(N, Kd) * 0.5).to(tdt)
    As = A.float().t().contiguous().to(tdt) if a_mn else A
    Bs = B.float().t().contiguous().to(tdt) if b_mn else B
    bias, C0 = torch.randn(N).to(BF), torch.randn(M, N).to(out_dt)
    sa, sb = torch.tensor([0.5]), torch.tensor([0.25])
    ref = (A.float().to(DEV) @ B.float().to(DEV).t()).cpu() * (0.5 * 0.25 * 2.0) + bias.float() + C0.float()
    out = C0.to(DEV)
    am = torch.zeros(1, device=DEV)
    K.gemm(out, As.to(DEV), Bs.to(DEV), a_mn=bool(a_mn), b_mn=bool(b_mn), bias=bias.to(DEV), accumulate=True, scale_a=sa.to(DEV),
           scale_b=sb.to(DEV), alpha=2.0, absmax=am)
    close(out, ref, rtol=1e-2, atol=5e-2)
    assert abs(am.item() - ref.abs().max().item()) <= 1e-2 * ref.abs().max().item() + 5e-2


@pytest.mark.parametrize("V", [512, 1000, 151936])
def test_fused_classifier(V):
    torch.manual_seed(8)
    rows = 24
    logits = (torch.randn(rows, V) * 2).to(BF)
    tg = torch.randint(0, V, (rows,), dtype=torch.int32)
    tg[3] = -100
    res = []
    for dev in ("cpu", DEV):
        lg = logits.clone().to(dev)
        losses = torch.zeros(rows, device=dev)
        lse = torch.zeros(rows, device=dev)
        K.fused_classifier(lg, losses, lse, tg.to(dev), 1.0 / rows, z_reg=1e-4)
        st = torch.zeros(2, device=dev)
        K.lse_stats(st, lse)
        res.append((lg, losses, lse, st))
    close(res[1][1], res[0][1], rtol=1e-3, atol=1e-3)
    close(res[1][2], res[0][2], rtol=1e-3, atol=1e-3)
    close(res[1][3], res[0][3], rtol=1e-3, atol=1e-3)
    close(res[1][0], res[0][0], rtol=2e-2, atol=1e-5)
    assert res[1][0][3].abs().max().item() == 0


@pytest.mark.parametrize("combo", [(BF, BF, BF), (BF, torch.float32, torch.float32), (BF, F8, BF), (torch.float32,) * 3])
def test_adamw(combo):
    torch.manual_seed(9)
    pd, md, vd = combo
    n = 128 * 37
    p0 = torch.randn(n).to(pd)
    g = (torch.randn(n) * 0.1).to(pd)
    res = []
    for dev in ("cpu", DEV):
        p = p0.clone().to(dev)
        m = torch.zeros(n, dtype=md, device=dev)
        v = torch.zeros(n, dtype=vd, device=dev)
        ms = torch.ones(n // 128, device=dev) if md == F8 else None
        gs = torch.tensor([0.5], device=dev)
        am = torch.zeros(1, device=dev)
        for step in (1, 2, 3):
            K.adamw(p, g.to(dev), m, v, lr=1e-2, beta1=0.9, beta2=0.95, step=step, eps=1e-8, weight_decay=0.1, grad_scale=gs,
                    absmax=am, m_scales=ms, seed=step, stochastic=True)
        mm = m.float() * ms.repeat_interleave(128) if md == F8 else m.float()
        res.append((p, mm, v, am))
    close(res[1][0], res[0][0], rtol=1e-2, atol=1e-2)
    close(res[1][1], res[0][1], rtol=8e-2, atol=1e-3)
    close(res[1][2], res[0][2], rtol=2e-2, atol=1e-5)
    close(res[1][3], res[0][3], rtol=1e-2, atol=1e-2)


def test_sr_unbiased_and_reduce():
    n = 1 << 16
    a = torch.full((n,), 1.0, dtype=BF, device=DEV)
    b = torch.full((n,), 2.0 ** -10, dtype=BF, device=DEV)        # far below bf16 resolution at 1.0
    dst = torch.zeros(n, dtype=BF, device=DEV)
    K.vector_add_sr(dst, a, b, 1.0, seed=5)
    mean = dst.float().mean().item()
    assert abs(mean - (1 + 2.0 ** -10)) < 2e-4, mean
    dst2 = torch.zeros(n, dtype=BF, device=DEV)
    K.vector_add_sr(dst2, a, b, 1.0, seed=5)
    assert torch.equal(dst, dst2)
    src = torch.randn(4, n, device=DEV).to(BF)
    out = torch.ones(n, dtype=BF, device=DEV)
    K.vector_reduce_sr(out, src, 0.25, 4, skip=1, accumulate=True, seed=1)
    ref = 0.25 * (src.float()[[0, 2, 3]].sum(0) + 1)
    close(out, ref, rtol=1e-2, atol=1e-2)


def test_global_norm():
    torch.manual_seed(10)
    xs = [torch.randn(1000, 37).to(BF).to(DEV), torch.randn(12345, device=DEV)]
    part = torch.zeros(K.NORM_PARTIALS, device=DEV)
    for x in xs:
        K.norm_squared(part, x)
    io = torch.zeros(2, device=DEV)
    K.deterministic_sum(io[:1], part)
    K.norm_finish(io, 1.0)
    ref = math.sqrt(sum(x.float().pow(2).sum().item() for x in xs))
    assert abs(io[0].item() - ref) / ref < 1e-4
    assert abs(io[1].item() - 1.0 / ref) / (1.0 / ref) < 1e-4


def test_encoder_and_bias():
    torch.manual_seed(11)
    V, C, B, T = 512, 64, 4, 96
    wte = torch.randn(V, C).to(BF)
    tok = torch.randint(0, 40, (B, T), dtype=torch.int32)
    res = []
    dout = torch.randn(B, T, C).to(BF)
    for dev in ("cpu", DEV):
        out = torch.zeros(B, T, C, dtype=BF, device=dev)
        K.encoder_forward(out, tok.to(dev), wte.to(dev))
        dw = torch.zeros(V, C, dtype=BF, device=dev)
        K.encoder_backward(dw, dout.to(dev), tok.to(dev))
        db = torch.ones(C, dtype=BF, device=dev)
        K.bias_backward(db, dout.to(dev), torch.zeros(64 * C, device=dev), accumulate=True)
        res.append((out, dw, db))
    assert torch.equal(res[1][0].cpu(), res[0][0])
    close(res[1][1], res[0][1], rtol=1e-2, atol=5e-2)
    close(res[1][2], res[0][2], rtol=1e-2, atol=5e-2)


@pytest.mark.parametrize("BT,n_distinct,C,dt", [(4096, 3, 128, BF), (1000, 700, 64, torch.float32), (16384, 5000, 896, BF)])
def test_encoder_backward_device_side(BT, n_distinct, C, dt):
    """Sort-free embedding backward: heavy duplicates (more than one list round per token), mostly distinct tokens, ids
    outside the vocabulary skipped; fp32 reference = ordered sum per token.  Run twice: bitwise reproducible."""
    torch.manual_seed(BT)
    V = 6000
    tok = torch.randint(0, n_distinct, (BT,), dtype=torch.int32)
    tok[5] = -100
    tok[17] = V + 3                                           # from a larger tokenizer: must not touch memory
    dout = torch.randn(BT, C).to(dt)
    prev = torch.randn(V, C).to(dt)
    ok = (tok >= 0) & (tok < V)
    ref = prev.float().clone()
    ref.index_add_(0, tok[ok].long(), dout.float()[ok])
    outs = []
    for _ in range(2):
        dw = prev.clone().to(DEV)
        K.encoder_backward(dw, dout.to(DEV), tok.to(DEV))
        outs.append(dw.cpu())
    assert torch.equal(outs[0], outs[1])
    close(outs[0], ref, rtol=1e-2 if dt == BF else 1e-5, atol=0.5 if dt == BF else 1e-3)
    untouched = torch.ones(V, dtype=torch.bool)
    untouched[tok[ok].long()] = False
    assert torch.equal(outs[0][untouched], prev[untouched])


def test_fused_classifier_ignores_out_of_range_targets():
    """Targets outside [0, V) behave like -100: zero loss, zero gradient row; rows with valid targets are unchanged."""
    torch.manual_seed(3)
    rows, V = 8, 1000
    logits = torch.randn(rows, V).to(BF)
    tg_ok = torch.randint(0, V, (rows,), dtype=torch.int32)
    tg_bad = tg_ok.clone()
    tg_bad[2], tg_bad[5] = V + 7, -3
    res = []
    for tg in (tg_ok, tg_bad):
        lg = logits.clone().to(DEV)
        losses = torch.zeros(rows, device=DEV)
        lse = torch.zeros(rows, device=DEV)
        K.fused_classifier(lg, losses, lse, tg.to(DEV), 1.0 / rows, write_dlogits=True)
        res.append((lg.cpu(), losses.cpu()))
    good = [i for i in range(rows) if i not in (2, 5)]
    assert torch.equal(res[0][0][good], res[1][0][good]) and torch.equal(res[0][1][good], res[1][1][good])
    assert (res[1][0][[2, 5]] == 0).all() and (res[1][1][[2, 5]] == 0).all()


@pytest.mark.parametrize("HS,Hq,Hkv,T", [(64, 4, 2, 256), (128, 4, 1, 384), (64, 14, 2, 128), (128, 7, 1, 200), (128, 8, 2, 1024), (128, 4, 4, 640),
                                         (128, 2, 1, 96)])
def test_attention(HS, Hq, Hkv, T):
    torch.manual_seed(12)
    B = 2
    qkv = torch.randn(B, T, Hq + 2 * Hkv, HS).to(BF)
    dout = torch.randn(B, T, Hq, HS).to(BF)
    res = []
    for dev in ("cpu", DEV):
        out = torch.zeros(B, T, Hq, HS, dtype=BF, device=dev)
        lse = torch.zeros(B, Hq, T, device=dev)
        am = torch.zeros(1, device=dev)
        K.attention_forward(out, lse, qkv.to(dev), Hq, Hkv, absmax=am)
        assert abs(am.item() - out.float().abs().max().item()) < 1e-6
        dqkv = torch.zeros_like(qkv, device=dev)
        scratch = torch.zeros(B * Hq * T, device=dev)
        K.attention_backward(dqkv, scratch, dout.to(dev), out, lse, qkv.to(dev), Hq, Hkv)
        res.append((out, lse, dqkv))
    close(res[1][0], res[0][0], rtol=2e-2, atol=2e-2)
    close(res[1][1], res[0][1], rtol=1e-3, atol=1e-2)
    close(res[1][2], res[0][2], rtol=3e-2, atol=3e-2)


def test_qk_norm():
    torch.manual_seed(13)
    B, T, Hq, Hkv, HS = 2, 40, 4, 2, 64
    qkv = torch.randn(B, T, Hq + 2 * Hkv, HS).to(BF)
    dout = torch.randn_like(qkv.float()).to(BF)
    qw, kw = (1 + 0.1 * torch.randn(HS)).to(BF), (1 + 0.1 * torch.randn(HS)).to(BF)
    res = []
    for dev in ("cpu", DEV):
        out = qkv.clone().to(dev)
        rstd = torch.zeros(B * T, Hq + Hkv, device=dev)
        K.qk_norm_forward(out, rstd, qkv.to(dev), qw.to(dev), kw.to(dev), 1e-6, Hq, Hkv)
        dqkv = torch.zeros_like(out)
        dqw, dkw = torch.zeros(HS, dtype=BF, device=dev), torch.zeros(HS, dtype=BF, device=dev)
        K.qk_norm_backward(dqkv, dqw, dkw, torch.zeros(128 * 2 * HS, device=dev), dout.to(dev), qkv.to(dev), qw.to(dev), kw.to(dev), rstd, Hq, Hkv)
        res.append((out, rstd, dqkv, dqw, dkw))
    for g, r in zip(res[1], res[0]):
        close(g, r, rtol=2e-2, atol=2e-2)
    assert torch.equal(res[1][0][:, :, Hq + Hkv:].cpu(), qkv[:, :, Hq + Hkv:])


def test_native_unit_tests():
    """The C++ test executable (kernels against host references, no Python in between) passes."""
    import subprocess
    from llmq_b200.build import build_tests
    exe = build_tests()
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ALL TESTS PASSED" in r.stdout, r.stdout + r.stderr


def test_guard_zones_catch_a_write_past_the_end():
    """The guard tooling itself: a write one element past a guarded tensor is reported, writes inside are not."""
    from llmq_b200.utils.guards import GuardedAllocator

    ga = GuardedAllocator(DEV)
    a = ga.empty((33, 7), BF, "a")
    b = ga.empty((5,), torch.float32, "b", fill=0.0)
    a.fill_(1.0)
    b.add_(2.0)
    assert ga.check() == []
    # the raw storage continues behind the view: address the first guard byte after `b` through an overlapping view
    over = torch.as_strided(b, (6,), (1,))
    over[5] = 3.0
    msgs = ga.check()
    assert len(msgs) == 1 and msgs[0].startswith("b ") and "after the buffer" in msgs[0] and "+0" in msgs[0]
