"""Multi-rank launch modes on CPU: worker-process pool behind LLMQTrainer(ngpu=2), and rank threads with the
copy-based collectives.  Both must agree with a single rank on the combined batch; errors must propagate."""
import pytest
import torch

from llmq_b200.api import LLMQTrainer
from llmq_b200.config import create_config_from_name
from llmq_b200.options import LLamaOptions
from llmq_b200.parallel.threads import run_in_threads

B, T = 2, 32


def _tokens():
    g = torch.Generator().manual_seed(11)
    t = torch.randint(0, 512, (2, 2 * B, T + 1), generator=g, dtype=torch.int32)
    return t[:, :, :-1].contiguous(), t[:, :, 1:].contiguous()


def _single():
    cfg = create_config_from_name("tiny-qwen2", torch.float32)
    tr = LLMQTrainer(1, cfg, LLamaOptions(), batch_size=2 * B, seq_len=T, grad_accum=1, device="cpu")
    tr.init_weights(5)
    x, y = _tokens()
    out = []
    for s in range(2):
        tr.step(x[s], y[s])
        out.append(tr.update(1e-3, 0.9, 0.95, s + 1, 0.1, 1.0))
    return out


def test_worker_pool_matches_single_rank():
    ref = _single()
    cfg = create_config_from_name("tiny-qwen2", torch.float32)
    tr = LLMQTrainer(2, cfg, LLamaOptions(shard_gradients=True), batch_size=B, seq_len=T, grad_accum=1, device="cpu")
    try:
        tr.init_weights(5)
        x, y = _tokens()
        for s in range(2):
            tr.step(x[s].numpy(), y[s].numpy())
            r = tr.update(1e-3, 0.9, 0.95, s + 1, 0.1, 1.0)
            assert r["loss"] == pytest.approx(ref[s]["loss"], abs=2e-5) and r["norm"] == pytest.approx(ref[s]["norm"], rel=1e-4)
        loss, _ = tr.validate(x[0].numpy(), y[0].numpy())
        assert loss < ref[0]["loss"]
        grads = tr.get_gradients(1)
        assert "layers.0.qkv_w" in grads
        with pytest.raises(ValueError, match="rows of tokens"):
            tr.step(x[0][:B].numpy(), y[0][:B].numpy())
        with pytest.raises(RuntimeError, match="not a complete checkpoint"):
            tr.load_checkpoint("/nonexistent-dir", 1)            # every worker raises; the pool re-raises and shuts down
    finally:
        tr.close()


@pytest.mark.parametrize("kw", [dict(), dict(shard_weights=True, shard_gradients=True)], ids=["zero1", "zero3"])
def test_rank_threads_match_single_rank(kw):
    ref = _single()
    x, y = _tokens()

    def rank_main(comm):
        cfg = create_config_from_name("tiny-qwen2", torch.float32)
        tr = LLMQTrainer(2, cfg, LLamaOptions(**kw), batch_size=B, seq_len=T, grad_accum=1)
        tr.init_weights(5)
        out = []
        for s in range(2):
            tr.step(x[s], y[s])                                  # global arrays: each rank takes its rows
            out.append(tr.update(1e-3, 0.9, 0.95, s + 1, 0.1, 1.0))
        return out

    res = run_in_threads(2, rank_main, devices=[torch.device("cpu")] * 2, timeout=60)
    for rank_out in res:
        for r, want in zip(rank_out, ref):
            assert r["loss"] == pytest.approx(want["loss"], abs=2e-5) and r["norm"] == pytest.approx(want["norm"], rel=1e-4)


def test_rank_thread_failure_reaches_launcher_and_peers():
    seen = {}

    def rank_main(comm):
        if comm.rank == 1:
            raise ValueError("rank 1 lost its data")
        try:
            comm.barrier()
        except RuntimeError as e:
            seen["peer"] = str(e)
            raise

    with pytest.raises(ValueError, match="rank 1 lost its data"):
        run_in_threads(2, rank_main, devices=[torch.device("cpu")] * 2, timeout=20)
    assert "peer rank failed" in seen["peer"]
