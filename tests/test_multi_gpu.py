"""1-rank vs 2-rank parity of the sharded DP engine (fused P2P reduce-scatter + noise + AdamW + all-gather)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world: int, out: str, extra=()):
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    if world == 1:
        cmd = [sys.executable, "-m", "tests.multi_gpu_selftest", "--out", out, *extra]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", "29533", "-m", "tests.multi_gpu_selftest", "--out", out,
               *extra]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return torch.load(out)


@pytest.mark.parametrize("blt", [False, True])
def test_two_ranks_match_one_rank(tmp_path, blt):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    extra = ("--blt",) if blt else ()
    one = _run(1, str(tmp_path / "w1.pt"), extra)
    two = _run(2, str(tmp_path / "w2.pt"), extra)
    assert one["losses"] == pytest.approx(two["losses"], rel=2e-3)
    diff = (one["params"] - two["params"]).abs().max().item()
    assert diff <= 2e-2 * one["params"].abs().max().item(), diff


@pytest.mark.parametrize("mode", ["params", "sums", "full", "full-graph"])
def test_two_ranks_fully_sharded_match_one_rank(tmp_path, mode):
    """Sharded parameters (fetched inside the forward GEMMs of the first example after each optimizer step) and sharded
    fp32 sums (accumulation groups reduce-scattered with reductions over NVLink) give the parameters of a 1-rank run.
    Sequences of 256 tokens so that the layer matrices take the staged two-CTA GEMM."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    extra = ["--seq", "256", "--steps", "3"]
    one = _run(1, str(tmp_path / "w1.pt"), extra)
    if mode in ("params", "full", "full-graph"):
        extra.append("--shard-params")
    if mode in ("sums", "full", "full-graph"):
        extra.append("--shard-sums")
    if mode == "full-graph":
        extra.append("--graph")
    two = _run(2, str(tmp_path / "w2.pt"), extra)
    if "--shard-params" in extra:
        assert len(two["staged"]) >= 2          # rank 0 pulled layer matrices it does not own inside their forward GEMMs
    assert one["losses"] == pytest.approx(two["losses"], rel=2e-3)
    diff = (one["params"] - two["params"]).abs().max().item()
    assert diff <= 2e-2 * one["params"].abs().max().item(), diff


def test_two_ranks_nccl_baseline_step_matches_one_rank(tmp_path):
    """The library-collective implementation of the optimizer step (reduce_scatter_tensor, local kernel,
    all_gather_into_tensor) gives the parameters of the fused peer-memory step."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    one = _run(1, str(tmp_path / "w1.pt"))
    two = _run(2, str(tmp_path / "w2.pt"), ("--comm", "nccl"))
    assert one["losses"] == pytest.approx(two["losses"], rel=2e-3)
    diff = (one["params"] - two["params"]).abs().max().item()
    assert diff <= 2e-2 * one["params"].abs().max().item(), diff


def test_two_ranks_match_one_rank_toeplitz(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    one = _run(1, str(tmp_path / "w1.pt"), ("--toeplitz", "--steps", "4"))
    two = _run(2, str(tmp_path / "w2.pt"), ("--toeplitz", "--steps", "4"))
    assert one["losses"] == pytest.approx(two["losses"], rel=2e-3)
    diff = (one["params"] - two["params"]).abs().max().item()
    assert diff <= 2e-2 * one["params"].abs().max().item(), diff


@pytest.mark.parametrize("graph", [False, True])
def test_expert_parallel_training_matches_local_experts(tmp_path, graph):
    """Two ranks with sharded experts (tokens exchanged over NVLink, per-example norms combined across ranks, clipped
    expert gradients formed in a second pass) train to the same losses and weights as one rank holding every expert.
    ``graph``: every example replayed from a CUDA graph on the two-rank side (exchange epochs relative to device-side
    counters); the one-rank side stays eager, so the two implementations are compared, not two replays."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    extra = ("--ep-train", "--steps", "3", "--batch", "8")
    one = _run(1, str(tmp_path / "w1.pt"), extra)
    two = _run(2, str(tmp_path / "w2.pt"), extra + (("--graph",) if graph else ()))
    assert one["clipped"] > 0 and two["clipped"] == one["clipped"]          # the clip factors were exercised
    assert one["losses"] == pytest.approx(two["losses"], rel=3e-3)
    for name in ("routers", "wgu", "wd", "wqkv"):
        assert torch.equal(one["init"][name], two["init"][name]), name         # same model however the experts are placed
        d1, d2 = one["delta"][name].flatten(), two["delta"][name].flatten()
        assert d1.abs().max().item() > 1e-3, name                              # the weights did move
        cos = torch.dot(d1, d2) / (d1.norm() * d2.norm())
        assert cos.item() > 0.98, (name, cos.item())                           # ... by the same update (bf16 storage rounding)
        assert abs(d1.norm().item() / d2.norm().item() - 1.0) < 0.05, name


def test_sharded_linear_reads_peer_shards(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    res = _run(2, str(tmp_path / "sl.pt"), ("--sharded-linear",))
    assert res["world"] == 2 and res["fwd_err"] < 2e-2 and res["dgrad_err"] < 2e-2


def test_expert_parallel_fused_two_ranks(tmp_path):
    """Dispatch / combine kernels over peer memory, grouped GEMMs and per-source norms against a dense fp32 oracle."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    res = _run(2, str(tmp_path / "ep.pt"), ("--ep-fused",))
    assert res["world"] == 2
    for name in ("out", "dx", "d_router", "acc_wgu", "acc_wd"):
        assert res[name] < 3e-2, (name, res)
    assert res["norms"] < 3e-2, res
