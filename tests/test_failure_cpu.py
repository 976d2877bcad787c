"""Failure detection with host-side injection only: gloo ranks on the CPU that raise, exit or stop their heartbeat."""
import datetime
import os
import sys
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.distributed


def _init(rank, world, port, timeout=8):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout))


def _barrier_worker(rank, world, port, q):
    from opake_b200.base.exceptions import CheckpointError
    from opake_b200.transformers.distributed import checkpoint_barrier
    _init(rank, world, port)
    try:
        checkpoint_barrier(failed=(rank == 1), what="unit test")
        q.put((rank, "passed"))
    except CheckpointError as e:
        q.put((rank, "raised:" + str(e)))
    checkpoint_barrier(False)        # the group is still usable afterwards
    dist.destroy_process_group()


def _heartbeat_worker(rank, world, port, q):
    from opake_b200.parallel.health import Heartbeat, PeerFailure, guarded_step
    _init(rank, world, port, timeout=5)
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval=0.2).start()
    dist.barrier()
    if rank == 1:
        hb.stop()                    # simulated hang: the process lives on but stops beating and never joins again
        time.sleep(4.0)
        q.put((rank, "silent"))
        return
    time.sleep(1.5)
    try:
        guarded_step(lambda: dist.all_reduce(torch.ones(1)), hb, max_age=1.0)
        q.put((rank, "ran"))
    except PeerFailure as e:
        q.put((rank, f"peer-failure:{e.ranks}"))


def _exit_worker(rank, world, port, q):
    from opake_b200.parallel.health import Heartbeat
    _init(rank, world, port, timeout=4)
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval=0.2).start()
    t = torch.ones(1)
    dist.all_reduce(t)               # step 0 completes everywhere
    if rank == 1:
        hb.leave()                   # clean departure between steps, nothing in flight
        q.put((rank, "left"))
        return
    time.sleep(0.8)
    q.put((rank, f"state:{hb.peer_state(1)[0]};missing:{hb.missing_peers(5.0)}"))


def _run(fn, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() + int(time.time())) % 300
    procs = [ctx.Process(target=fn, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    deadline = time.time() + 60
    while len(out) < world and time.time() < deadline:
        try:
            r, msg = q.get(timeout=1.0)
            out[r] = msg
        except Exception:
            pass
    for p in procs:
        p.join(timeout=10)
        if p.is_alive():
            p.kill()             # exact child process handle
    return out


def test_checkpoint_barrier_propagates_failure_to_all_ranks():
    out = _run(_barrier_worker)
    assert out[0].startswith("raised:") and out[1].startswith("raised:") and "this one" in out[1]


def test_heartbeat_detects_silent_rank_before_launching():
    out = _run(_heartbeat_worker)
    assert out[0] == "peer-failure:[1]" and out[1] == "silent"


def test_clean_departure_is_seen_as_left():
    out = _run(_exit_worker)
    assert out[1] == "left" and out[0] == "state:left;missing:[1]"


# ---------------------------------------------------------------------------------------------- expert parallelism
def _ep_worker(rank, world, port, q):
    import torch.nn.functional as F
    from opake_b200.parallel.expert_parallel import ExpertParallelLayer
    _init(rank, world, port, timeout=30)
    torch.manual_seed(0)
    E, k, d, I, T = 4, 2, 8, 6, 20
    router = torch.randn(E, d, dtype=torch.float64) * 0.5
    wgu = torch.randn(E, 2 * I, d, dtype=torch.float64) * 0.3
    wd = torch.randn(E, d, I, dtype=torch.float64) * 0.3
    xs = [torch.randn(T, d, dtype=torch.float64, generator=torch.Generator().manual_seed(10 + b)) for b in range(world)]
    dys = [torch.randn(T, d, dtype=torch.float64, generator=torch.Generator().manual_seed(20 + b)) for b in range(world)]
    El = E // world
    layer = ExpertParallelLayer(router, wgu[rank * El:(rank + 1) * El], wd[rank * El:(rank + 1) * El], k, norm_topk=True)
    y = layer.forward(xs[rank])
    dx, d_router, norms = layer.backward(dys[rank])
    scales = torch.tensor([0.5, 0.25], dtype=torch.float64)[:world]
    acc_gu, acc_d = torch.zeros(El, 2 * I, d, dtype=torch.float64), torch.zeros(El, d, I, dtype=torch.float64)
    layer.accumulate_clipped(scales, acc_gu, acc_d)

    # single-process reference with autograd, every expert local
    def ref(b):
        x = xs[b].clone().requires_grad_()
        r, g_, d_ = router.clone().requires_grad_(), wgu.clone().requires_grad_(), wd.clone().requires_grad_()
        probs = (x @ r.t()).softmax(-1)
        w, idx = torch.topk(probs, k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        gate = torch.zeros_like(probs).scatter(1, idx, w)
        gu = torch.einsum("td,efd->tef", x, g_)
        h = F.silu(gu[..., :I]) * gu[..., I:]
        out = (torch.einsum("tei,edi->ted", h, d_) * gate.unsqueeze(-1)).sum(1)
        (out * dys[b]).sum().backward()
        return out.detach(), x.grad, r.grad, g_.grad, d_.grad

    outs = [ref(b) for b in range(world)]
    mine = outs[rank]
    ok = {
        "y": torch.allclose(y, mine[0], atol=1e-9), "dx": torch.allclose(dx, mine[1], atol=1e-9),
        "router": torch.allclose(d_router, mine[2], atol=1e-9),
        "norms": all(abs(norms[b].item() - (outs[b][3][rank * El:(rank + 1) * El].pow(2).sum()
                                            + outs[b][4][rank * El:(rank + 1) * El].pow(2).sum()).item()) < 1e-8 for b in range(world)),
        "acc_gu": torch.allclose(acc_gu, sum(scales[b] * outs[b][3][rank * El:(rank + 1) * El] for b in range(world)), atol=1e-9),
        "acc_d": torch.allclose(acc_d, sum(scales[b] * outs[b][4][rank * El:(rank + 1) * El] for b in range(world)), atol=1e-9),
    }
    q.put((rank, ",".join(k_ for k_, v in ok.items() if not v) or "ok"))
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_two_pass_clipping_matches_single_process():
    out = _run(_ep_worker)
    assert out == {0: "ok", 1: "ok"}, out


def _aux_sync_worker(rank, world, port, q):
    _init(rank, world, port)
    from opake_b200.dpsgd import clipped_grad  # noqa: F401  (registers the sync handlers)
    from opake_b200.engine import distributed as D
    from opake_b200.engine.clipping.core import ClippedGradAux, ClippingStats, FixedClipState
    from opake_b200.engine.clipping.distributed import sync_clip_state, sync_clipping_rate

    b = 3 + rank                                       # ranks hold different numbers of examples
    base = 10.0 * rank
    aux = ClippedGradAux(loss_values=torch.arange(b, dtype=torch.float32) + base, grad_norms=torch.full((b,), 2.0 + rank),
                         clipped_grad_norms=torch.ones(b), loss_aux={"logits": torch.arange(b * 2, dtype=torch.float32).view(b, 2) + base},
                         clipping_rate=1.0 if rank == 0 else 0.5, batch_size=b)
    got = D.sync(aux)
    stats = D.sync(ClippingStats(num_clipped=float(rank + 1), clipping_rate=None, batch_size=b))
    c, n, r = sync_clipping_rate({"a": 1.0 + rank, "b": 0.0}, b)
    assert sync_clip_state(FixedClipState()) == FixedClipState()
    q.put((rank, (got.loss_values.tolist(), got.grad_norms.tolist(), got.loss_aux["logits"].shape, got.batch_size, got.clipping_rate,
                  stats.num_clipped, stats.batch_size, stats.clipping_rate, c, n, r)))
    dist.barrier()
    dist.destroy_process_group()


def test_clipping_aux_and_statistics_are_gathered_over_ranks():
    out = _run(_aux_sync_worker)
    assert out[0] == out[1]                                                   # every rank ends with the same global view
    losses, norms, shape, b, rate, nclip, nb, srate, c, n, r = out[0]
    assert losses == [0.0, 1.0, 2.0, 10.0, 11.0, 12.0, 13.0] and norms == [2.0] * 3 + [3.0] * 4
    assert tuple(shape) == (7, 2) and b == 7 and rate == pytest.approx((3 * 1.0 + 4 * 0.5) / 7)
    assert (nclip, nb) == (3.0, 7) and srate == pytest.approx(3 / 7)
    assert c == {"a": 3.0, "b": 0.0} and n == 7 and r["a"] == pytest.approx(3 / 7)
