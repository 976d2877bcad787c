"""DPTrainer under two gloo ranks: sharded data, per-rank sampler streams, summed clipped gradients, identical noise,
identical parameters on every rank, rank-0 checkpoint files."""
import os
import time

import pytest
import torch
import torch.multiprocessing as mp
from torch import nn

pytestmark = pytest.mark.distributed


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.l1, self.l2 = nn.Linear(6, 8), nn.Linear(8, 2)

    def forward(self, x, labels=None):
        return {"logits": self.l2(torch.tanh(self.l1(x)))}


class _DS(torch.utils.data.Dataset):
    def __init__(self, n):
        g = torch.Generator().manual_seed(0)
        self.x = torch.randn(n, 6, generator=g)
        self.y = (self.x[:, 0] > 0).long()

    def __len__(self):
        return len(self.x)

    def __getitem__(self, i):
        return {"x": self.x[i], "labels": self.y[i]}


def _worker(rank, world, port, out_dir, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    from opake_b200.transformers import DPTrainer, TrainingArguments
    torch.manual_seed(0)
    args = TrainingArguments(output_dir=out_dir, per_device_train_batch_size=16, max_steps=4, learning_rate=0.05, optim="adamw-bc",
                             privacy_noise_multiplier=1.0, logging_steps=2, save_steps=4, use_cpu=True, ddp_backend="gloo",
                             use_compat_patches=False)
    tr = DPTrainer(_Net(), args, train_dataset=_DS(256))
    out = tr.train()
    flat = torch.cat([p.detach().reshape(-1) for p in tr.model.parameters()])
    q.put((rank, flat.tolist(), out.global_step, tr.ddp.world_size, tr._rt["sample_rate"], out.metrics.get("privacy_epsilon")))
    import torch.distributed as dist
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_training_keeps_replicas_identical(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + (os.getpid() + int(time.time())) % 90
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path), q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    deadline = time.time() + 240
    while len(got) < 2 and time.time() < deadline:
        try:
            item = q.get(timeout=1.0)
            got[item[0]] = item[1:]
        except Exception:
            pass
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.kill()
    assert set(got) == {0, 1}
    assert got[0][0] == got[1][0]                               # bitwise identical parameters
    assert got[0][1] == 4 and got[0][2] == 2
    assert got[0][3] == pytest.approx(32 / 256)                 # global batch over global dataset
    assert got[0][4] == pytest.approx(got[1][4]) and got[0][4] > 0
    assert sorted(os.listdir(tmp_path)) == ["checkpoint-4"]
