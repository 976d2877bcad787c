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


def _resume_worker(rank, world, port, out_dir, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    from opake_b200.transformers import DPTrainer, TrainingArguments

    def make(sub, **kw):
        torch.manual_seed(0)
        args = TrainingArguments(output_dir=os.path.join(out_dir, sub), per_device_train_batch_size=16, max_steps=4, learning_rate=0.05,
                                 optim="adamw-bc", privacy_noise_multiplier=1.0, logging_steps=2, save_steps=2, use_cpu=True,
                                 ddp_backend="gloo", use_compat_patches=False, **kw)
        return DPTrainer(_Net(), args, train_dataset=_DS(257))      # 257: the two shards differ in length (128 / 129)

    def flat(tr):
        return torch.cat([p.detach().reshape(-1) for p in tr.model.parameters()]).tolist()

    full = make("run")
    full.train()
    want = flat(full)
    seed_full = int(full._rt["sampler"]._stream_key.seed)
    # resume from the step-2 checkpoint of the same run: every rank must continue ITS OWN stream, so the result is bitwise the same
    again = make("run")
    again.train(resume_from_checkpoint=os.path.join(out_dir, "run", "checkpoint-2"))
    got = flat(again)
    seed_resumed = int(again._rt["sampler"]._stream_key.seed)
    # ignore_data_skip: a fresh stream, installed in the sampler object the data loader iterates, rank-folded
    skip = make("run", ignore_data_skip=True)
    skip.train(resume_from_checkpoint=os.path.join(out_dir, "run", "checkpoint-2"))
    loader_sampler = skip.callback_handler.train_dataloader.batch_sampler
    q.put((rank, want == got, seed_full, seed_resumed, int(loader_sampler._stream_key.seed), loader_sampler is skip._rt["sampler"],
           flat(skip) != want, int(loader_sampler.consumed)))
    import torch.distributed as dist
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_resume_keeps_rank_local_sampler_streams(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() + int(time.time())) % 90
    procs = [ctx.Process(target=_resume_worker, args=(r, 2, port, str(tmp_path), q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    deadline = time.time() + 300
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
    for r in (0, 1):
        same, seed_full, seed_resumed, seed_skip, is_loader_sampler, differs, consumed = got[r]
        assert same, f"rank {r}: resumed run differs from the uninterrupted one"
        assert seed_full == seed_resumed                         # the rank's own stream key survives the resume
        assert seed_skip != seed_full and is_loader_sampler      # ignore_data_skip: fresh key, in the iterated sampler
        assert differs and consumed == 2                         # fresh stream drawn from its start for the 2 remaining steps
    assert got[0][1] != got[1][1]                                # ranks never share coins: before the checkpoint,
    assert got[0][2] != got[1][2]                                # after a resume,
    assert got[0][3] != got[1][3]                                # and on the fresh ignore_data_skip stream
