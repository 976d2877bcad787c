"""Host-side sizing rules of the sharded engine (no GPU needed)."""
import types

import torch

from opake_b200.parallel.engine import ShardedDPEngine


def _engine(dense_total: int, device_type: str = "cuda"):
    e = ShardedDPEngine.__new__(ShardedDPEngine)
    e.device = types.SimpleNamespace(type=device_type)
    e.layout = types.SimpleNamespace(dense_total=dense_total)
    return e


def test_accumulation_group_follows_free_memory(monkeypatch):
    """One gradient buffer of an 8B model is 16 GB: the group grows with the memory that sharding the optimizer state
    frees, never below 2, and a fixed reserve stays for activations."""
    gb = 1 << 30
    e = _engine(8 * gb)                                        # 8G bf16 values = 16 GB per buffer
    sizes = {}
    for free_gb in (40, 71, 103, 119, 127, 400):
        monkeypatch.setattr(torch.cuda, "mem_get_info", lambda dev=None, f=free_gb: (f * gb, 183 * gb))
        sizes[free_gb] = e._pick_group_size()
    assert sizes[40] == 2 and sizes[71] == 3                   # one GPU holding all optimizer state
    assert sizes[103] == 5 and sizes[119] == 6 and sizes[127] == 6
    assert sizes[400] == 6                                     # large models: never more than 6 automatically
    assert all(a <= b for a, b in zip(list(sizes.values()), list(sizes.values())[1:]))


def test_accumulation_group_override_and_cpu(monkeypatch):
    from opake_b200.parallel.engine import EngineConfig
    assert EngineConfig().accumulate_group == 0                # automatic unless the configuration names a size
    assert _engine(1000, "cpu")._pick_group_size() == 2
    # small models: the reserve scales with the model instead of the fixed 32 GB
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda dev=None: (64 << 30, 183 << 30))
    assert _engine(1 << 20)._pick_group_size() == 8


def test_consolidate_per_rank_shards_into_one_state():
    """The per-rank optimizer shards of a run concatenate, in flat-parameter order, into the state of a one-rank run."""
    total = 24
    params = torch.arange(total, dtype=torch.float32)
    bounds = [0, 8, 8, 24]            # one rank owns nothing (a model with fewer tensors than ranks)
    shards = []
    for r in range(3):
        b, e = bounds[r], bounds[r + 1]
        shards.append({"world": 3, "shard_begin": b, "shard_len": e - b, "m": params[b:e] * 2, "v": params[b:e] * 3, "master": None,
                       "blt_state": torch.stack([params[b:e], -params[b:e]]), "toep_state": None, "toep_pos": 1, "step_count": 5,
                       "phi": 0.25, "noise_key": {"seed": 1, "impl": "x"}, "params": params if r == 0 else None})
    full = ShardedDPEngine.consolidate([shards[2], shards[0], shards[1]])
    assert full["world"] == 1 and full["shard_len"] == total and full["step_count"] == 5
    assert torch.equal(full["m"], params * 2) and torch.equal(full["v"], params * 3)
    assert torch.equal(full["blt_state"], torch.stack([params, -params])) and full["master"] is None
    import pytest
    with pytest.raises(ValueError):
        ShardedDPEngine.consolidate(shards[:2])
