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
