"""Guard-banded buffers (``opake_b200.utils.canary``) on CPU tensors."""
import pytest
import torch

from opake_b200.utils import CanaryPool, DeviceIntegrityError


def test_canary_pool_detects_writes_on_both_sides_and_repairs():
    pool = CanaryPool("cpu")
    a = pool.empty(5, 7, dtype=torch.bfloat16, name="a")
    b = pool.zeros(3, dtype=torch.float32, name="b")
    c = pool.empty((2, 2), dtype=torch.float64, name="c")
    assert a.shape == (5, 7) and b.shape == (3,) and c.shape == (2, 2) and len(pool) == 3
    assert a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0
    a.fill_(1.0)
    b.fill_(2.0)
    c.fill_(3.0)
    assert pool.check() == []
    pool.assert_intact()
    # one byte past ``b`` (12 payload bytes; the rounding slack up to 16 belongs to the trailing band)
    pool._raw[1][256 + 12] = 0
    # one byte before ``c``
    pool._raw[2][255] = 7
    bad = pool.check()
    assert [(v.name, v.side, v.offset, v.value) for v in bad] == [("b", "after", 0, 0), ("c", "before", 255, 7)]
    with pytest.raises(DeviceIntegrityError, match="b: after the buffer"):
        pool.assert_intact()
    pool.repair()
    assert pool.check() == []
    assert float(b.sum()) == 6.0 and float(c.sum()) == 12.0           # payloads untouched by the repair
