"""Guard-banded ("canary") buffers for the native runtime's workspaces.

``compute-sanitizer``-style tooling is not always available where the kernels run, so the runtime can allocate its
workspaces through a :class:`CanaryPool`: every buffer sits between two guard bands filled with a fixed byte pattern,
and :meth:`CanaryPool.check` verifies, with ONE device-to-host transfer for the whole pool, that no kernel wrote
outside the buffer it was given. A violation names the buffer, the side and the first damaged byte. The bands are 256
bytes, so the payload keeps the 256-byte alignment of the allocation (TMA operands need 16).

The reference has no race or bounds tooling for its kernels (spin locks in its Triton kernels, packages/opake-patches/
src/opake/api/patches/kernels/_utils.py:238-257, without a checker).
"""
from __future__ import annotations

import dataclasses
import math

import torch

__all__ = ["CanaryPool", "CanaryViolation", "DeviceIntegrityError"]

GUARD_BYTES = 256
PATTERN = 0xA5


class DeviceIntegrityError(RuntimeError):
    """A kernel wrote outside a buffer of a canary pool."""


@dataclasses.dataclass(frozen=True)
class CanaryViolation:
    name: str
    side: str            # "before" | "after"
    offset: int          # byte offset of the first damaged guard byte, relative to the band's start
    value: int


class CanaryPool:
    def __init__(self, device: torch.device | str):
        self.device = torch.device(device)
        self._raw: list[torch.Tensor] = []
        self._meta: list[tuple[str, int]] = []        # (name, payload bytes rounded up to 16)

    def __len__(self) -> int:
        return len(self._raw)

    def empty(self, *shape: int, dtype: torch.dtype = torch.bfloat16, name: str | None = None) -> torch.Tensor:
        if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
            shape = tuple(shape[0])
        itemsize = torch.empty((), dtype=dtype).element_size()
        nbytes = int(math.prod(shape)) * itemsize
        padded = (nbytes + 15) // 16 * 16
        raw = torch.empty(GUARD_BYTES + padded + GUARD_BYTES, dtype=torch.uint8, device=self.device)
        raw[:GUARD_BYTES].fill_(PATTERN)
        raw[GUARD_BYTES + nbytes:].fill_(PATTERN)       # the rounding slack belongs to the trailing band
        self._raw.append(raw)
        self._meta.append((name or f"buffer{len(self._raw) - 1}", nbytes))
        return raw[GUARD_BYTES : GUARD_BYTES + nbytes].view(dtype).view(*shape)

    def zeros(self, *shape: int, dtype: torch.dtype = torch.bfloat16, name: str | None = None) -> torch.Tensor:
        return self.empty(*shape, dtype=dtype, name=name).zero_()

    def check(self) -> list[CanaryViolation]:
        """All damaged guard bands (synchronises the device once)."""
        if not self._raw:
            return []
        bad = torch.stack([torch.stack(((r[:GUARD_BYTES] != PATTERN).any(), (r[GUARD_BYTES + n:] != PATTERN).any()))
                           for r, (_, n) in zip(self._raw, self._meta)]).cpu()
        out: list[CanaryViolation] = []
        for i in torch.nonzero(bad.any(dim=1)).flatten().tolist():
            r, (name, n) = self._raw[i], self._meta[i]
            for side, band in (("before", r[:GUARD_BYTES]), ("after", r[GUARD_BYTES + n:])):
                diff = torch.nonzero(band != PATTERN).flatten()
                if diff.numel():
                    off = int(diff[0])
                    out.append(CanaryViolation(name, side, off, int(band[off])))
        return out

    def assert_intact(self) -> None:
        bad = self.check()
        if bad:
            lines = ", ".join(f"{v.name}: {v.side} the buffer, guard byte {v.offset} = 0x{v.value:02x}" for v in bad[:8])
            raise DeviceIntegrityError(f"{len(bad)} guard band(s) overwritten: {lines}")

    def repair(self) -> None:
        """Refill every guard band (after a reported violation, to keep checking later steps)."""
        for r, (_, n) in zip(self._raw, self._meta):
            r[:GUARD_BYTES].fill_(PATTERN)
            r[GUARD_BYTES + n:].fill_(PATTERN)
