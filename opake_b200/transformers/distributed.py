"""Process-group glue of the trainer (packages/opake-transformers/src/opake/api/transformers/trainer/
_distributed.py:52-260): rank bookkeeping, backend validation, automatic ``init_process_group`` under a launcher,
and a barrier that propagates failure (if any rank reports an error every rank raises, so nobody waits forever on a
collective that a failed rank will never join)."""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass

import torch

from ..base.exceptions import CheckpointError, ConfigurationError
from ..engine import distributed as D

__all__ = ["DDPState", "resolve_ddp_state", "validate_ddp_backend", "checkpoint_barrier"]

_BACKENDS = ("nccl", "gloo", "mpi")


@dataclass(frozen=True)
class DDPState:
    rank: int = 0
    local_rank: int = 0
    world_size: int = 1
    backend: str | None = None
    initialised_here: bool = False

    @property
    def is_distributed(self) -> bool:
        return self.world_size > 1

    @property
    def is_main(self) -> bool:
        return self.rank == 0


def validate_ddp_backend(backend: str | None, device: torch.device) -> str:
    if backend is None:
        return "nccl" if device.type == "cuda" else "gloo"
    if backend not in _BACKENDS:
        raise ConfigurationError(f"ddp_backend must be one of {_BACKENDS}, got {backend!r}")
    if backend == "nccl" and device.type != "cuda":
        raise ConfigurationError("ddp_backend='nccl' needs CUDA devices; use 'gloo' on CPU")
    if backend == "mpi" and not torch.distributed.is_mpi_available():
        raise ConfigurationError("ddp_backend='mpi' requested but this PyTorch build has no MPI support")
    return backend


def resolve_ddp_state(backend: str | None, device: torch.device, timeout_s: int = 1800) -> DDPState:
    """Existing process group -> describe it; ``WORLD_SIZE > 1`` in the environment -> create one; else single."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        return DDPState(dist.get_rank(), int(os.environ.get("LOCAL_RANK", 0)), dist.get_world_size(), dist.get_backend(), False)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return DDPState()
    be = validate_ddp_backend(backend, device)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    kwargs = {}
    if be == "nccl":
        kwargs["device_id"] = device
    dist.init_process_group(backend=be, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return DDPState(dist.get_rank(), int(os.environ.get("LOCAL_RANK", 0)), dist.get_world_size(), be, True)


def checkpoint_barrier(failed: bool = False, *, what: str = "checkpoint", device: torch.device | None = None) -> None:
    """All ranks meet; if any passed ``failed=True`` all raise ``CheckpointError``."""
    if not D.is_distributed():
        if failed:
            raise CheckpointError(f"{what} failed on this process")
        return
    flag = int(D.reduce_scalar(int(bool(failed)), op="max", device=device))
    if flag:
        raise CheckpointError(f"{what} failed on at least one rank" + (" (this one)" if failed else ""))
