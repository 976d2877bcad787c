"""Process-group plumbing and peer-addressable ("symmetric") device buffers.

One process drives one GPU. ``torch.distributed`` (NCCL on GPUs, gloo on CPU ranks) does rank discovery, barriers
and small scalar reductions; large buffers that the fused kernels read or write on other GPUs (the fp32
clipped-gradient sums, the bf16 parameter replicas) are allocated from CUDA symmetric memory so that every rank
holds the device address of every peer's copy and kernels reach them with plain NVLink loads and stores.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


def init_distributed(backend: str | None = None, timeout_s: int = 1800) -> tuple[int, int, int]:
    """Initialises the default process group from the torchrun environment. Returns (rank, world, local_rank)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        import datetime

        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group(backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s),
                                    device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
    elif torch.cuda.is_available():
        torch.cuda.set_device(local)
    return rank, world, local


@dataclass
class PeerBuffer:
    """A tensor plus the device addresses of the same buffer on every rank (index = rank)."""

    local: torch.Tensor
    ptrs: list[int]
    handle: object | None = None

    def barrier(self) -> None:
        """Device-side barrier across the ranks sharing this buffer (stream-ordered, no host sync)."""
        if self.handle is not None:
            self.handle.barrier()

    def peer_view(self, rank: int, shape, dtype: torch.dtype | None = None, offset: int = 0) -> torch.Tensor:
        """A tensor aliasing rank ``rank``'s copy of the buffer (``offset`` in elements). Reads and writes through it
        are NVLink loads / stores; only this package's own kernels may be given such a tensor."""
        dtype = dtype or self.local.dtype
        if self.handle is None:
            if rank != 0:
                raise ValueError("single-rank buffer has no peers")
            n = 1
            for d in shape:
                n *= d
            return self.local.view(dtype)[offset:offset + n].view(*shape)
        return self.handle.get_buffer(rank, tuple(shape), dtype, offset)


def alloc_peer_buffer(numel: int, dtype: torch.dtype, device: torch.device, group=None) -> PeerBuffer:
    """Allocates ``numel`` elements that every rank of ``group`` can address.

    With one rank this is an ordinary allocation. With several it uses CUDA symmetric memory; if that is not
    available the caller must fall back to the NCCL path (``PeerBuffer.handle is None`` and one pointer).
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        t = torch.empty(numel, dtype=dtype, device=device)
        return PeerBuffer(t, [t.data_ptr()])
    import torch.distributed._symmetric_memory as symm

    t = symm.empty(numel, dtype=dtype, device=device)
    hdl = symm.rendezvous(t, group=group if group is not None else dist.group.WORLD)
    return PeerBuffer(t, [int(p) for p in hdl.buffer_ptrs], hdl)
