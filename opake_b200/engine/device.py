"""Device capability probes (packages/opake-engine/src/opake/api/engine/device/_capabilities.py:70-198).

``fused_kernels_available()`` means: a CUDA device of compute capability 10.x is present and the in-tree sm_100a
kernel library loads. There is no Triton or multi-backend dispatch in this build.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache

import torch


@dataclass(frozen=True)
class DeviceCapabilities:
    device_type: str
    name: str = ""
    compute_capability: tuple[int, int] | None = None
    total_memory_gb: float = 0.0
    num_sms: int = 0
    bf16: bool = False
    fused_kernels: bool = False
    cuda_graphs: bool = False
    peer_access: bool = False


@lru_cache(maxsize=1)
def fused_kernels_available() -> bool:
    if not torch.cuda.is_available():
        return False
    if torch.cuda.get_device_capability(0)[0] != 10:
        return False
    try:
        from ..ops import _lib

        _lib.lib()
        return True
    except Exception:
        return False


def device_capabilities(device: torch.device | str | None = None) -> DeviceCapabilities:
    dev = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    if dev.type != "cuda":
        return DeviceCapabilities(dev.type, bf16=True)
    p = torch.cuda.get_device_properties(dev)
    return DeviceCapabilities("cuda", p.name, (p.major, p.minor), p.total_memory / 2**30, p.multi_processor_count,
                              bf16=True, fused_kernels=fused_kernels_available(), cuda_graphs=True,
                              peer_access=torch.cuda.device_count() > 1)


def sdpa_autocast_under_vmap_broken() -> bool:
    """MPS-only quirk in the reference; never true on CUDA or CPU."""
    return False


__all__ = ["DeviceCapabilities", "device_capabilities", "fused_kernels_available", "sdpa_autocast_under_vmap_broken"]
