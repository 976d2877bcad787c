"""opake_b200 — functional differentially-private training (DP-SGD / DP-FTRL) built for NVIDIA B200.

The framework layer (pytrees, RngKey, clipping, noise mechanisms, samplers, optimizers, accountant, trainers)
is plain PyTorch/NumPy; the hot paths are hand-written sm_100a kernels in ``csrc/kernels`` reached through
``opake_b200.ops``.

Namespaces (loaded on first use, mirroring the ``opake.<name>`` façades of the reference): ``exceptions``,
``serialization``, ``types``, ``pytree``, ``random``, ``functional``, ``distributed``, ``profiling``, ``scheduling``,
``device``, ``dpsgd``, ``dpftrl``, ``accounting``, ``optimizers``, ``patches``, ``alignment``, ``auditing``,
``transformers``, ``models``, ``ops``, ``parallel``.
"""
import importlib

__version__ = "0.1.0"

_ALIASES = {
    "exceptions": "opake_b200.base.exceptions", "serialization": "opake_b200.base.serialization",
    "types": "opake_b200.engine.types", "pytree": "opake_b200.engine.pytree", "random": "opake_b200.engine.random",
    "functional": "opake_b200.engine.functional", "distributed": "opake_b200.engine.distributed",
    "profiling": "opake_b200.engine.profiling", "scheduling": "opake_b200.engine.scheduling",
    "device": "opake_b200.engine.device",
}
_PACKAGES = ("dpsgd", "dpftrl", "accounting", "optimizers", "patches", "alignment", "auditing", "transformers", "models",
             "ops", "parallel", "base", "engine")

__all__ = ["__version__", *_ALIASES, *_PACKAGES]


def __getattr__(name):
    if name in _ALIASES:
        mod = importlib.import_module(_ALIASES[name])
    elif name in _PACKAGES:
        mod = importlib.import_module(f"opake_b200.{name}")
    else:
        raise AttributeError(f"module 'opake_b200' has no attribute {name!r}")
    globals()[name] = mod
    return mod
