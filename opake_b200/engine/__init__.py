"""Layer 2: DP pytree types, RngKey, clipping core, functional models, distributed, profiling, schedules."""
from . import serialization as _tensor_codecs  # noqa: F401  (registers tensor / ndarray codecs)
from . import device, distributed, functional, noise_allocation, profiling, pytree, random, scheduling, types  # noqa: F401
