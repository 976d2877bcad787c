"""Layer 2: DP pytree types, RngKey, clipping core, functional models, distributed, profiling, schedules."""
