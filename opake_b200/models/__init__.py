"""Native model runtimes (explicit forward/backward on the sm_100a kernels) and architecture presets."""
