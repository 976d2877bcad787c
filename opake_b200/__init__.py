"""opake_b200 — functional differentially-private training (DP-SGD / DP-FTRL) built for NVIDIA B200.

The framework layer (pytrees, RngKey, clipping, noise mechanisms, samplers, optimizers, accountant, trainers)
is plain PyTorch/NumPy; the hot paths are hand-written sm_100a kernels in ``csrc/kernels`` reached through
``opake_b200.ops``.
"""
__version__ = "0.1.0"
