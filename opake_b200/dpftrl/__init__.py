"""DP-FTRL: correlated-noise (matrix-factorisation) mechanisms, their samplers and accounting
(packages/opake-dpftrl/src/opake/dpftrl/__init__.py)."""
from . import clipping, noise, sampling, strategies  # noqa: F401
from .clipping import auto_clipped_grad, clipped_grad, per_group  # noqa: F401
from .noise import mf_gaussian_noise  # noqa: F401
from .sampling import BallsInBinsSampler, BMinSepSampler, CyclicPoissonSampler, SequentialBatchSampler  # noqa: F401
from .strategies import (band_mf_strategy, bisr_strategy, blt_strategy, bsr_strategy, identity_strategy,  # noqa: F401
                         lambda_cgd_strategy)

__all__ = ["accounting", "clipping", "noise", "sampling", "clipped_grad", "auto_clipped_grad", "per_group", "mf_gaussian_noise",
           "band_mf_strategy", "bisr_strategy", "bsr_strategy", "blt_strategy", "identity_strategy", "lambda_cgd_strategy",
           "BallsInBinsSampler", "BMinSepSampler", "CyclicPoissonSampler", "SequentialBatchSampler"]


def __getattr__(name):
    if name == "accounting":
        import importlib

        return importlib.import_module(".accounting", __name__)
    raise AttributeError(name)
