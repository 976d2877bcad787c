"""DP-FTRL: correlated-noise (matrix-factorisation) mechanisms, their samplers and accounting."""
from . import noise, sampling, strategies  # noqa: F401
from .noise import mf_gaussian_noise  # noqa: F401
from .strategies import (band_mf_strategy, bisr_strategy, blt_strategy, bsr_strategy, identity_strategy,  # noqa: F401
                         lambda_cgd_strategy)


def __getattr__(name):
    if name == "accounting":
        import importlib

        return importlib.import_module(".accounting", __name__)
    raise AttributeError(name)
