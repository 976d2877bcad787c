"""DP-SGD: clipping variants, the Gaussian mechanism, privacy samplers and their accounting (lazy import)."""
from . import clipping, noise, sampling  # noqa: F401
from .clipping import adaptive_clipped_grad, auto_clipped_grad, clipped_grad, per_group  # noqa: F401
from .noise import gaussian_noise  # noqa: F401
from .sampling import PoissonSampler  # noqa: F401


def __getattr__(name):
    if name == "accounting":
        import importlib

        return importlib.import_module(".accounting", __name__)
    raise AttributeError(name)
