"""Clipping entry points of the DP-FTRL namespace (packages/opake-dpftrl/src/opake/dpftrl/clipping/__init__.py): the
same transforms as DP-SGD; DP-FTRL changes the noise, not the clipping."""
from ..dpsgd.clipping import auto_clipped_grad, clipped_grad, per_group

__all__ = ["auto_clipped_grad", "clipped_grad", "per_group"]
