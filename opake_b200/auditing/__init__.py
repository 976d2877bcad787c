"""Empirical privacy auditing: coin-flipped canaries, membership scores, one-run lower bounds (counterpart of
``opake.auditing``, packages/opake-auditing/src/opake/auditing/__init__.py)."""
from . import attacks, one_run as _one_run_module
from .attacks import gradient_scores, loss_scores
from .coin_flip import CanaryScores, CoinFlip, canary_scores, coin_flip
from .one_run import EpsDeltaMethod, GdpMethod, OneRunEstimate, one_run

__all__ = ["attacks", "CanaryScores", "CoinFlip", "canary_scores", "coin_flip", "loss_scores", "gradient_scores",
           "one_run", "OneRunEstimate", "EpsDeltaMethod", "GdpMethod"]
