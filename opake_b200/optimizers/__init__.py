"""DP-aware optimizers as (init, update) gradient transformations."""
from . import chain as types  # noqa: F401
from .adam import AdamState, adam, adamw  # noqa: F401
from .chain import GradientTransformation, apply_updates, make_optimizer_chain  # noqa: F401
from .distributed import sync_optimizer_state  # noqa: F401
from .others import adadelta, adafactor, adagrad, ademamix, lion, radam, rmsprop, schedule_free, sgd  # noqa: F401
