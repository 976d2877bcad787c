"""``torchopt.alias`` stand-in: ready-made optimizers assembled from the elementary transformations."""
from .utils import flip_sign_and_add_weight_decay, scale_by_neg_lr  # noqa: F401
