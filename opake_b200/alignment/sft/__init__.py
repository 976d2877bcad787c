"""``alignment.sft``: NLL / DFT losses and the language-modelling collator."""
from . import collator, loss
from .collator import language_modeling_collator
from .loss import dft_loss, fused_dft_loss, fused_nll_loss, nll_loss

__all__ = ["collator", "loss", "nll_loss", "fused_nll_loss", "dft_loss", "fused_dft_loss", "language_modeling_collator"]
