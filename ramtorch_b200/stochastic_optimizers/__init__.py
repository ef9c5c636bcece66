from .adamw import AdamW, copy_stochastic_

__all__ = ["AdamW", "copy_stochastic_"]
