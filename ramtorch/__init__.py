"""Alias package: the reference's import paths (``ramtorch``, ``ramtorch.zero1``, ``ramtorch.zero2``,
``ramtorch.helpers``, ``ramtorch.stochastic_optimizers``) served by ``ramtorch_b200``.

Only the optimizer-step path is provided; ``ramtorch.Linear`` is not part of this package.
"""
import sys as _sys

import ramtorch_b200 as _impl
from ramtorch_b200 import AdamW, copy_stochastic_, helpers, stochastic_optimizers, zero1, zero2

for _name, _mod in (("zero1", zero1), ("zero2", zero2), ("helpers", helpers),
                    ("stochastic_optimizers", stochastic_optimizers),
                    ("stochastic_optimizers.adamw", stochastic_optimizers.adamw)):
    _sys.modules[__name__ + "." + _name] = _mod

__all__ = ["AdamW", "copy_stochastic_"]
__version__ = _impl.__version__


def __getattr__(name):
    if name == "Linear":
        raise AttributeError("ramtorch.Linear (the CPU-bouncing linear layer) is outside this package: "
                             "only the optimizer-step path is implemented")
    raise AttributeError(name)
