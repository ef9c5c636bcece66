"""ramtorch_b200 — the optimizer-step path of RamTorch, rebuilt for B200 (sm_100a).

Public surface (same names as the reference package, ramtorch/__init__.py:1-4 and its
``zero1`` / ``zero2`` modules):

    from ramtorch_b200 import AdamW
    from ramtorch_b200.zero1 import create_zero_param_groups, broadcast_zero_params
    from ramtorch_b200.zero2 import setup_grad_sharding_hooks

The arithmetic runs in ``librt_b200.so`` (hand-written CUDA behind the C ABI declared in
``include/rt_b200.h``).  There is no CPU implementation.
"""
from . import helpers, stochastic_optimizers, zero1, zero2
from .stochastic_optimizers.adamw import AdamW, copy_stochastic_

__all__ = ["AdamW", "copy_stochastic_"]
__version__ = "0.1.0"
