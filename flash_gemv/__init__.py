"""Drop-in ``flash_gemv`` package: the reference's operator names served by ``cats_b200``.

``import flash_gemv`` is what the reference's model code and scripts do
(experiments/models/sparse_silu/ugly_utils.py:27; flash_gemv/test, flash_gemv/bench); this alias
re-exports the same public names (flash_gemv/flash_gemv/__init__.py:62-80) and registers
``torch.ops.flash_gemv.*``.
"""
from cats_b200.flash_gemv import *  # noqa: F401,F403
from cats_b200.flash_gemv import __all__ as _names, register_torch_ops

__version__ = "0.0.1"
__all__ = list(_names)
register_torch_ops()
