"""B200-native drop-in for the hot path of OpenEquivariance: ``TPProblem``, ``TensorProduct``,
``TensorProductConv`` and the ``libtorch_tp_jit::jit_*`` torch ops, backed by hand-written sm_100a kernels
behind a C ABI (``include/oeq_b200.h``).  Public surface follows openequivariance/openequivariance/__init__.py:35-116.
"""

import os

import numpy as np

from .core.irreps import Irrep, Irreps, _MulIr
from .core.problem import Instruction, TPProblem
from .core.graph import CoordGraph, prepare_graph
from .core.utils import torch_to_oeq_dtype

__version__ = "0.1.0"

# BUILT_EXTENSION / BUILT_EXTENSION_ERROR are resolved on first access (module __getattr__ below): the native library
# is loaded when something needs it, so a process that only uses the problem definitions never maps it.
# The reference reports whether its extension linked libpython; this library has no Python dependency.
LINKED_LIBPYTHON = False
LINKED_LIBPYTHON_ERROR = None

if os.environ.get("OEQ_NOTORCH") != "1":
    import torch

    from . import native
    from ._torch.TensorProduct import TensorProduct
    from ._torch.TensorProductConv import TensorProductConv
    from ._torch.layout import transpose_irreps

    torch.serialization.add_safe_globals(
        [TensorProduct, TensorProductConv, TPProblem, Irrep, Irreps, _MulIr, Instruction, np.float32, np.float64])


def __getattr__(name):
    if name in ("BUILT_EXTENSION", "BUILT_EXTENSION_ERROR"):
        from . import native as _n
        try:
            _n.load()
        except Exception:  # noqa: BLE001 - recorded in native.BUILT_EXTENSION_ERROR; every kernel call raises
            pass
        return getattr(_n, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def torch_ext_so_path():
    """Path of the shared library that implements the ops (``None`` when it has not been built)."""
    try:
        from . import native as _n
        return _n.LIB_PATH if os.path.exists(_n.LIB_PATH) else None
    except Exception:  # noqa: BLE001
        return None


__all__ = ["TPProblem", "Irreps", "Irrep", "TensorProduct", "TensorProductConv", "CoordGraph", "prepare_graph",
           "torch_to_oeq_dtype", "torch_ext_so_path", "transpose_irreps"]
