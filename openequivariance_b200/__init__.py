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

BUILT_EXTENSION = False
BUILT_EXTENSION_ERROR = None
# The reference reports whether its extension linked libpython; this library has no Python dependency.
LINKED_LIBPYTHON = False
LINKED_LIBPYTHON_ERROR = None

if os.environ.get("OEQ_NOTORCH") != "1":
    import torch

    from . import native
    from ._torch.TensorProduct import TensorProduct
    from ._torch.TensorProductConv import TensorProductConv
    from ._torch.layout import transpose_irreps

    try:
        native.load()
        BUILT_EXTENSION, BUILT_EXTENSION_ERROR = True, None
    except Exception as _exc:  # noqa: BLE001 - recorded; every kernel call will raise
        BUILT_EXTENSION, BUILT_EXTENSION_ERROR = False, _exc

    torch.serialization.add_safe_globals(
        [TensorProduct, TensorProductConv, TPProblem, Irrep, Irreps, _MulIr, Instruction, np.float32, np.float64])


def torch_ext_so_path():
    """Path of the shared library that implements the ops (``None`` when it has not been built)."""
    try:
        from . import native as _n
        return _n.LIB_PATH if os.path.exists(_n.LIB_PATH) else None
    except Exception:  # noqa: BLE001
        return None


__all__ = ["TPProblem", "Irreps", "Irrep", "TensorProduct", "TensorProductConv", "CoordGraph", "prepare_graph",
           "torch_to_oeq_dtype", "torch_ext_so_path", "transpose_irreps"]
