"""Counterpart of the reference's tests/import_test.py: the package imports, carries a version, reports that its native
library is built and loadable, and exports the names of openequivariance/openequivariance/__init__.py:35-116."""


def test_import_and_version():
    import openequivariance_b200 as oeq
    assert oeq.__version__ is not None and oeq.__version__ != "0.0.0"


def test_extension_built():
    from openequivariance_b200 import BUILT_EXTENSION, BUILT_EXTENSION_ERROR
    assert BUILT_EXTENSION_ERROR is None
    assert BUILT_EXTENSION


def test_public_names():
    import os

    import openequivariance_b200 as oeq
    for name in ("TPProblem", "Irreps", "TensorProduct", "TensorProductConv", "transpose_irreps", "torch_to_oeq_dtype",
                 "torch_ext_so_path", "CoordGraph", "LINKED_LIBPYTHON"):
        assert hasattr(oeq, name), name
    path = oeq.torch_ext_so_path()
    assert path is not None and os.path.exists(path)
