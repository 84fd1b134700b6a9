"""CPU-side checks of the native boundary: the library loads, exports every declared symbol, parses and rejects
descriptors, and specialises + compiles its kernels for sm_100a without a GPU."""
import os
import re

import numpy as np
import pytest

from helpers import ROOT, tp_problem_matrix, with_dtype
from openequivariance_b200 import native
from openequivariance_b200.core import problems as P
from openequivariance_b200.core.descriptor import build_descriptor, descriptor_hash


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "oeq_b200.h")).read()
    declared = sorted(set(re.findall(r"OEQB_API [a-z0-9_ \*]+?(oeqb_[a-z_]+)\(", header)))
    assert declared == native.exported_symbols()
    lib = native.load()
    for name in declared:
        assert getattr(lib, name) is not None
    assert b"sm_100a" in lib.oeqb_version()


def test_descriptor_roundtrip_and_query():
    p = P.mace_like_problem()
    text = build_descriptor(p, conv=True, deterministic=True)
    prop = native.query(text.encode(), descriptor_hash(text))
    assert (prop.L1_dim, prop.L2_dim, prop.L3_dim, prop.weight_numel) == (2048, 16, 12672, 2944)
    assert prop.shared_weights == 0 and prop.irrep_dtype == 1 and prop.idx_dtype == 4
    assert prop.is_conv == 1 and prop.deterministic == 1 and prop.is_uvw == 0 and prop.fast_path == 1
    q = P.nequip_like_problem(np.float64)
    text = build_descriptor(q)
    prop = native.query(text.encode(), descriptor_hash(text))
    assert (prop.L1_dim, prop.L3_dim, prop.weight_numel, prop.shared_weights) == (576, 576, 30720, 1)
    assert prop.irrep_dtype == 2 and prop.is_uvw == 1 and prop.fast_path == 0


@pytest.mark.parametrize("mangle", ["header", "truncate", "index", "wn"])
def test_malformed_descriptor_is_rejected(mangle):
    text = build_descriptor(P.readme_problem())
    if mangle == "header":
        bad = text.replace("OEQB 1", "OEQB 9")
    elif mangle == "truncate":
        bad = text[: len(text) // 2]
    elif mangle == "index":
        bad = text.replace("I 0 0 0 0", "I 0 3 0 0")
    else:
        bad = text.replace("wn 1", "wn 2")
    with pytest.raises(RuntimeError, match="descriptor"):
        native.query(bad.encode(), 7_000_000 + hash(mangle) % 1000)


def test_unsupported_problems_fail_at_construction():
    from openequivariance_b200.core.problem import TPProblem
    with pytest.raises(AssertionError, match="layout='ir_mul'"):
        build_descriptor(TPProblem("5x5e", "1x3e", "5x5e", [(0, 0, 0, "uvw", True)], shared_weights=False,
                                   internal_weights=False, layout="ir_mul"))
    with pytest.raises(AssertionError, match="same connection mode"):
        build_descriptor(TPProblem("2x1e", "2x1e", "2x1e", [(0, 0, 0, "uvw", True), (0, 0, 0, "uvu", True)],
                                   shared_weights=False, internal_weights=False))
    with pytest.raises(AssertionError, match="trainable weights"):
        build_descriptor(TPProblem("2x1e", "2x1e", "2x1e", [(0, 0, 0, "uvu", False)], shared_weights=False,
                                   internal_weights=False))


def test_emitted_source_is_specialised():
    text = build_descriptor(P.readme_problem())
    src = native.emit_source(text.encode(), "generic")
    assert "struct Ins<0>" in src and "oeq_generic_forward" in src and "L3_DIM = 5" in src


_BIG = {"mace_like", "mace_medium", "nequip_like", "diffdock1", "tetris_poly2", "nequip_water_uvu", "ctpp_ir_mul",
        "uvu_ir_mul_fast"}


@pytest.mark.parametrize("name,problem", [t for t in tp_problem_matrix() if t[0] not in _BIG],
                         ids=[t[0] for t in tp_problem_matrix() if t[0] not in _BIG])
def test_kernels_compile_for_sm100a(name, problem):
    """NVRTC needs no GPU: every small test problem must specialise and compile (cubins land in the cache that
    travels with the tree, so the GPU suite starts warm)."""
    for dt in (np.float32, np.float64):
        text = build_descriptor(with_dtype(problem, dt))
        assert native.precompile(text.encode()) >= 1


def test_cpp_operator_library_defines_the_six_ops():
    """csrc/torch_ops.cpp registers the libtorch_tp_jit operators from C++ (schemas of the reference's
    extension/torch_core.hpp:636-644); the Python layer must have picked it up instead of defining them itself."""
    import torch

    import openequivariance_b200  # noqa: F401
    from openequivariance_b200 import build_native
    from openequivariance_b200._torch import ops
    assert os.path.exists(build_native.TORCH_LIB) and not build_native.torch_ops_need_build()
    assert ops.CPP_OPS
    for name in ops._SCHEMAS:
        op = getattr(torch.ops.libtorch_tp_jit, name)
        assert str(op.default._schema).replace(" ", "").startswith(f"libtorch_tp_jit::{name}(Tensorjson_bytes,inthash,")


def test_a_key_reused_for_another_problem_is_refused():
    a = build_descriptor(P.readme_problem())
    b = build_descriptor(P.mace_like_problem())
    key = 9_100_000_001
    native.query(a.encode(), key)
    native.query(a.encode(), key)                       # same problem again: fine
    with pytest.raises(RuntimeError, match="different descriptor"):
        native.query(b.encode(), key)


def test_planning_entry_points_check_their_arguments():
    """The device planner refuses inconsistent ranges before it touches the device, and sizes its workspace from the
    arguments alone."""
    import ctypes
    lib = native.load()
    small = lib.oeqb_plan_workspace_bytes(1000, 8000, 500, 500, 2)
    large = lib.oeqb_plan_workspace_bytes(100000, 800000, 50000, 50000, 8)
    assert 0 < small < large
    assert lib.oeqb_plan_workspace_bytes(-1, 10, 1, 1, 1) < 0
    null = ctypes.c_void_p(0)
    bounds = (ctypes.c_int64 * 3)(0, 500, 1000)
    # receiver range past the end of the nodes; rank outside the world; bounds that do not ascend
    assert lib.oeqb_plan_count(1000, 0, null, null, 0, 2000, 0, 500, 2, 0, bounds, null, 0, null, null) == 1  # OEQB_EINVAL
    assert lib.oeqb_plan_count(1000, 0, null, null, 0, 500, 0, 500, 2, 2, bounds, null, 0, null, null) == 1  # OEQB_EINVAL
    bad = (ctypes.c_int64 * 3)(0, 800, 500)
    assert lib.oeqb_plan_count(1000, 0, null, null, 0, 500, 0, 500, 2, 0, bad, null, 0, null, null) == 1  # OEQB_EINVAL
    assert lib.oeqb_plan_fill(1000, 10, null, null, 0, 500, 0, 500, 2, bounds, 5, 3, 0, null, 0, null, null, null, null, null,
                              null) == 1  # OEQB_EINVAL
    assert b"oeqb_plan" in lib.oeqb_last_error()


def test_tensor_core_programs_compile_for_other_block_shapes():
    """The tcgen05 'uvw' programs (forward and the three gradients) specialise and compile without a GPU for the
    NequIP-like problem, for 7-component blocks and for multiplicities above 32."""
    feats3 = "32x0e+32x1o+32x2e+32x3o"
    problems = [P.nequip_like_problem(),
                P.FullyConnectedTPProblem(feats3, "1x0e+1x1o+1x2e+1x3o", feats3, shared_weights=True, label="uvw-l3",
                                          irrep_dtype=np.float32, weight_dtype=np.float32),
                P.FullyConnectedTPProblem("64x0e+64x0o+64x1e+64x1o+64x2e+64x2o", "1x0e+1x1o+1x2e", "32x0e+64x1o+96x2e",
                                          shared_weights=True, label="uvw-mixed", irrep_dtype=np.float32,
                                          weight_dtype=np.float32)]
    for problem in problems:
        text = build_descriptor(problem)
        assert native.query(text.encode(), descriptor_hash(text)).fast_path == 2
        assert native.precompile(text.encode()) >= 5      # general + forward + three gradient programs
