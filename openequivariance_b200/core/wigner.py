"""Real-basis Wigner 3j tensors (the Clebsch-Gordan constants of every kernel in this package).

``wigner_3j(l1, l2, l3)`` returns the ``(2l1+1, 2l2+1, 2l3+1)`` tensor C that is invariant under
simultaneous rotation of its three indices by the real Wigner-D matrices, normalised to unit
Frobenius norm, in the same basis and with the same signs as the reference
(openequivariance/openequivariance/core/e3nn_lite.py:656-864, itself following e3nn's
``o3.wigner_3j``).  The construction is the textbook one:

1. SU(2) Clebsch-Gordan coefficients <j1 m1 j2 m2 | j3 m3> from Racah's closed formula,
   evaluated in exact rational arithmetic (``fractions.Fraction``) so no cancellation error enters;
2. change of basis from complex to real spherical harmonics with the unitary
   ``Q_l`` (rows: complex m = -l..l, columns: real components), carrying the extra phase
   ``(-i)^l`` that makes the transformed tensor purely real;
3. Frobenius normalisation.

The golden-vector test pins every entry for l <= 7 against the reference's own generator.
"""

from __future__ import annotations

import functools
from fractions import Fraction
from math import factorial

import numpy as np


def _racah_cg(j1: int, m1: int, j2: int, m2: int, j3: int, m3: int) -> float:
    """<j1 m1 j2 m2 | j3 m3> for integer spins (Condon-Shortley phase), via Racah's formula."""
    if m1 + m2 != m3 or not (abs(j1 - j2) <= j3 <= j1 + j2) or abs(m3) > j3:
        return 0.0
    fact = factorial
    prefactor = Fraction(
        (2 * j3 + 1) * fact(j3 + j1 - j2) * fact(j3 - j1 + j2) * fact(j1 + j2 - j3),
        fact(j1 + j2 + j3 + 1),
    ) * Fraction(
        fact(j3 + m3) * fact(j3 - m3),
        fact(j1 - m1) * fact(j1 + m1) * fact(j2 - m2) * fact(j2 + m2),
    )
    lo = max(-j1 + j2 + m3, -j1 + m1, 0)
    hi = min(j2 + j3 + m1, j3 - j1 + j2, j3 + m3)
    series = Fraction(0)
    for v in range(lo, hi + 1):
        term = Fraction(
            fact(j2 + j3 + m1 - v) * fact(j1 - m1 + v),
            fact(v) * fact(j3 - j1 + j2 - v) * fact(j3 + m3 - v) * fact(v + j1 - j2 - m3),
        )
        series += term if (v + j2 + m2) % 2 == 0 else -term
    return float(prefactor) ** 0.5 * float(series)


@functools.lru_cache(maxsize=None)
def _su2_cg_tensor(j1: int, j2: int, j3: int) -> np.ndarray:
    out = np.zeros((2 * j1 + 1, 2 * j2 + 1, 2 * j3 + 1), dtype=np.float64)
    for m1 in range(-j1, j1 + 1):
        for m2 in range(-j2, j2 + 1):
            m3 = m1 + m2
            if abs(m3) <= j3:
                out[j1 + m1, j2 + m2, j3 + m3] = _racah_cg(j1, m1, j2, m2, j3, m3)
    return out


def real_to_complex_basis(l: int) -> np.ndarray:
    """Unitary Q with ``Y_complex[m] = sum_a Q[l+m, a] * Y_real[a]``, times the phase ``(-i)^l``."""
    q = np.zeros((2 * l + 1, 2 * l + 1), dtype=np.complex128)
    s = 1.0 / np.sqrt(2.0)
    q[l, l] = 1.0
    for m in range(1, l + 1):
        sign = (-1.0) ** m
        # negative m row
        q[l - m, l + m] = s
        q[l - m, l - m] = -1j * s
        # positive m row
        q[l + m, l + m] = sign * s
        q[l + m, l - m] = 1j * sign * s
    return (-1j) ** l * q


@functools.lru_cache(maxsize=None)
def _real_cg(l1: int, l2: int, l3: int) -> np.ndarray:
    q1, q2, q3 = (real_to_complex_basis(l) for l in (l1, l2, l3))
    c = _su2_cg_tensor(l1, l2, l3).astype(np.complex128)
    # C_real[a,b,c] = sum_{m1,m2,m3} Q1[m1,a] Q2[m2,b] conj(Q3[m3,c]) C[m1,m2,m3]
    c = np.einsum("ia,jb,kc,ijk->abc", q1, q2, np.conj(q3), c)
    assert np.abs(c.imag).max() < 1e-5
    c = np.ascontiguousarray(c.real)
    return c / np.linalg.norm(c.ravel())


def wigner_3j(l1: int, l2: int, l3: int, dtype=np.float64) -> np.ndarray:
    """Real Wigner 3j tensor of shape ``(2l1+1, 2l2+1, 2l3+1)`` with unit Frobenius norm (always a copy)."""
    assert isinstance(l1, int) and isinstance(l2, int) and isinstance(l3, int)
    assert abs(l2 - l3) <= l1 <= l2 + l3
    return _real_cg(l1, l2, l3).copy().astype(dtype)
