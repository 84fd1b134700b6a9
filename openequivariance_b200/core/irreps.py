"""Irreducible-representation bookkeeping for O(3): ``Irrep``, ``_MulIr`` and ``Irreps``.

These classes reproduce the observable behaviour of the reference's torch-free
e3nn clone (openequivariance/openequivariance/core/e3nn_lite.py:57-350): the same
string grammar ("128x0e+128x1o"), tuple structure, ordering, ``dim``/``slices``/
``sort``/``simplify`` results, so that a ``TPProblem`` written for the reference
constructs unchanged here.  e3nn's own ``Irreps`` objects are accepted anywhere an
``Irreps`` is expected because construction only relies on iteration and ``str``.
"""

from __future__ import annotations

import collections
import itertools
from typing import List, Union

_PARITY_CHAR = {1: "e", -1: "o"}


class Irrep(tuple):
    """One irreducible representation of O(3): degree ``l`` and parity ``p`` (+1 even, -1 odd)."""

    def __new__(cls, l, p=None):
        if p is None:
            if isinstance(l, Irrep):
                return l
            if isinstance(l, str):
                text = l.strip()
                try:
                    degree = int(text[:-1])
                    tag = text[-1]
                    if degree < 0 or tag not in "eoy":
                        raise ValueError
                    parity = {"e": 1, "o": -1, "y": (-1) ** degree}[tag]
                except Exception:
                    raise ValueError(f'unable to convert string "{text}" into an Irrep')
                l, p = degree, parity
            elif isinstance(l, tuple):
                l, p = l
            elif hasattr(l, "l") and hasattr(l, "p"):  # duck-typed foreign Irrep (e.g. e3nn's)
                l, p = int(l.l), int(l.p)
        if not isinstance(l, int) or l < 0:
            raise ValueError(f"l must be positive integer, got {l}")
        if p not in (-1, 1):
            raise ValueError(f"parity must be on of (-1, 1), got {p}")
        return super().__new__(cls, (l, p))

    @property
    def l(self) -> int:  # noqa: E743
        return self[0]

    @property
    def p(self) -> int:
        return self[1]

    @property
    def dim(self) -> int:
        return 2 * self[0] + 1

    def is_scalar(self) -> bool:
        return self[0] == 0 and self[1] == 1

    def __repr__(self) -> str:
        return f"{self[0]}{_PARITY_CHAR[self[1]]}"

    @classmethod
    def iterator(cls, lmax=None):
        """Yields 0e, 0o, 1o, 1e, 2e, 2o, ... (natural parity first), optionally up to ``lmax``."""
        for degree in itertools.count():
            natural = (-1) ** degree
            yield Irrep(degree, natural)
            yield Irrep(degree, -natural)
            if degree == lmax:
                return

    def __mul__(self, other):
        """Selection rule: generator over the irreps contained in ``self ⊗ other``."""
        other = Irrep(other)
        parity = self.p * other.p
        for degree in range(abs(self.l - other.l), self.l + other.l + 1):
            yield Irrep(degree, parity)

    def __rmul__(self, mul):
        assert isinstance(mul, int)
        return Irreps([(mul, self)])

    def __add__(self, other):
        return Irreps(self) + Irreps(other)

    # tuple methods that make no sense on an Irrep are disabled, as in e3nn
    def count(self, _value):
        raise NotImplementedError

    def index(self, _value):
        raise NotImplementedError

    def __contains__(self, _object):
        raise NotImplementedError

    def __len__(self):
        raise NotImplementedError


class _MulIr(tuple):
    """A multiplicity paired with an irrep, e.g. ``128x1o``."""

    def __new__(cls, mul, ir=None):
        if ir is None:
            mul, ir = mul
        assert isinstance(mul, int)
        assert isinstance(ir, Irrep)
        return super().__new__(cls, (mul, ir))

    @property
    def mul(self) -> int:
        return self[0]

    @property
    def ir(self) -> Irrep:
        return self[1]

    @property
    def dim(self) -> int:
        return self[0] * self[1].dim

    def __repr__(self) -> str:
        return f"{self[0]}x{self[1]}"

    def count(self, _value):
        raise NotImplementedError

    def index(self, _value):
        raise NotImplementedError


def _parse_term(term) -> _MulIr:
    """Turns one element of an iterable passed to ``Irreps`` into a ``_MulIr``."""
    if isinstance(term, _MulIr):
        return term
    if isinstance(term, str):
        return _MulIr(1, Irrep(term))
    if isinstance(term, Irrep):
        return _MulIr(1, term)
    mul = ir = None
    try:
        if len(term) == 2:
            mul, ir = term
            ir = Irrep(ir)
            mul = int(mul) if not isinstance(mul, bool) and hasattr(mul, "__index__") else mul
    except Exception:
        mul = ir = None
    if not (isinstance(mul, int) and mul >= 0 and ir is not None):
        raise ValueError(f'Unable to interpret "{term}" as an irrep.')
    return _MulIr(mul, ir)


class Irreps(tuple):
    """A direct sum of irreps with multiplicities; a tuple of ``_MulIr``."""

    def __new__(cls, irreps=None):
        if isinstance(irreps, Irreps):
            return super().__new__(cls, irreps)
        terms: List[_MulIr] = []
        if irreps is None:
            pass
        elif isinstance(irreps, Irrep):
            terms.append(_MulIr(1, irreps))
        elif isinstance(irreps, str):
            try:
                if irreps.strip():
                    for chunk in irreps.split("+"):
                        if "x" in chunk:
                            mul_text, ir_text = chunk.split("x")
                            mul = int(mul_text)
                        else:
                            mul, ir_text = 1, chunk
                        assert mul >= 0
                        terms.append(_MulIr(mul, Irrep(ir_text)))
            except Exception:
                raise ValueError(f'Unable to convert string "{irreps}" into an Irreps')
        else:
            terms = [_parse_term(t) for t in irreps]
        return super().__new__(cls, terms)

    @staticmethod
    def spherical_harmonics(lmax: int, p: int = -1) -> "Irreps":
        return Irreps([(1, (l, p**l)) for l in range(lmax + 1)])

    def slices(self):
        """One ``slice`` of the flattened feature axis per (mul, ir) block."""
        bounds = list(itertools.accumulate((m.dim for m in self), initial=0))
        return [slice(a, b) for a, b in zip(bounds[:-1], bounds[1:])]

    def __getitem__(self, i) -> Union[_MulIr, "Irreps"]:
        got = super().__getitem__(i)
        return Irreps(got) if isinstance(i, slice) else got

    def __contains__(self, ir) -> bool:
        ir = Irrep(ir)
        return any(ir == mine for _, mine in self)

    def count(self, ir) -> int:
        ir = Irrep(ir)
        return sum(mul for mul, mine in self if mine == ir)

    def index(self, _object):
        raise NotImplementedError

    def __add__(self, irreps) -> "Irreps":
        return Irreps(super().__add__(Irreps(irreps)))

    def __mul__(self, other) -> "Irreps":
        if isinstance(other, Irreps):
            raise NotImplementedError("Use o3.TensorProduct for this, see the documentation")
        return Irreps(super().__mul__(other))

    def __rmul__(self, other) -> "Irreps":
        return Irreps(super().__rmul__(other))

    def simplify(self) -> "Irreps":
        """Merges neighbouring blocks of the same irrep and drops empty ones."""
        merged: List[list] = []
        for mul, ir in self:
            if merged and merged[-1][1] == ir:
                merged[-1][0] += mul
            elif mul > 0:
                merged.append([mul, ir])
        return Irreps([(m, ir) for m, ir in merged])

    def remove_zero_multiplicities(self) -> "Irreps":
        return Irreps([(mul, ir) for mul, ir in self if mul > 0])

    def sort(self):
        """Stable sort by (l, p).  Returns ``(irreps, p, inv)`` with ``p[old] = new`` and ``inv[new] = old``."""
        Ret = collections.namedtuple("sort", ["irreps", "p", "inv"])
        order = sorted(range(len(self)), key=lambda i: (self[i].ir, i))
        inv = tuple(order)
        p = tuple(inv.index(i) for i in range(len(inv)))
        return Ret(Irreps([self[i] for i in order]), p, inv)

    def regroup(self) -> "Irreps":
        return self.sort().irreps.simplify()

    @property
    def dim(self) -> int:
        return sum(m.dim for m in self)

    @property
    def num_irreps(self) -> int:
        return sum(mul for mul, _ in self)

    @property
    def ls(self) -> List[int]:
        return [ir.l for mul, ir in self for _ in range(mul)]

    @property
    def lmax(self) -> int:
        if len(self) == 0:
            raise ValueError("Cannot get lmax of empty Irreps")
        return max(self.ls)

    def __repr__(self) -> str:
        return "+".join(repr(m) for m in self)
