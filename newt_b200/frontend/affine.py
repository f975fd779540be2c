"""Integer / pointer expressions as polynomials over index atoms.

The reference never analyses pointer blocks: contiguity and alignment are
checked at run time, per 16-byte group, inside the generated kernel
(newt/compiler/codegen.py:1643-1656, 2612-2616).  TMA needs the opposite: base
pointer, extents, strides and per-iteration coordinates known before launch.
This module recovers them from the traced graph.

Atoms (hashable tuples):
    ("param", name)          a runtime integer argument
    ("pid", axis)            program id
    ("ax", d)                position along dimension d of the block being described
    ("iter", loop)           0-based iteration number of a runtime loop
    ("carried", loop, name)  a loop-carried value not (yet) resolved to a closed form
A Poly maps monomials (sorted tuples of atoms) to integer coefficients.
"""

from .trace import Node


class Poly:
    __slots__ = ("terms",)

    def __init__(self, terms=None):
        self.terms = {m: c for m, c in (terms or {}).items() if c != 0}

    @staticmethod
    def const(c):
        return Poly({(): int(c)})

    @staticmethod
    def atom(a):
        return Poly({(a,): 1})

    def __add__(self, o):
        t = dict(self.terms)
        for m, c in o.terms.items():
            t[m] = t.get(m, 0) + c
        return Poly(t)

    def __neg__(self):
        return Poly({m: -c for m, c in self.terms.items()})

    def __sub__(self, o):
        return self + (-o)

    def __mul__(self, o):
        t = {}
        for m1, c1 in self.terms.items():
            for m2, c2 in o.terms.items():
                m = tuple(sorted(m1 + m2, key=repr))
                t[m] = t.get(m, 0) + c1 * c2
        return Poly(t)

    def __eq__(self, o):
        return isinstance(o, Poly) and self.terms == o.terms

    def __hash__(self):
        return hash(frozenset(self.terms.items()))

    def is_zero(self):
        return not self.terms

    def is_const(self):
        return all(m == () for m in self.terms)

    def const_value(self):
        return self.terms.get((), 0) if self.is_const() else None

    def atoms(self):
        return {a for m in self.terms for a in m}

    def has_kind(self, *kinds):
        return any(a[0] in kinds for a in self.atoms())

    def coeff_of(self, atom):
        """Collects the terms linear in `atom` and divides it out; returns
        (quotient, remainder) or None when `atom` appears with a power > 1."""
        q, r = {}, {}
        for m, c in self.terms.items():
            n = m.count(atom)
            if n == 0:
                r[m] = c
            elif n == 1:
                mm = list(m)
                mm.remove(atom)
                q[tuple(mm)] = q.get(tuple(mm), 0) + c
            else:
                return None
        return Poly(q), Poly(r)

    def map_atoms(self, fn):
        """Substitutes atoms: fn(atom) -> Poly or None (keep)."""
        out = Poly()
        for m, c in self.terms.items():
            term = Poly.const(c)
            for a in m:
                sub = fn(a)
                term = term * (sub if sub is not None else Poly.atom(a))
            out = out + term
        return out

    def divide_by(self, d):
        """Exact division by a single-term polynomial; None if not divisible."""
        if len(d.terms) != 1:
            return None
        (dm, dc), = d.terms.items()
        out = {}
        for m, c in self.terms.items():
            if c % dc:
                return None
            mm = list(m)
            for a in dm:
                if a not in mm:
                    return None
                mm.remove(a)
            out[tuple(mm)] = c // dc
        return Poly(out)

    def to_python(self, arg="a"):
        """Source of a Python expression evaluating the polynomial from a dict of
        runtime arguments; only ("param", name) atoms may be present."""
        if not self.terms:
            return "0"
        parts = []
        for m, c in sorted(self.terms.items(), key=repr):
            fac = [str(c)] if (c != 1 or not m) else []
            for a in m:
                if a[0] != "param":
                    raise ValueError(f"cannot evaluate atom {a} on the host")
                fac.append(f"{arg}[{a[1]!r}]")
            parts.append("*".join(fac))
        return "(" + " + ".join(parts) + ")"

    def __repr__(self):
        if not self.terms:
            return "0"
        out = []
        for m, c in sorted(self.terms.items(), key=repr):
            names = ["%s%s" % (a[0], "".join("_" + str(x) for x in a[1:])) for a in m]
            out.append("*".join(([str(c)] if c != 1 or not names else []) + names))
        return " + ".join(out)


class NotAffine(Exception):
    pass


def _shift_axes(p, fn):
    def sub(a):
        if a[0] == "ax":
            return Poly.atom(("ax", fn(a[1])))
        return None
    return p.map_atoms(sub)


class Analyzer:
    """Polynomial view of the integer and pointer nodes of one trace.

    `closed_forms` maps ("carried", loop, name) to the polynomial of that value
    as a function of the iteration number, for carried values recognised as
    inductions (see `resolve_inductions`)."""

    def __init__(self, trace):
        self.trace = trace
        self.loops = {l.uid: l for l in trace.loops}
        self.closed_forms = {}
        self.closed_bases = {}
        self._memo = {}

    # value of an integer expression, in the numbering of its own dimensions
    def poly(self, v):
        if isinstance(v, bool):
            raise NotAffine("bool")
        if isinstance(v, int):
            return Poly.const(v)
        if not isinstance(v, Node):
            raise NotAffine(repr(v))
        hit = self._memo.get(v.uid)
        if hit is None:
            hit = self._poly(v)
            self._memo[v.uid] = hit
        return hit

    def _aligned(self, a, b, rank):
        pa, pb = self.poly(a), self.poly(b)
        ra = len(a.shape) if isinstance(a, Node) else 0
        rb = len(b.shape) if isinstance(b, Node) else 0
        if ra < rank:
            pa = _shift_axes(pa, lambda d, k=rank - ra: d + k)
        if rb < rank:
            pb = _shift_axes(pb, lambda d, k=rank - rb: d + k)
        return pa, pb

    def _poly(self, n):
        op = n.op
        if n.is_pointer and op not in ("ptradd", "ptrsub", "param", "carried", "loopout",
                                       "expand", "broadcast"):
            raise NotAffine(op)
        if op == "const":
            if not isinstance(n.args[0], int) or isinstance(n.args[0], bool):
                raise NotAffine("non-integer constant")
            return Poly.const(n.args[0])
        if op == "param":
            if n.is_pointer:
                return Poly()  # offset relative to its own base
            if not n.dtype.is_int:
                raise NotAffine("float parameter")
            return Poly.atom(("param", dict(n.attrs)["name"]))
        if op == "pid":
            return Poly.atom(("pid", dict(n.attrs)["axis"]))
        if op == "arange":
            return Poly.atom(("ax", 0)) + Poly.const(n.args[0])
        if op == "loopvar":
            loop = self.loops[dict(n.attrs)["loop"]]
            return self.poly(loop.lo) + Poly.atom(("iter", loop.uid)) * self.poly(loop.step)
        if op == "carried":
            at = dict(n.attrs)
            key = ("carried", at["loop"], at["name"])
            if key in self.closed_forms:
                return self.closed_forms[key]
            return Poly.atom(key)
        if op == "expand":
            axis = dict(n.attrs)["axis"]
            return _shift_axes(self.poly(n.args[0]), lambda d: d + 1 if d >= axis else d)
        if op == "broadcast":
            src = n.args[0]
            k = len(n.shape) - len(src.shape)
            return _shift_axes(self.poly(src), lambda d: d + k)
        if op == "trans":
            return _shift_axes(self.poly(n.args[0]), lambda d: 1 - d)
        if op == "neg":
            return -self.poly(n.args[0])
        if op == "cast":
            if not n.dtype.is_int or not n.args[0].dtype.is_int:
                raise NotAffine("cast")
            return self.poly(n.args[0])
        if op in ("ptradd", "ptrsub"):
            pa, pb = self._aligned(n.args[0], n.args[1], len(n.shape))
            return pa + pb if op == "ptradd" else pa - pb
        if op == "bin":
            fn = dict(n.attrs)["fn"]
            if not n.dtype.is_int:
                raise NotAffine("float arithmetic")
            if fn in ("add", "sub", "mul"):
                pa, pb = self._aligned(n.args[0], n.args[1], len(n.shape))
                return pa + pb if fn == "add" else (pa - pb if fn == "sub" else pa * pb)
            raise NotAffine(fn)
        raise NotAffine(op)

    def base_of(self, n):
        """The pointer parameter a pointer expression is built on (its name)."""
        while True:
            if n.op == "param":
                return dict(n.attrs)["name"]
            if n.op in ("ptradd", "ptrsub", "expand", "broadcast"):
                n = n.args[0]
                continue
            if n.op == "carried":
                at = dict(n.attrs)
                key = ("carried", at["loop"], at["name"])
                if key in self.closed_bases:
                    return self.closed_bases[key]
                raise NotAffine("pointer carried through a loop without a closed form")
            if n.op == "loopout":
                at = dict(n.attrs)
                _, init, _ = self.loops[at["loop"]].carried[at["name"]]
                n = init
                continue
            raise NotAffine(f"pointer built by {n.op}")

    def pointer(self, n):
        """(base parameter name, offset polynomial in elements)."""
        return self.base_of(n), self.poly(n)

    def resolve_inductions(self):
        """Finds loop-carried integers / pointers of the form v <- v + delta with a
        loop-invariant delta (e.g. `a_ptrs += BLOCK_K * sak`) and records
        v(iter) = init + iter * delta."""
        for loop in self.trace.loops:
            for name, (ph, init, nxt) in loop.carried.items():
                if not (init.is_pointer or init.dtype.is_int):
                    continue
                key = ("carried", loop.uid, name)
                try:
                    p_next = self.poly(nxt)
                    p_init = self.poly(init)
                    if init.is_pointer:
                        base = self.base_of(init)
                        self.closed_bases[key] = base
                        if self.base_of(nxt) != base:
                            raise NotAffine("rebased")
                except NotAffine:
                    self.closed_bases.pop(key, None)
                    continue
                delta = p_next - Poly.atom(key)
                if delta.has_kind("iter", "carried"):
                    self.closed_bases.pop(key, None)
                    continue
                self.closed_forms[key] = p_init + Poly.atom(("iter", loop.uid)) * delta
                self._memo.clear()
