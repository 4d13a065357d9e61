"""Affine expressions and maps of the builder surface, MLIR-free.

The reference binds MLIR's ``AffineExpr`` / ``AffineMap`` directly (``ffi/ir.cpp:640-875``; used by
``test/python/map_expr_test.py`` and by explicit copy maps).  MLIR is not available here, so this is
a restatement of the published behaviour of those classes: expressions are immutable trees that are
simplified as they are built (constants fold, a constant operand moves to the right, ``x + 0``,
``x * 1`` and ``x * 0`` collapse, nested constant additions / multiplications merge), and they print
the way MLIR's printer does (``d0 * 5 + s0``, ``d0 - d1``, ``(d0 + 1) * 2``).  The deeper
simplifier (``simplifyAffineExpr``: flattening to a linear form) is not restated.
"""
import enum


class AffineExprKind(enum.IntEnum):
    Add = 0
    Mul = 1
    Mod = 2
    FloorDiv = 3
    CeilDiv = 4
    LAST_AFFINE_BINARY_OP = 4
    Constant = 5
    DimId = 6
    SymbolId = 7

    def __str__(self):  # the binding's enum prints its qualified name
        return f"AffineExprKind.{self.name}"


_BINARY = (AffineExprKind.Add, AffineExprKind.Mul, AffineExprKind.Mod, AffineExprKind.FloorDiv,
           AffineExprKind.CeilDiv)


def _floordiv(a, b):
    return a // b  # Python floors toward minus infinity, like MLIR's floorDiv


def _ceildiv(a, b):
    return -((-a) // b)


class AffineExpr:
    """Immutable expression node; a default-constructed one is null (prints ``<<NULL AFFINE EXPR>>``)."""
    __slots__ = ("kind", "lhs", "rhs", "value")

    def __init__(self, kind=None, lhs=None, rhs=None, value=None):
        object.__setattr__(self, "kind", kind)
        object.__setattr__(self, "lhs", lhs)
        object.__setattr__(self, "rhs", rhs)
        object.__setattr__(self, "value", value)

    def __setattr__(self, *_):
        raise AttributeError("AffineExpr is immutable")

    # ---- identity
    def _key(self):
        return (self.kind, self.lhs._key() if self.lhs is not None else None,
                self.rhs._key() if self.rhs is not None else None, self.value)

    def __eq__(self, other):
        if isinstance(other, int):
            return self.kind == AffineExprKind.Constant and self.value == other
        return isinstance(other, AffineExpr) and self._key() == other._key()

    def __ne__(self, other):
        return not self.__eq__(other)

    def __hash__(self):
        return hash(self._key())

    def __bool__(self):
        return self.kind is not None

    # ---- queries
    def get_kind(self):
        return self.kind

    def is_symbolic_or_constant(self):
        if self.kind in (AffineExprKind.Constant, AffineExprKind.SymbolId):
            return True
        if self.kind == AffineExprKind.DimId:
            return False
        return self.lhs.is_symbolic_or_constant() and self.rhs.is_symbolic_or_constant()

    def is_pure_affine(self):
        k = self.kind
        if k in (AffineExprKind.Constant, AffineExprKind.SymbolId, AffineExprKind.DimId):
            return True
        if k == AffineExprKind.Add:
            return self.lhs.is_pure_affine() and self.rhs.is_pure_affine()
        if k == AffineExprKind.Mul:  # one side has to be a constant
            return (self.lhs.is_pure_affine() and self.rhs.is_pure_affine() and
                    AffineExprKind.Constant in (self.lhs.kind, self.rhs.kind))
        return self.lhs.is_pure_affine() and self.rhs.kind == AffineExprKind.Constant

    def get_largest_known_divisor(self):
        import math
        k = self.kind
        if k == AffineExprKind.Constant:
            return abs(self.value)
        if k in (AffineExprKind.DimId, AffineExprKind.SymbolId):
            return 1
        if k == AffineExprKind.Mul:
            return self.lhs.get_largest_known_divisor() * self.rhs.get_largest_known_divisor()
        if k in (AffineExprKind.Add, AffineExprKind.Mod):
            return math.gcd(self.lhs.get_largest_known_divisor(), self.rhs.get_largest_known_divisor())
        return 1

    def is_multiple_of(self, factor):
        k = self.kind
        if k == AffineExprKind.Constant:
            return self.value % factor == 0
        if k in (AffineExprKind.DimId, AffineExprKind.SymbolId):
            return factor * factor == 1
        if k == AffineExprKind.Mul:
            l, r = self.lhs.get_largest_known_divisor(), self.rhs.get_largest_known_divisor()
            return l % factor == 0 or r % factor == 0 or (l * r) % factor == 0
        if k in (AffineExprKind.Add, AffineExprKind.Mod):
            import math
            return math.gcd(self.lhs.get_largest_known_divisor(), self.rhs.get_largest_known_divisor()) % factor == 0
        return factor * factor == 1

    def _depends(self, kind, position):
        if self.kind == kind:
            return self.value == position
        if self.kind in _BINARY:
            return self.lhs._depends(kind, position) or self.rhs._depends(kind, position)
        return False

    def is_function_of_dim(self, position):
        return self._depends(AffineExprKind.DimId, position)

    def is_function_of_symbol(self, position):
        return self._depends(AffineExprKind.SymbolId, position)

    # ---- substitution
    def replace_dims_and_symbols(self, dim_replacements, sym_replacements=()):
        k = self.kind
        if k == AffineExprKind.DimId:
            return dim_replacements[self.value] if self.value < len(dim_replacements) else self
        if k == AffineExprKind.SymbolId:
            return sym_replacements[self.value] if self.value < len(sym_replacements) else self
        if k in _BINARY:
            return get_affine_binary_op_expr(k, self.lhs.replace_dims_and_symbols(dim_replacements, sym_replacements),
                                             self.rhs.replace_dims_and_symbols(dim_replacements, sym_replacements))
        return self

    def replace_dims(self, dim_replacements):
        return self.replace_dims_and_symbols(dim_replacements, ())

    def replace_symbols(self, sym_replacements):
        return self.replace_dims_and_symbols((), sym_replacements)

    def replace(self, target, replacement):
        if self == target:
            return replacement
        if self.kind in _BINARY:
            return get_affine_binary_op_expr(self.kind, self.lhs.replace(target, replacement),
                                             self.rhs.replace(target, replacement))
        return self

    def compose(self, affine_map):
        return self.replace_dims_and_symbols(affine_map.get_results(), ())

    # ---- casts (None when the kind does not match, like the binding's dyn_cast wrappers)
    def as_binary(self):
        return AffineBinaryOpExpr(self) if self.kind in _BINARY else None

    def as_dim(self):
        return AffineDimExpr(self) if self.kind == AffineExprKind.DimId else None

    def as_symbol(self):
        return AffineSymbolExpr(self) if self.kind == AffineExprKind.SymbolId else None

    def as_constant(self):
        return AffineConstantExpr(self) if self.kind == AffineExprKind.Constant else None

    # ---- arithmetic
    @staticmethod
    def _wrap(v):
        return get_affine_constant_expr(v) if isinstance(v, int) else v

    def __add__(self, other):
        return _add(self, self._wrap(other))

    __radd__ = __add__

    def __neg__(self):
        return _mul(self, get_affine_constant_expr(-1))

    def __sub__(self, other):
        return _add(self, -self._wrap(other))

    def __rsub__(self, other):
        return _add(self._wrap(other), -self)

    def __mul__(self, other):
        return _mul(self, self._wrap(other))

    __rmul__ = __mul__

    def floor_div(self, other):
        return _floor_div(self, self._wrap(other))

    def ceil_div(self, other):
        return _ceil_div(self, self._wrap(other))

    def __mod__(self, other):
        return _mod(self, self._wrap(other))

    # ---- printing (MLIR's AsmPrinter rules for affine expressions)
    def _print(self, strong):
        k = self.kind
        if k is None:
            return "<<NULL AFFINE EXPR>>"
        if k == AffineExprKind.SymbolId:
            return f"s{self.value}"
        if k == AffineExprKind.DimId:
            return f"d{self.value}"
        if k == AffineExprKind.Constant:
            return str(self.value)
        if k != AffineExprKind.Add:
            word = {AffineExprKind.Mul: " * ", AffineExprKind.FloorDiv: " floordiv ",
                    AffineExprKind.CeilDiv: " ceildiv ", AffineExprKind.Mod: " mod "}[k]
            if k == AffineExprKind.Mul and self.rhs.kind == AffineExprKind.Constant and self.rhs.value == -1:
                return "-" + self.lhs._print(True)
            return self.lhs._print(True) + word + self.rhs._print(True)
        # additions: a term that is a multiplication by a negative constant prints as a subtraction
        lhs, rhs = self.lhs, self.rhs
        text = None
        if rhs.kind == AffineExprKind.Mul and rhs.rhs.kind == AffineExprKind.Constant:
            c = rhs.rhs.value
            if c == -1:
                text = lhs._print(False) + " - " + rhs.lhs._print(True)
            elif c < -1:
                text = lhs._print(False) + " - " + rhs.lhs._print(True) + " * " + str(-c)
        if text is None and rhs.kind == AffineExprKind.Constant and rhs.value < 0:
            text = lhs._print(False) + " - " + str(-rhs.value)
        if text is None:
            text = lhs._print(False) + " + " + rhs._print(False)
        return "(" + text + ")" if strong else text

    def __str__(self):
        return self._print(False)

    def __repr__(self):
        return f"AffineExpr({self})"


class _View(AffineExpr):
    __slots__ = ()

    def __init__(self, e):
        AffineExpr.__init__(self, e.kind, e.lhs, e.rhs, e.value)


class AffineBinaryOpExpr(_View):
    __slots__ = ()

    def get_lhs(self):
        return self.lhs

    def get_rhs(self):
        return self.rhs


class AffineDimExpr(_View):
    __slots__ = ()

    def get_position(self):
        return self.value


class AffineSymbolExpr(_View):
    __slots__ = ()

    def get_position(self):
        return self.value


class AffineConstantExpr(_View):
    __slots__ = ()

    def get_value(self):
        return self.value


def get_affine_dim_expr(position, context=None):
    return AffineExpr(AffineExprKind.DimId, value=int(position))


def get_affine_symbol_expr(position, context=None):
    return AffineExpr(AffineExprKind.SymbolId, value=int(position))


def get_affine_constant_expr(value, context=None):
    return AffineExpr(AffineExprKind.Constant, value=int(value))


def get_affine_constant_exprs(values, context=None):
    return [get_affine_constant_expr(v) for v in values]


def _const(e):
    return e.value if e.kind == AffineExprKind.Constant else None


def _add(lhs, rhs):
    lc, rc = _const(lhs), _const(rhs)
    if lc is not None and rc is not None:
        return get_affine_constant_expr(lc + rc)
    # canonical form: the constant, else the symbolic operand, on the right
    if lc is not None or (lhs.is_symbolic_or_constant() and not rhs.is_symbolic_or_constant()):
        return _add(rhs, lhs)
    if rc == 0:
        return lhs
    if rc is not None and lhs.kind == AffineExprKind.Add and _const(lhs.rhs) is not None:
        return _add(lhs.lhs, get_affine_constant_expr(lhs.rhs.value + rc))  # (x + c1) + c2
    if lhs.kind == AffineExprKind.Add and _const(lhs.rhs) is not None:
        return _add(_add(lhs.lhs, rhs), lhs.rhs)  # (x + c) + y  ->  (x + y) + c
    # c1 * x + c2 * x  ->  x * (c1 + c2)
    first, c1 = (lhs.lhs, lhs.rhs.value) if lhs.kind == AffineExprKind.Mul and _const(lhs.rhs) is not None else (lhs, 1)
    second, c2 = (rhs.lhs, rhs.rhs.value) if rhs.kind == AffineExprKind.Mul and _const(rhs.rhs) is not None else (rhs, 1)
    if first == second:
        return _mul(first, get_affine_constant_expr(c1 + c2))
    return AffineExpr(AffineExprKind.Add, lhs, rhs)


def _mul(lhs, rhs):
    lc, rc = _const(lhs), _const(rhs)
    if lc is not None and rc is not None:
        return get_affine_constant_expr(lc * rc)
    if not lhs.is_symbolic_or_constant() and not rhs.is_symbolic_or_constant():
        raise ValueError("non-affine expression -> a multiplication needs a symbolic or constant operand")
    if lc is not None or (lhs.is_symbolic_or_constant() and not rhs.is_symbolic_or_constant()):
        return _mul(rhs, lhs)
    if rc == 1:
        return lhs
    if rc == 0:
        return rhs
    if rc is not None and lhs.kind == AffineExprKind.Mul and _const(lhs.rhs) is not None:
        return _mul(lhs.lhs, get_affine_constant_expr(lhs.rhs.value * rc))  # (x * c1) * c2
    if lhs.kind == AffineExprKind.Mul and _const(lhs.rhs) is not None:
        return _mul(_mul(lhs.lhs, rhs), lhs.rhs)  # (x * c) * s  ->  (x * s) * c
    return AffineExpr(AffineExprKind.Mul, lhs, rhs)


def _div_checks(rhs):
    rc = _const(rhs)
    if not rhs.is_symbolic_or_constant():
        raise ValueError("non-affine expression -> the divisor has to be symbolic or constant")
    return rc


def _floor_div(lhs, rhs):
    rc = _div_checks(rhs)
    if rc is None or rc < 1:
        return AffineExpr(AffineExprKind.FloorDiv, lhs, rhs)
    lc = _const(lhs)
    if lc is not None:
        return get_affine_constant_expr(_floordiv(lc, rc))
    if rc == 1:
        return lhs
    if lhs.kind == AffineExprKind.Mul and _const(lhs.rhs) is not None and lhs.rhs.value % rc == 0:
        return _mul(lhs.lhs, get_affine_constant_expr(lhs.rhs.value // rc))  # (x * c) floordiv d, d | c
    return AffineExpr(AffineExprKind.FloorDiv, lhs, rhs)


def _ceil_div(lhs, rhs):
    rc = _div_checks(rhs)
    if rc is None or rc < 1:
        return AffineExpr(AffineExprKind.CeilDiv, lhs, rhs)
    lc = _const(lhs)
    if lc is not None:
        return get_affine_constant_expr(_ceildiv(lc, rc))
    if rc == 1:
        return lhs
    if lhs.kind == AffineExprKind.Mul and _const(lhs.rhs) is not None and lhs.rhs.value % rc == 0:
        return _mul(lhs.lhs, get_affine_constant_expr(lhs.rhs.value // rc))
    return AffineExpr(AffineExprKind.CeilDiv, lhs, rhs)


def _mod(lhs, rhs):
    rc = _div_checks(rhs)
    if rc is None or rc < 1:
        return AffineExpr(AffineExprKind.Mod, lhs, rhs)
    lc = _const(lhs)
    if lc is not None:
        return get_affine_constant_expr(lc % rc)
    if lhs.get_largest_known_divisor() % rc == 0:
        return get_affine_constant_expr(0)
    return AffineExpr(AffineExprKind.Mod, lhs, rhs)


def get_affine_binary_op_expr(kind, lhs, rhs):
    kind = AffineExprKind(int(kind))
    if kind == AffineExprKind.Add:
        return _add(lhs, rhs)
    if kind == AffineExprKind.Mul:
        return _mul(lhs, rhs)
    if kind == AffineExprKind.FloorDiv:
        return _floor_div(lhs, rhs)
    if kind == AffineExprKind.CeilDiv:
        return _ceil_div(lhs, rhs)
    if kind == AffineExprKind.Mod:
        return _mod(lhs, rhs)
    raise ValueError("not a binary affine expression kind")


class AffineMap:
    """``(d0, ...)[s0, ...] -> (results)``.  Default-constructed: the null map (false in a boolean
    context), which the builders read as "no map given"."""

    def __init__(self, rank=None, empty=False, num_dims=None, num_symbols=0, results=None):
        if results is not None or num_dims is not None:
            self._null = False
            self.num_dims, self.num_symbols = int(num_dims or 0), int(num_symbols)
            self.results = list(results or [])
        elif empty:
            self._null, self.num_dims, self.num_symbols, self.results = False, 0, 0, []
        elif rank is not None:
            self._null, self.num_dims, self.num_symbols = False, int(rank), 0
            self.results = [get_affine_dim_expr(i) for i in range(int(rank))]
        else:
            self._null, self.num_dims, self.num_symbols, self.results = True, 0, 0, []

    # ---- factories (ffi/ir.cpp:645-681)
    @staticmethod
    def get(*args):
        """get(context) | get(dims, symbols, context) | get(dims, symbols, expr) |
        get(dims, symbols, [exprs], context)"""
        if len(args) == 1:
            return AffineMap(empty=True)
        if len(args) == 3 and isinstance(args[2], AffineExpr):
            return AffineMap(num_dims=args[0], num_symbols=args[1], results=[args[2]])
        if len(args) == 3:
            return AffineMap(num_dims=args[0], num_symbols=args[1], results=[])
        if len(args) == 4:
            return AffineMap(num_dims=args[0], num_symbols=args[1], results=list(args[2]))
        raise TypeError("AffineMap.get: unsupported arguments")

    @staticmethod
    def get_constant_map(value, context=None):
        return AffineMap(num_dims=0, num_symbols=0, results=[get_affine_constant_expr(value)])

    @staticmethod
    def get_multi_dim_identity_map(num_dims, context=None):
        return AffineMap(rank=num_dims)

    get_multi_dim_map_with_targets = get_multi_dim_identity_map

    @staticmethod
    def get_minor_identity_map(dims, results, context=None):
        if dims < results:
            raise ValueError("Dimension mismatch")
        return AffineMap(num_dims=dims, results=[get_affine_dim_expr(i) for i in range(dims - results, dims)])

    @staticmethod
    def get_permutation_map(permutation, context=None):
        perm = [int(p) for p in permutation]
        if sorted(perm) != list(range(len(perm))):
            raise ValueError("Invalid permutation when making an AffineMap")
        return AffineMap(num_dims=len(perm), results=[get_affine_dim_expr(p) for p in perm])

    # ---- compatibility with the rank / empty view the op builders use
    @property
    def rank(self):
        return None if self._null or self.is_empty() else self.num_dims

    @property
    def empty(self):
        return (not self._null) and self.is_empty()

    def __bool__(self):
        return not self._null

    def __eq__(self, other):
        return (isinstance(other, AffineMap) and self._null == other._null and
                (self.num_dims, self.num_symbols, self.results) == (other.num_dims, other.num_symbols, other.results))

    def __ne__(self, other):
        return not self.__eq__(other)

    def __hash__(self):
        return hash((self._null, self.num_dims, self.num_symbols, tuple(self.results)))

    # ---- queries
    def get_num_dims(self):
        return self.num_dims

    def get_num_symbols(self):
        return self.num_symbols

    def get_num_results(self):
        return len(self.results)

    def get_num_inputs(self):
        return self.num_dims + self.num_symbols

    def get_results(self):
        return list(self.results)

    def get_result(self, idx):
        return self.results[idx]

    def is_empty(self):
        return self.num_dims == 0 and self.num_symbols == 0 and not self.results

    def is_identity(self):
        if self.num_dims != len(self.results):
            return False
        return all(r.kind == AffineExprKind.DimId and r.value == i for i, r in enumerate(self.results))

    def is_symbol_identity(self):
        if self.num_symbols != len(self.results):
            return False
        return all(r.kind == AffineExprKind.SymbolId and r.value == i for i, r in enumerate(self.results))

    def is_minor_identity(self):
        n = len(self.results)
        return self.num_dims >= n and self == AffineMap.get_minor_identity_map(self.num_dims, n)

    def is_constant(self):
        return all(r.kind == AffineExprKind.Constant for r in self.results)

    def is_single_constant(self):
        return len(self.results) == 1 and self.results[0].kind == AffineExprKind.Constant

    def get_single_constant_result(self):
        if not self.is_single_constant():
            raise ValueError("map must have a single constant result")
        return self.results[0].value

    def get_constant_results(self):
        if not self.is_constant():
            raise ValueError("map must have only constant results")
        return [r.value for r in self.results]

    def is_projected_permutation(self, allow_zero_in_results=False):
        if self.num_symbols > 0 or len(self.results) > self.num_dims:
            return False
        seen = set()
        for r in self.results:
            if r.kind == AffineExprKind.DimId:
                if r.value in seen:
                    return False
                seen.add(r.value)
            elif not (allow_zero_in_results and r.kind == AffineExprKind.Constant and r.value == 0):
                return False
        return True

    def is_permutation(self):
        return self.num_dims == len(self.results) and self.is_projected_permutation()

    def get_dim_position(self, idx):
        r = self.results[idx]
        if r.kind != AffineExprKind.DimId:
            raise ValueError("result is not a dimension")
        return r.value

    def get_result_position(self, expr):
        if expr.kind != AffineExprKind.DimId:
            return None
        for i, r in enumerate(self.results):
            if r == expr:
                return i
        return None

    def __str__(self):
        if self._null:
            return "<<NULL AFFINE MAP>>"
        dims = ", ".join(f"d{i}" for i in range(self.num_dims))
        syms = "[" + ", ".join(f"s{i}" for i in range(self.num_symbols)) + "]" if self.num_symbols else ""
        return f"({dims}){syms} -> (" + ", ".join(str(r) for r in self.results) + ")"

    def __repr__(self):
        return f"AffineMap({self})"
