"""Index symbols: ``sym.M`` is an integer-valued sympy symbol named ``M``.

Same surface as the reference's ``hckernel/indexing.py`` (:13-38): ``sym`` is an
expando whose attributes are created on first use, ``index_symbol`` and
``index_expr`` build symbols and expressions explicitly.  Symbols with the same
name are equal, so ``sym.M`` written in two places is one symbol.
"""

import sympy

IndexSymbol = sympy.Symbol
IndexExpr = sympy.Expr


def index_symbol(name: str) -> IndexSymbol:
    return sympy.Symbol(name, integer=True)


def index_expr(value) -> IndexExpr:
    return sympy.sympify(value)


class _SymbolNamespace:
    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return index_symbol(name)


sym = _SymbolNamespace()
