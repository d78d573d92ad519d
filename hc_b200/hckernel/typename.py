"""Type names: ``typename.DT`` stands for "whatever element type the argument
has" in a ``Buffer[...]`` annotation (reference: ``hckernel/typename.py:9-29``).
The element type is taken from the actual argument at call time.
"""


class Typename:
    def __init__(self, name):
        self.name = name

    def __repr__(self):
        return f"typename.{self.name}"


class _TypenameNamespace:
    def __init__(self):
        self._known = {}

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)
        return self._known.setdefault(name, Typename(name))


typename = _TypenameNamespace()
