"""Reversible, instance-local attribute patches (reference: optimizations/patching.py:6-46)."""

from types import FunctionType, MethodType

_REGISTRIES = ("_modules", "_parameters", "_buffers")
_ABSENT = object()


class Patches:
    """Records every change it makes so that `restore` can undo them in reverse order."""

    def __init__(self):
        self._undo = []

    def set(self, obj, name, value):
        """setattr with memory: remembers the previous value, or that there was none."""
        own = vars(obj)
        present = name in own or any(name in own.get(registry, {}) for registry in _REGISTRIES)
        self._undo.append((obj, name, getattr(obj, name) if present else _ABSENT))
        setattr(obj, name, value)

    def bind(self, obj, name, function):
        """Install `function` as a bound method of this one instance."""
        self.set(obj, name, MethodType(function, obj))

    def globals(self, obj, name, replacements):
        """Re-bind method `name` of `obj` to a copy of its function that sees `replacements` as
        module globals; the module itself and other instances are untouched."""
        original = getattr(obj, name).__func__
        missing = [key for key in replacements if key not in original.__globals__]
        if missing:
            raise ValueError(f"Unsupported callable: missing global {missing[0]}")
        clone = FunctionType(
            original.__code__, {**original.__globals__, **replacements}, original.__name__,
            original.__defaults__, original.__closure__,
        )
        clone.__kwdefaults__ = original.__kwdefaults__
        self.bind(obj, name, clone)

    def restore(self):
        while self._undo:
            obj, name, previous = self._undo.pop()
            if previous is _ABSENT:
                delattr(obj, name)
            else:
                setattr(obj, name, previous)
