"""A small runtime-patch helper: replace one attribute of an upstream vLLM module or class.

    @patch("vllm.some.module")                      # attribute name = function name
    def target(...): ...

    @patch("vllm.some.module", "Cls.method")        # dotted path into a class
    def method(self, ...): ...

    @patch("vllm.some.module", "Cls.prop")          # property / staticmethod / classmethod keep
    @property                                       # their descriptor kind (given explicitly or
    def prop(self): ...                             # inherited from the attribute being replaced)

Every applied patch is recorded (``applied()``), the replacement carries the marker attribute
``__b200_patch__`` = (module, path) and keeps the original reachable as ``__b200_original__``.
Patching one target twice raises ``RuntimeError``; ``revert_all()`` restores the originals (tests).

On NVIDIA hardware almost none of the reference's patches are needed (they exist because its
runtime, collectives library and shared-memory size differ from CUDA's); what remains here are
behavioural ones.  Parity: vllm_metax/patch/utils.py:16-254 and patch/README.md.
"""
from __future__ import annotations

import importlib
import inspect
import threading
from dataclasses import dataclass
from typing import Any, Callable, Optional

MARKER = "__b200_patch__"
ORIGINAL = "__b200_original__"
_MISSING = object()


@dataclass
class PatchRecord:
    module: str
    path: str
    original: Any
    replacement: Any
    owner: Any
    attr: str
    existed: bool


_applied: dict[tuple[str, str], PatchRecord] = {}
_lock = threading.Lock()


def applied() -> list[PatchRecord]:
    return list(_applied.values())


def is_patched(module: str, path: str) -> bool:
    return (module, path) in _applied


def _resolve_owner(module_name: str, path: str):
    mod = importlib.import_module(module_name)
    owner: Any = mod
    parts = path.split(".")
    for p in parts[:-1]:
        owner = getattr(owner, p)
    return owner, parts[-1]


def _raw_attr(owner: Any, attr: str):
    """The attribute as stored (descriptor object), not as looked up."""
    if inspect.isclass(owner):
        for klass in owner.__mro__:
            if attr in klass.__dict__:
                return klass.__dict__[attr]
        return _MISSING
    return getattr(owner, attr, _MISSING)


def _mark(obj: Any, key: tuple[str, str], original: Any) -> None:
    target = obj
    if isinstance(obj, (staticmethod, classmethod)):
        target = obj.__func__
    elif isinstance(obj, property):
        target = obj.fget
    for name, val in ((MARKER, key), (ORIGINAL, original)):
        try:
            setattr(target, name, val)
        except (AttributeError, TypeError):
            pass


def _wrap_like(original: Any, replacement: Any) -> Any:
    """Give a plain function the descriptor kind of the attribute it replaces."""
    if isinstance(replacement, (staticmethod, classmethod, property)):
        return replacement
    if isinstance(original, staticmethod):
        return staticmethod(replacement)
    if isinstance(original, classmethod):
        return classmethod(replacement)
    if isinstance(original, property) and callable(replacement):
        return property(replacement, original.fset, original.fdel, original.__doc__)
    return replacement


def apply_patch(module_name: str, path: str, replacement: Any, *, allow_new: bool = False) -> PatchRecord:
    key = (module_name, path)
    with _lock:
        if key in _applied:
            raise RuntimeError(f"{module_name}:{path} is already patched by "
                               f"{getattr(_applied[key].replacement, '__module__', '?')}")
        owner, attr = _resolve_owner(module_name, path)
        original = _raw_attr(owner, attr)
        existed = original is not _MISSING
        if not existed and not allow_new:
            raise AttributeError(f"{module_name}:{path} does not exist (pass allow_new=True to add it)")
        if existed and getattr(getattr(original, "__func__", original), MARKER, None) is not None:
            raise RuntimeError(f"{module_name}:{path} already carries a patch marker")
        new = _wrap_like(original, replacement) if inspect.isclass(owner) else replacement
        _mark(new, key, None if not existed else original)
        setattr(owner, attr, new)
        rec = PatchRecord(module_name, path, original if existed else None, new, owner, attr, existed)
        _applied[key] = rec
        return rec


def patch(module_name: str, path: Optional[str] = None, *, allow_new: bool = False,
          when: Optional[Callable[[], bool]] = None) -> Callable[[Any], Any]:
    """Decorator form of ``apply_patch``.  ``when`` (evaluated once, at decoration) gates the patch;
    a missing upstream module makes the patch a no-op rather than an import error."""

    def deco(obj: Any) -> Any:
        name = path
        if name is None:
            fn = obj
            if isinstance(obj, (staticmethod, classmethod)):
                fn = obj.__func__
            elif isinstance(obj, property):
                fn = obj.fget
            name = fn.__name__
        if when is not None and not when():
            return obj
        try:
            importlib.import_module(module_name)
        except ImportError:
            return obj
        apply_patch(module_name, name, obj, allow_new=allow_new)
        return obj

    return deco


def revert(module_name: str, path: str) -> None:
    with _lock:
        rec = _applied.pop((module_name, path))
        if rec.existed:
            setattr(rec.owner, rec.attr, rec.original)
        else:
            delattr(rec.owner, rec.attr)


def revert_all() -> None:
    for rec in list(_applied.values()):
        revert(rec.module, rec.path)
