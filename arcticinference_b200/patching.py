"""Class-patching utility.

This engine owns its scheduler, runner and models, so nothing inside it is patched.
The utility is kept as part of the public surface for users who extend third-party
classes the way the reference extends vLLM (arctic_inference/patching.py:85-139):

    class MyPatch(ArcticPatch[Target]):
        def method(self): ...
    MyPatch.apply_patch()

copies every attribute defined in ``MyPatch`` onto ``Target`` (classmethods are re-bound,
so ``cls`` is the class they are called on), records the origin of each attribute in
``Target._arctic_patches`` and refuses to patch the same attribute twice.
"""

from __future__ import annotations

from typing import Generic, TypeVar

T = TypeVar("T")

_SKIP = frozenset(("__dict__", "__weakref__", "__module__", "__doc__", "__qualname__",
                   "__orig_bases__", "__parameters__", "__annotations__", "__firstlineno__",
                   "__static_attributes__", "_arctic_patch_target"))


class ArcticPatch(Generic[T]):
    _arctic_patch_target = None

    def __class_getitem__(cls, target):
        if isinstance(target, TypeVar):
            return super().__class_getitem__(target)
        if not isinstance(target, type):
            raise TypeError("ArcticPatch[...] expects a class, got %r" % (target,))
        # a fresh base class that remembers what it patches
        return type("%s[%s]" % (cls.__name__, target.__name__), (cls,),
                    {"_arctic_patch_target": target})

    @classmethod
    def apply_patch(cls) -> None:
        target = cls._arctic_patch_target
        if target is None:
            raise TypeError("%s does not name a target; subclass ArcticPatch[Target]" % cls.__name__)
        if "_arctic_patches" not in target.__dict__:
            target._arctic_patches = {}
        for name, value in list(cls.__dict__.items()):
            if name in _SKIP:
                continue
            owner = target._arctic_patches.get(name)
            if owner is not None:
                raise ValueError("%s.%s is already patched by %s" %
                                 (target.__name__, name, owner.__name__))
            if isinstance(value, classmethod):
                # bind through the descriptor protocol so that subclasses receive themselves
                value = classmethod(value.__func__)
            setattr(target, name, value)
            target._arctic_patches[name] = cls
