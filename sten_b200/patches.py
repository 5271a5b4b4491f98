"""``patch(old, new, module_scope)``: replace a function everywhere it is referenced inside a set of modules.

Reference: src/sten/patches.py:21-54.  Only this generic helper belongs to the grouped n:m path; the DDP gradient hook
and the Apex optimizer patches of the reference are training plumbing and are not provided.
"""
import inspect
import sys


def _callables(owner):
    for name, member in inspect.getmembers(owner):
        if callable(member) and not inspect.isclass(member):
            yield name, member


def patch(old, new, module_scope=None):
    """Rebind every module-level name and every class attribute in ``module_scope`` that is ``old`` to ``new``.

    ``module_scope`` defaults to all currently imported ``torch*`` modules, as in the reference."""
    if module_scope is None:
        module_scope = [m for name, m in list(sys.modules.items()) if name.startswith("torch") and m is not None]
    for mod in module_scope:
        for _, cls in inspect.getmembers(mod, inspect.isclass):
            for name, member in _callables(cls):
                if member is old:
                    setattr(cls, name, new)
        for name, member in _callables(mod):
            if member is old:
                setattr(mod, name, new)
