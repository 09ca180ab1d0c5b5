"""Keeps a package attribute bound to a function when a sub-module of the same name exists.

The reference has modules named after the function they define (``models/build_processor.py`` defines
``build_processor`` and the package re-exports it). Importing such a sub-module, under this package's name or under the
``mindformers`` alias, makes the import system set the package attribute to the module, which would hide a function
that the package defined elsewhere. ``keep_functions`` gives the package a module class whose attribute assignment
ignores a module for the listed names, so ``package.name`` stays the function and ``import package.name`` still
works (the module is in ``sys.modules``)."""
import sys
import types


class _Package(types.ModuleType):
    def __setattr__(self, name, value):
        if isinstance(value, types.ModuleType) and name in self.__dict__.get("_kept_functions", ()):
            return
        super().__setattr__(name, value)


def keep_functions(package_name: str, names):
    pkg = sys.modules[package_name]
    for name in names:
        if isinstance(pkg.__dict__.get(name), types.ModuleType) or name not in pkg.__dict__:
            raise ImportError(f"{package_name}.{name} is not bound to a function")
    pkg.__dict__["_kept_functions"] = tuple(names)
    pkg.__class__ = _Package
