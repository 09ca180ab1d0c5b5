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
        if isinstance(value, types.ModuleType) and (name in self.__dict__.get("_kept_functions", ()) or (
                name in self.__dict__ and not isinstance(self.__dict__[name], types.ModuleType))):
            return
        super().__setattr__(name, value)


def keep_functions(package_name: str, names):
    pkg = sys.modules[package_name]
    for name in names:
        if isinstance(pkg.__dict__.get(name), types.ModuleType) or name not in pkg.__dict__:
            raise ImportError(f"{package_name}.{name} is not bound to a function")
    pkg.__dict__["_kept_functions"] = tuple(names)
    _guard(pkg)


def _guard(mod):
    """Gives ``mod`` the guarded attribute assignment, keeping what its current module class adds (e.g. ``__call__``)."""
    cls = type(mod)
    if issubclass(cls, _Package):
        return
    mod.__class__ = _Package if cls is types.ModuleType else type(cls.__name__, (_Package, cls), {})


# ---- reference paths below a module that is a single file here -------------------------------------------------------
# The reference splits some packages over several files (``core/callback/callback.py`` + ``build_callback.py``) that
# are one module here (``core/callback.py``). ``alias_children(module, children)`` lets ``import module.child``
# resolve: the module gets an empty ``__path__`` (which is what makes the import system look for children at all) and
# a finder returns, for each listed child, the module itself (or another module given by name).
import importlib
import importlib.abc
import importlib.util

_CHILDREN = {}


class _SameModuleLoader(importlib.abc.Loader):
    def __init__(self, target: str):
        self.target = target

    def create_module(self, spec):
        module = importlib.import_module(self.target)
        self._spec = module.__spec__          # the import system rebinds ``__spec__`` to the alias's; put it back
        return module

    def exec_module(self, module):
        module.__spec__ = self._spec


_NODES = set()


class _EmptyPackageLoader(importlib.abc.Loader):
    def create_module(self, spec):
        return None

    def exec_module(self, module):
        module.__doc__ = "Directory level of a reference module path; the leaves below it resolve to modules of this package."


class _ChildFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        real = _CHILDREN.get(fullname)
        if real is not None:
            return importlib.util.spec_from_loader(fullname, _SameModuleLoader(real))
        if fullname in _NODES:
            return importlib.util.spec_from_loader(fullname, _EmptyPackageLoader(), is_package=True)
        return None


def _install_finder():
    if not any(isinstance(f, _ChildFinder) for f in sys.meta_path):
        sys.meta_path.append(_ChildFinder())


def register_paths(root: str, table):
    """``table``: ``{"a.b.leaf": "x.y"}`` relative to package ``root``: ``root.a.b.leaf`` resolves to module ``root.x.y``;
    directory levels that do not exist (``root.a.b``) become empty packages."""
    for rel, target in table.items():
        _CHILDREN.setdefault(f"{root}.{rel}", f"{root}.{target}")
        parts = rel.split(".")
        for i in range(1, len(parts)):
            _NODES.add(f"{root}." + ".".join(parts[:i]))
    _install_finder()


def alias_children(module_name: str, children):
    """``children``: names (resolve to ``module_name`` itself) or ``(name, target module)`` pairs."""
    mod = sys.modules[module_name]
    if not hasattr(mod, "__path__"):
        mod.__path__ = []
    for child in children:
        name, target = (child, module_name) if isinstance(child, str) else child
        _CHILDREN[f"{module_name}.{name}"] = target
    _install_finder()
    mod.__dict__.setdefault("_kept_functions", ())
    _guard(mod)
