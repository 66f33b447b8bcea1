"""Run code written against the reference's package names on this package, unchanged.

``install()`` registers an import hook that resolves ``heuristic_secrets[.x.y]`` and ``zoology[.x.y]`` to
``ml_experiments_b200.heuristic_secrets[.x.y]`` / ``ml_experiments_b200.zoology[.x.y]`` (the same module objects, not
copies: ``heuristic_secrets.models.Model is ml_experiments_b200.heuristic_secrets.models.Model``). A real package of
either name that is importable takes precedence unless ``override=True``.

    import ml_experiments_b200.compat as compat
    compat.install()
    from heuristic_secrets import Detector                      # this package's Detector
    from zoology.mixers.mamba_ssm.ops.selective_scan_interface import selective_scan_fn

``python -m ml_experiments_b200.compat pytest <the reference's tests folder>`` runs a command line with the hook
installed; with the reference's own ``tests/`` this is the drop-in check: every test the reference's code passes there
passes here as well (the ones that clone from the network excepted).
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

ALIASES = {"heuristic_secrets": "ml_experiments_b200.heuristic_secrets", "zoology": "ml_experiments_b200.zoology"}


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def __init__(self, names):
        self.names = dict(names)

    def _real(self, name: str) -> str | None:
        top = name.split(".", 1)[0]
        if top not in self.names:
            return None
        real = self.names[top] + name[len(top):]
        if top == "zoology":      # modules the reference splits into sub-packages and this package keeps in one file
            from .zoology.utils import _MODULE_ALIASES
            real = _MODULE_ALIASES.get(real, real)
        return real

    def _has_aliased_children(self, name: str) -> bool:
        """``name`` is one module here but a package with sub-modules in the reference (``feature_maps``, ``h3``, ...)."""
        if name.split(".", 1)[0] != "zoology":
            return False
        from .zoology.utils import _MODULE_ALIASES
        prefix = self.names["zoology"] + name[len("zoology"):] + "."
        return any(k.startswith(prefix) for k in _MODULE_ALIASES)

    def find_spec(self, name, path=None, target=None):
        real = self._real(name)
        if real is None:
            return None
        try:
            spec = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            spec = None
        children = self._has_aliased_children(name)
        if spec is None and not children:
            return None
        is_pkg = children or spec.submodule_search_locations is not None
        return importlib.util.spec_from_loader(name, self, is_package=is_pkg)

    def create_module(self, spec):
        import types
        try:
            real = importlib.import_module(self._real(spec.name))
        except ImportError:           # a package of the reference with no counterpart of its own here: only its sub-modules map
            empty = types.ModuleType(spec.name)
            empty.__path__ = []
            return empty
        if hasattr(real, "__path__") or not self._has_aliased_children(spec.name):
            return real
        # a single module standing in for a package of the reference: a stand-in with the same contents and an (empty)
        # search path, so that ``import pkg.sub`` reaches this finder for ``sub``
        proxy = types.ModuleType(spec.name, real.__doc__)
        proxy.__dict__.update({k: v for k, v in vars(real).items() if k not in ("__name__", "__spec__", "__loader__", "__path__")})
        proxy.__path__ = []
        return proxy

    def exec_module(self, module):          # the real module is already executed
        return None


def install(override: bool = False) -> list[str]:
    """Install the hook (idempotent). Returns the top-level names it now serves."""
    for f in sys.meta_path:
        if isinstance(f, _AliasFinder):
            return sorted(f.names)
    names = {}
    for top, real in ALIASES.items():
        if not override and top not in sys.modules:
            try:
                if importlib.util.find_spec(top) is not None:
                    continue                      # a real package of that name is installed: leave it alone
            except (ImportError, ValueError):
                pass
        names[top] = real
    finder = _AliasFinder(names)
    sys.meta_path.insert(0, finder)
    return sorted(names)


def uninstall() -> None:
    sys.meta_path[:] = [f for f in sys.meta_path if not isinstance(f, _AliasFinder)]
    for name in [n for n in sys.modules if n.split(".", 1)[0] in ALIASES]:
        if getattr(sys.modules[name], "__name__", name) != name:      # an alias entry, not a real module of that name
            del sys.modules[name]


def main(argv=None) -> int:
    """``python -m ml_experiments_b200.compat <module> [args...]``: ``python -m <module> args`` with the hook installed."""
    import runpy

    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        print(__doc__)
        return 2
    install(override=True)
    sys.argv = argv
    runpy.run_module(argv[0], run_name="__main__", alter_sys=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
