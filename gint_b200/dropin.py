"""Install the B200 executor into an installed ``gint`` package, so that gint's own frontend, small-matrix helpers and
torch.compile backend run on these kernels without any change to gint.

    import gint_b200
    gint_b200.install()                 # before the first gint call
    torch.compile(fn, backend="gint")   # gint's conductor now launches through libgint_b200.so

The seam is the one the reference provides itself: ``gint.host.executor.BaseExecutor`` reached through the module-global
``gint.host.executor.executor`` that ``get_executor()`` returns (``gint/host/executor.py:200-233``). ``install`` makes a
``B200Executor`` that is also a subclass of that package's ``BaseExecutor`` and assigns it to the global. Everything that
asks ``get_executor()`` afterwards -- ``BaseExecutableProgram.__call__`` (``executor.py:170-171``), the conductor's compiled
``execute`` closure (``gint/conductor/compiler.py:1438-1466``), ``tests/test_indirect.py`` -- gets it; gint's own
``CudaExecutor`` and its fatbin are never loaded.
"""
from __future__ import annotations

import importlib
import sys
from typing import Optional

from .host.executor import B200Executor

_installed: dict = {}


def install(package_path: Optional[str] = None, accelerate_conductor: bool = False):
    """Make the B200 executor the executor of the importable ``gint`` package and return it.

    ``package_path``: a directory to put in front of ``sys.path`` first (the folder that contains ``gint/``), for a gint
    that is not installed into the environment. Calling ``install`` again returns the executor already installed.
    ``accelerate_conductor``: also route the launches of graphs compiled by ``gint.conductor`` from now on through
    ``gint_execute_plan`` (``gint_b200/conductor_fastpath.py``: one library call per run of consecutive subgraphs instead of a
    Python-level ``execute`` per subgraph; the conductor's source is not touched).
    """
    if package_path and package_path not in sys.path:
        sys.path.insert(0, package_path)
    gx = importlib.import_module("gint.host.executor")
    cur = getattr(gx, "executor", None)
    if cur is not None and isinstance(cur, B200Executor):
        if accelerate_conductor:
            from . import conductor_fastpath
            conductor_fastpath.patch_conductor(cur)
        return cur
    cls = _installed.get(id(gx.BaseExecutor))
    if cls is None:
        cls = type("B200DropInExecutor", (B200Executor, gx.BaseExecutor), {
            "__doc__": "B200Executor registered as a gint.host.executor.BaseExecutor (see gint_b200.dropin.install)."})
        _installed[id(gx.BaseExecutor)] = cls
    _installed["previous"] = cur
    gx.executor = cls()
    if accelerate_conductor:
        from . import conductor_fastpath
        conductor_fastpath.patch_conductor(gx.executor)
    return gx.executor


def uninstall() -> None:
    """Put back whatever executor gint had before ``install`` (None: gint picks its own on next use)."""
    from . import conductor_fastpath
    conductor_fastpath.unpatch_conductor()
    gx = sys.modules.get("gint.host.executor")
    if gx is not None and isinstance(getattr(gx, "executor", None), B200Executor):
        gx.executor = _installed.get("previous")
