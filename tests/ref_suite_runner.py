#!/usr/bin/env python
"""Run the reference's own unittest modules, unmodified, with the B200 executor installed (or with the reference's own).

    python tests/ref_suite_runner.py --executor b200|b200_plan|reference [--json out.json] tests.test_frontend tests.test_bmm4x4 ...

Child process of ``tests/test_gpu_reference_suite.py``: the reference package and its ``tests`` package are imported from
``baseline/_ref`` (installed by ``baseline/build_ref.py``), ``gint_b200.install()`` swaps the executor in through the reference's
own seam (``gint/host/executor.py:212-233``), and ``unittest`` runs the named modules. Prints one JSON object: per test id its
outcome (``ok`` / ``fail`` / ``error`` / ``skip``) and, for failures, the last line of the traceback.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import unittest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


class _Collect(unittest.TextTestResult):
    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.outcomes: dict[str, dict] = {}

    def addSuccess(self, test):
        super().addSuccess(test)
        self.outcomes[test.id()] = {"outcome": "ok"}

    def addFailure(self, test, err):
        super().addFailure(test, err)
        self.outcomes[test.id()] = {"outcome": "fail", "why": self._short(err)}

    def addError(self, test, err):
        super().addError(test, err)
        self.outcomes[test.id()] = {"outcome": "error", "why": self._short(err)}

    def addSkip(self, test, reason):
        super().addSkip(test, reason)
        self.outcomes[test.id()] = {"outcome": "skip", "why": reason}

    def addSubTest(self, test, subtest, err):
        super().addSubTest(test, subtest, err)
        if err is not None:
            self.outcomes[subtest.id()] = {"outcome": "fail", "why": self._short(err)}

    @staticmethod
    def _short(err) -> str:
        return f"{err[0].__name__}: {str(err[1]).strip().splitlines()[-1][:300] if str(err[1]).strip() else ''}"


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--executor", choices=["b200", "b200_plan", "reference"], default="b200",
                    help="b200_plan: also launch conductor-compiled graphs through gint_execute_plan (gint_b200/conductor_fastpath.py)")
    ap.add_argument("--json", default=None)
    ap.add_argument("modules", nargs="+")
    o = ap.parse_args()
    # the reference tree first: `gint` and `tests` must be ITS packages; then this repository for gint_b200
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != os.path.join(ROOT, "tests")]
    sys.path.insert(0, ROOT)
    sys.path.insert(0, REF)
    import torch
    torch.cuda.init()
    torch.zeros(1, device="cuda")          # the reference asks for an existing CUDA context (gint/host/cuda/driver.py:84-95)
    loaded = None
    if o.executor in ("b200", "b200_plan"):
        import gint_b200
        ex = gint_b200.install(accelerate_conductor=(o.executor == "b200_plan"))
        loaded = type(ex).__mro__[1].__name__
    suite = unittest.TestSuite()
    loader = unittest.TestLoader()
    for m in o.modules:
        suite.addTests(loader.loadTestsFromName(m))
    runner = unittest.TextTestRunner(stream=sys.stderr, verbosity=1, resultclass=_Collect)
    result = runner.run(suite)
    import gint.host.executor as gx
    out = {"executor": o.executor, "executor_class": type(gx.executor).__name__ if gx.executor is not None else None, "installed": loaded,
           "gint_from": os.path.relpath(os.path.dirname(gx.__file__), ROOT), "launches": getattr(gx.executor, "launches", None),
           "run": result.testsRun, "outcomes": result.outcomes}
    text = json.dumps(out)
    if o.json:
        with open(o.json, "w") as f:
            f.write(text)
    print(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
