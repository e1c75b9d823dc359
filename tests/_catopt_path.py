"""Where the tests find catopt (the reference): not a test module.

Tried in order: ``$CATOPT_SRC`` (a source checkout: ``packages/*/src``), a
``reference`` checkout next to this repository, and ``baseline/_ref`` inside it
(an offline ``pip install --target`` of catopt's packages, which is what a GPU
box has).  ``add_catopt_to_path()`` returns the layout it used, or ``None``.
"""
from __future__ import annotations

import glob
import os
import sys

_ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def add_catopt_to_path() -> str | None:
    try:
        import catopt_core  # noqa: F401

        return "already importable"
    except ImportError:
        pass
    for root in (os.environ.get("CATOPT_SRC"), os.path.join(_ROOT, "..", "reference")):
        srcs = sorted(glob.glob(os.path.join(root, "packages", "*", "src"))) if root else []
        if srcs:
            for p in srcs:
                if p not in sys.path:
                    sys.path.insert(0, p)
            return f"source tree {os.path.abspath(root)}"
    target = os.path.join(_ROOT, "baseline", "_ref")
    if os.path.isdir(os.path.join(target, "catopt_core")):
        if target not in sys.path:
            sys.path.insert(0, target)
        return "baseline/_ref"
    return None


SKIP_REASON = ("catopt is not importable: no $CATOPT_SRC, no ../reference checkout and no baseline/_ref "
               "(install it with `python -m catopt_b200.install_reference <catopt checkout>`)")
