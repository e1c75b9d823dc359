"""Install catopt (the reference) next to this package for the GPU tests.

    python -m catopt_b200.install_reference /path/to/catopt [target]

catopt's root project is a meta distribution with nothing importable; its code lives in
``packages/*`` (pure-Python src layouts).  Each of them is installed, offline and
without dependency resolution (torch and numpy are already here), into
``baseline/_ref`` at the repository root — the place ``tests/_catopt_path.py``
looks for when there is no source checkout.  The checkout is copied to a scratch
directory first because a setuptools build writes ``*.egg-info`` beside the
sources and the checkout may be read-only.  ``catopt-native`` (Rust) is skipped.
"""
from __future__ import annotations

import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

PACKAGES = ["catopt-core", "catopt-torch", "catopt-carriers", "catopt-orchestrator", "catopt-cuda",
            "catopt-discovery", "catopt-onnx"]
DEFAULT_TARGET = Path(__file__).resolve().parent.parent / "baseline" / "_ref"


def install(checkout: str | Path, target: str | Path = DEFAULT_TARGET) -> Path:
    checkout, target = Path(checkout), Path(target)
    if not (checkout / "packages" / "catopt-core").is_dir():
        raise SystemExit(f"{checkout} is not a catopt checkout (no packages/catopt-core)")
    target.mkdir(parents=True, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        for name in PACKAGES:
            src = Path(tmp) / name
            shutil.copytree(checkout / "packages" / name, src)
            subprocess.check_call([sys.executable, "-m", "pip", "install", "--quiet", "--no-index",
                                   "--no-build-isolation", "--no-deps", "--upgrade", "--target", str(target),
                                   str(src)])
    return target


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    print(install(*sys.argv[1:3]))
