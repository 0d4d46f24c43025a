"""Puts an UNMODIFIED MagiCompiler next to this package so the GPU tests can run the fused op under the real thing.

    python baseline/install_reference.py [path/to/MagiCompiler]

Installs the checkout (``$MAGI_COMPILER_ROOT``, the argument, or a directory ``reference`` beside this repository)
with pip, offline, into ``baseline/_ref/`` (not tracked by git), copies the checkout's own ``tests/`` folder to
``baseline/_ref/reference_tests/tests`` (the GPU tests import ``tests.model_definition`` from there and run a few of
the reference's own test files with this package loaded), and writes the one-class ``graphviz`` stand-in the
package's visualisation modules import at load time.  Nothing from the checkout enters the git history.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
TARGET = ROOT / "baseline" / "_ref"
WHEELHOUSE = Path("/opt/wheelhouse")


def find_checkout(arg: str | None = None) -> Path | None:
    for cand in (arg, os.environ.get("MAGI_COMPILER_ROOT"), ROOT.parent / "reference"):
        if cand and (Path(cand) / "magi_compiler" / "__init__.py").exists():
            return Path(cand)
    return None


def install(checkout: Path | None = None, force: bool = False) -> Path | None:
    """Returns ``baseline/_ref`` once it holds the package, or None when there is no checkout to install from."""
    checkout = checkout or find_checkout()
    have = (TARGET / "magi_compiler" / "__init__.py").exists()
    if checkout is None:
        return TARGET if have else None
    if have and not force:
        newest_src = max(p.stat().st_mtime for p in (checkout / "magi_compiler").rglob("*.py"))
        if (TARGET / "magi_compiler" / "__init__.py").stat().st_mtime >= newest_src and \
                (TARGET / "reference_tests" / "tests" / "model_definition.py").exists():
            return TARGET
    if TARGET.exists():
        shutil.rmtree(TARGET)
    TARGET.mkdir(parents=True)
    base = [sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation", "--target", str(TARGET)]
    if WHEELHOUSE.exists():
        base += ["--find-links", str(WHEELHOUSE)]
    proc = subprocess.run(base + [str(checkout)], capture_output=True, text=True)
    if proc.returncode != 0:  # dependency resolution is the usual reason: the image already has the dependencies
        proc = subprocess.run(base + ["--no-deps", str(checkout)], capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"pip could not install {checkout} into {TARGET}:\n{proc.stdout}\n{proc.stderr}")
    shutil.copytree(checkout / "tests", TARGET / "reference_tests" / "tests",
                    ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    (TARGET / "graphviz.py").write_text("class Digraph:  # stand-in: the real package is only CALLED behind a debug flag\n    pass\n")
    return TARGET


if __name__ == "__main__":
    where = install(find_checkout(sys.argv[1] if len(sys.argv) > 1 else None), force="--force" in sys.argv)
    print(where if where else "no MagiCompiler checkout found; nothing installed")
