"""Packaging hooks (the metadata itself lives in pyproject.toml).

* Every build first compiles the two native libraries in-tree (``open_transformers_b200/_ext/libotb_{cpu,cuda}.so``, see
  ``build_native.py``) so that a wheel carries them; ``OTB_SKIP_NATIVE_BUILD=1`` packages whatever is already there.
* ``PRETRAIN_PYTHON_NATIVE=1`` produces the *compiled* audit distribution: every Python module of the package except the
  ``__init__`` / ``__main__`` files is translated by Cython and compiled with ``-ffp-contract=off`` (host arithmetic must
  not fuse multiply-adds behind the back of the kernels' twins), the ``.py`` sources of the compiled modules are left out
  of the wheel, and ``_build_info.json`` records the commit the wheel was built from (``PRETRAIN_BUILD_COMMIT`` or
  ``git rev-parse HEAD``). Such a build cannot be editable. Ordinary development wheels stay pure Python + the two
  libraries. (reference hatch_build.py:114-172, docs/native-python-wheels.md)
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent
PKG = "open_transformers_b200"
NATIVE = os.environ.get("PRETRAIN_PYTHON_NATIVE") == "1"
KEEP_AS_SOURCE = {"__init__.py", "__main__.py", "build_native.py"}


def compiled_modules(root: Path = ROOT) -> list[Path]:
    """The package's Python files that the compiled distribution ships as extension modules."""
    return sorted(p for p in (root / PKG).rglob("*.py") if p.name not in KEEP_AS_SOURCE and "csrc" not in p.parts and "_ext" not in p.parts)


def build_commit(root: Path = ROOT) -> str:
    commit = os.environ.get("PRETRAIN_BUILD_COMMIT", "")
    if not commit:
        r = subprocess.run(["git", "rev-parse", "HEAD"], cwd=root, capture_output=True, text=True)
        commit = r.stdout.strip() if r.returncode == 0 else "unknown"
    return commit


def cython_extensions(modules: list[Path], root: Path = ROOT, build_dir: str | None = None):
    from Cython.Build import cythonize
    from setuptools import Extension

    exts = [Extension(".".join(p.relative_to(root).with_suffix("").parts), [str(p)], extra_compile_args=["-O2", "-ffp-contract=off", "-fno-fast-math"])
            for p in modules]
    return cythonize(exts, language_level=3, build_dir=build_dir, compiler_directives={"annotation_typing": False, "binding": True}, quiet=True)


class BuildPy(build_py):
    def run(self):
        if os.environ.get("OTB_SKIP_NATIVE_BUILD") != "1":
            sys.path.insert(0, str(ROOT))
            from open_transformers_b200 import build_native

            build_native.build()
        (ROOT / PKG / "_build_info.json").write_text(json.dumps({"commit": build_commit(), "python_native": NATIVE}) + "\n")
        super().run()

    def find_package_modules(self, package, package_dir):
        found = super().find_package_modules(package, package_dir)
        if not NATIVE:
            return found
        hidden = {str(p) for p in compiled_modules()}
        return [(pkg, mod, path) for pkg, mod, path in found if str(Path(path).resolve()) not in hidden]


def main() -> None:
    if NATIVE and any(a in ("develop", "editable_wheel") for a in sys.argv):
        raise SystemExit("PRETRAIN_PYTHON_NATIVE=1 builds cannot be editable")
    kwargs = {"cmdclass": {"build_py": BuildPy}, "package_data": {PKG: ["_build_info.json"]}}
    if NATIVE:
        kwargs["ext_modules"] = cython_extensions(compiled_modules())
    setup(**kwargs)


if __name__ == "__main__":
    main()
