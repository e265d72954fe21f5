"""Puts the unmodified reference under `baseline/_ref` (git-ignored) for `bench.py --impl reference`.

    python baseline/install_reference.py /path/to/reference [/path/to/wheelhouse]

(the source tree may also be named by OTB_REFERENCE_SRC). First tries an offline pip install; where the reference's build
backend (hatchling) is not installed that fails, and because the package is pure Python a plain copy of `src/pretrain`
and `configs` is the install.
"""
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def main() -> int:
    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("OTB_REFERENCE_SRC", "")
    if not where:
        print(__doc__)
        return 2
    src = Path(where)
    dst = HERE / "_ref"
    if not (src / "src" / "pretrain").is_dir():
        print("no reference source tree at %s" % src)
        return 1
    wheels = sys.argv[2] if len(sys.argv) > 2 else os.environ.get("PIP_FIND_LINKS", "")
    pip = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps"] +
                         (["--find-links", wheels] if wheels else []) + ["--target", str(dst), str(src)], capture_output=True, text=True)
    if pip.returncode == 0 and (dst / "pretrain").is_dir():
        print("pip install succeeded")
    else:
        print("pip install failed (%s); copying the pure-Python package instead"
              % (pip.stderr.strip().splitlines() or ["no message"])[-1])
        if (dst / "pretrain").exists():
            shutil.rmtree(dst / "pretrain")
        shutil.copytree(src / "src" / "pretrain", dst / "pretrain")
    if (dst / "configs").exists():
        shutil.rmtree(dst / "configs")
    shutil.copytree(src / "configs", dst / "configs")
    print("reference installed under %s" % dst)
    return 0


if __name__ == "__main__":
    sys.exit(main())
