"""Puts the unmodified reference under `baseline/_ref` (git-ignored) for `bench.py --impl reference`.

    python baseline/install_reference.py [/path/to/reference]

First tries the offline pip install; the reference's build backend (hatchling) is not on this image, so that
fails, and because the package is pure Python a plain copy of `src/pretrain` and `configs` is the install.
"""
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def main() -> int:
    src = Path(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
    dst = HERE / "_ref"
    if not (src / "src" / "pretrain").is_dir():
        print("no reference source tree at %s" % src)
        return 1
    pip = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--find-links",
                          "/opt/wheelhouse", "--target", str(dst), str(src)], capture_output=True, text=True)
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
