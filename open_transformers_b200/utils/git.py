"""Provenance: commit and dirty state of this checkout, recorded in every checkpoint."""
from __future__ import annotations

import subprocess
from pathlib import Path

_ROOT = Path(__file__).resolve().parent.parent.parent


def _git(*args: str, cwd: Path | None = None) -> str | None:
    try:
        r = subprocess.run(["git", *args], cwd=str(cwd or _ROOT), capture_output=True, text=True, timeout=10)
        return r.stdout.strip() if r.returncode == 0 else None
    except Exception:
        return None


def git_sha(cwd: Path | None = None) -> str:
    return _git("rev-parse", "HEAD", cwd=cwd) or "unknown"


def git_diff(cwd: Path | None = None, max_bytes: int = 200_000) -> str:
    d = _git("diff", "HEAD", cwd=cwd) or ""
    return d[:max_bytes]


def native_source_digests() -> dict:
    """{library: sha256 of its sources and compiler flags} for every native library built in this checkout (the stamp the
    build writes beside each library): two machines that report the same digests ran the same kernels."""
    ext = _ROOT / "open_transformers_b200" / "_ext"
    return {p.stem: p.read_text().strip() for p in sorted(ext.glob("*.stamp"))} if ext.is_dir() else {}


def run_provenance() -> dict:
    from .. import __version__
    from ..ops import native

    return {"framework": "open_transformers_b200", "version": __version__, "git_sha": git_sha(), "dirty": bool(git_diff()),
            "native_libs": native.loaded_libraries(), "native_source_digests": native_source_digests()}
