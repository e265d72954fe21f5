"""Provenance: commit and dirty state of this checkout, recorded in every checkpoint."""
from __future__ import annotations

import subprocess
from pathlib import Path

_ROOT = Path(__file__).resolve().parent.parent.parent


def _git(*args: str, cwd: Path | None = None) -> str | None:
    """A read-only git command; None when it fails. ``safe.directory=*``: a checkout on shared storage is often owned by
    another uid than the training process, and git refuses such a tree otherwise."""
    try:
        r = subprocess.run(["git", "-c", "safe.directory=*", *args], cwd=str(cwd or _ROOT), capture_output=True, text=True, timeout=10)
        return r.stdout.strip() if r.returncode == 0 else None
    except Exception:
        return None


def git_sha(cwd: Path | None = None) -> str:
    return _git("rev-parse", "HEAD", cwd=cwd) or "unknown"


def git_diff(cwd: Path | None = None, max_bytes: int = 200_000) -> str:
    d = _git("diff", "HEAD", cwd=cwd) or ""
    return d[:max_bytes]


def repo_provenance(name: str, start: Path | None = None) -> dict:
    """Commit, branch and dirty flag of the checkout that encloses ``start`` (any path inside it; default: this package).
    A copy without ``.git`` gives ``available: False`` and a run carries on.
    (role of the reference's src/pretrain/util/git.py:97-118)"""
    start = Path(start) if start is not None else _ROOT
    start = start if start.is_dir() else start.parent
    out = {"name": name, "available": False, "root": None, "commit": None, "branch": None, "dirty": None}
    root = _git("rev-parse", "--show-toplevel", cwd=start)
    if not root:
        return out
    status = _git("status", "--porcelain", cwd=Path(root))
    out.update(available=True, root=root, commit=_git("rev-parse", "--short=12", "HEAD", cwd=Path(root)),
               branch=_git("rev-parse", "--abbrev-ref", "HEAD", cwd=Path(root)), dirty=None if status is None else bool(status.strip()))
    return out


def describe_provenance(p: dict) -> str:
    if not p.get("available"):
        return "%s=unknown (no .git)" % p["name"]
    return "%s=%s@%s (%s)" % (p["name"], p["commit"], p["branch"], "dirty" if p["dirty"] else "clean")


def native_source_digests() -> dict:
    """{library: sha256 of its sources and compiler flags} for every native library built in this checkout (the stamp the
    build writes beside each library): two machines that report the same digests ran the same kernels."""
    ext = _ROOT / "open_transformers_b200" / "_ext"
    return {p.stem: p.read_text().strip() for p in sorted(ext.glob("*.stamp"))} if ext.is_dir() else {}


def run_provenance() -> dict:
    from .. import __version__, build_info
    from ..ops import native

    return {"framework": "open_transformers_b200", "version": __version__, "git_sha": git_sha(), "dirty": bool(git_diff()),
            "repo": repo_provenance("open_transformers_b200"), "backends": build_info()["backends"],
            "native_libs": native.loaded_libraries(), "native_source_digests": native_source_digests()}
