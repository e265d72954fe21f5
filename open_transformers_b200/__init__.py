"""B200-native bitwise-reproducible pretraining and audit-replay framework."""
__version__ = "0.1.0"


def build_info() -> dict:
    """What this installation can run and where it came from: ``{"version", "commit", "python_native", "backends",
    "native_source_digests"}``. ``backends`` lists ``cpu`` when the twin library is built and ``cuda`` when the sm_100a library
    is; ``commit`` comes from the stamp a wheel build writes (``_build_info.json``) or, in a checkout, from git. The replay
    records it in every result, and refuses a GPU replay on an installation without the GPU library.
    (role of the reference kernel library's ``build_info()``: src/pretrain/cli/audit_replay.py:1114-1141)"""
    import json
    from pathlib import Path

    from .utils.git import git_sha, native_source_digests

    here = Path(__file__).resolve().parent
    stamp = {}
    if (here / "_build_info.json").is_file():
        try:
            stamp = json.loads((here / "_build_info.json").read_text())
        except ValueError:
            stamp = {}
    backends = [name for name, lib in (("cpu", "libotb_cpu.so"), ("cuda", "libotb_cuda.so")) if (here / "_ext" / lib).is_file()]
    return {"version": __version__, "commit": stamp.get("commit") or git_sha(), "python_native": bool(stamp.get("python_native", False)),
            "backends": backends, "native_source_digests": native_source_digests()}
