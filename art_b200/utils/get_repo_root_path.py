"""Locate the enclosing git work tree (parity: reference ``src/art/utils/get_repo_root_path.py:4-14``)."""
import os


def get_repo_root_path(start: str | None = None) -> str:
    """Walk up from ``start`` (default: the current working directory) to a directory
    holding ``.git``; fall back to ``"."``."""
    cur = os.path.abspath(start or os.getcwd())
    while True:
        if os.path.exists(os.path.join(cur, ".git")):
            return cur
        parent = os.path.dirname(cur)
        if parent == cur:
            return "."
        cur = parent
