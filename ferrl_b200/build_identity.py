"""Build/source identity: which commit is running, and whether the tree is clean.

The reference embeds the git commit at build time and ``train`` refuses a dirty
tree (``crates/ferrl/build.rs:327-362``, ``README.md:236-239``) so a run
directory can always be traced to source.  Here the identity is read from git at
launch (Python has no build step); ``FERRL_B200_ALLOW_DIRTY=1`` or
``allow_dirty`` relaxes the gate for development.
"""
from __future__ import annotations

import os
import subprocess
from dataclasses import dataclass
from typing import Optional


class BuildIdentityError(RuntimeError):
    pass


@dataclass(frozen=True)
class BuildIdentity:
    commit: str
    dirty: bool

    def to_json(self):
        return {"git_commit": self.commit, "git_dirty": self.dirty}


def _git(args, cwd):
    return subprocess.run(["git"] + args, cwd=cwd, capture_output=True, text=True, timeout=30)


def source_identity(root: Optional[str] = None) -> BuildIdentity:
    root = root or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        head = _git(["rev-parse", "HEAD"], root)
        if head.returncode != 0:
            return BuildIdentity("unknown", True)
        st = _git(["status", "--porcelain", "--untracked-files=no"], root)
        return BuildIdentity(head.stdout.strip(), st.returncode != 0 or st.stdout.strip() != "")
    except (OSError, subprocess.TimeoutExpired):
        return BuildIdentity("unknown", True)


def require_clean(identity: BuildIdentity, allow_dirty: bool = False) -> None:
    if allow_dirty or os.environ.get("FERRL_B200_ALLOW_DIRTY") == "1":
        return
    if identity.commit == "unknown":
        raise BuildIdentityError("cannot determine the source commit (not a git checkout); set "
                                 "FERRL_B200_ALLOW_DIRTY=1 to run anyway")
    if identity.dirty:
        raise BuildIdentityError(f"the source tree at {identity.commit[:12]} has uncommitted changes; commit them "
                                 "or set FERRL_B200_ALLOW_DIRTY=1 so the run can be traced to its source")
