"""
Git state of the working tree, as recorded with a launched job (role of src/olmo_core/launch/utils.py:14-90).
The repository is queried with the ``git`` command line, so no Python git binding is required.
"""

from __future__ import annotations

import os
import subprocess
from dataclasses import dataclass
from typing import Optional, Tuple

from ..config import Config

__all__ = ["GIT_REPO_URL_ENV_VAR", "GIT_REF_ENV_VAR", "GIT_BRANCH_ENV_VAR", "parse_git_remote_url", "GitConfig"]

GIT_REPO_URL_ENV_VAR = "REPO_URL"
GIT_REF_ENV_VAR = "GIT_REF"
GIT_BRANCH_ENV_VAR = "GIT_BRANCH"


def parse_git_remote_url(url: str) -> Tuple[str, str]:
    """``git@github.com:acct/repo.git`` or ``https://github.com/acct/repo(.git)`` → ``("acct", "repo")``."""
    if "github.com" not in url:
        raise ValueError(f"Remote ('{url}') must point to a GitHub repo")
    path = url.split("github.com", 1)[1].strip("/:")
    if path.endswith(".git"):
        path = path[: -len(".git")]
    parts = path.split("/")
    if len(parts) != 2 or not all(parts):
        raise ValueError(f"Failed to parse GitHub repo path from remote '{url}'")
    return parts[0], parts[1]


def _git(*args: str) -> Optional[str]:
    try:
        out = subprocess.run(["git", *args], capture_output=True, text=True, check=True)
    except (OSError, subprocess.CalledProcessError):
        return None
    return out.stdout.strip()


@dataclass
class GitConfig(Config):
    repo_url: str
    ref: str
    branch: Optional[str] = None

    @property
    def is_dirty(self) -> bool:
        status = _git("status", "--porcelain", "--untracked-files=no")
        return bool(status)

    @property
    def is_public(self) -> bool:
        import requests

        response = requests.get(self.repo_url)
        if response.status_code not in (200, 404):
            response.raise_for_status()
        return response.status_code == 200

    @classmethod
    def from_env(cls) -> Optional["GitConfig"]:
        """From the repository in the current directory; environment variables override what git reports."""
        head = _git("rev-parse", "HEAD")
        if head is None:
            return None
        ref = os.environ.get(GIT_REF_ENV_VAR, head)
        branch = os.environ.get(GIT_BRANCH_ENV_VAR)
        remote_name = "origin"
        upstream = _git("rev-parse", "--abbrev-ref", "--symbolic-full-name", "@{upstream}")  # e.g. origin/main
        if upstream and "/" in upstream:
            remote_name, tracked = upstream.split("/", 1)
            branch = branch or tracked
        repo_url = os.environ.get(GIT_REPO_URL_ENV_VAR)
        if repo_url is None:
            remote_url = _git("remote", "get-url", remote_name)
            if remote_url is None:
                return None
            account, name = parse_git_remote_url(remote_url)
            repo_url = f"https://github.com/{account}/{name}"
        return cls(repo_url=repo_url, ref=ref, branch=branch)
