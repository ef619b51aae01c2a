"""
Upload a converted checkpoint directory to a branch of a Hugging Face Hub repository (the role of
src/examples/huggingface/upload_checkpoint_to_hf.py)::

    python examples/huggingface/upload_checkpoint_to_hf.py --local-checkpoint-dir /tmp/my-run-hf \
        --repo-id my-org/my-model --branch step1000 [--token ...] [--dry-run]

The branch is created when it does not exist. Files are sent one by one so that a failed file is reported and the rest
still go up; the exit code is 1 if any file failed. The token is read from ``$HF_TOKEN`` when not given. ``--dry-run``
lists what would be uploaded and needs neither a token nor the ``huggingface_hub`` package.
"""

import argparse
import os
import sys
from typing import List, Tuple


def files_to_upload(local_dir: str) -> List[Tuple[str, str]]:
    """``(local path, path in the repository)`` of every file under ``local_dir``, in a stable order."""
    pairs = []
    for root, _, names in os.walk(local_dir):
        for name in names:
            local = os.path.join(root, name)
            pairs.append((local, os.path.relpath(local, local_dir).replace(os.sep, "/")))
    return sorted(pairs, key=lambda p: p[1])


def upload(local_dir: str, repo_id: str, branch: str, token: str) -> int:
    from huggingface_hub import HfApi

    api = HfApi(token=token)
    try:
        api.create_branch(repo_id=repo_id, branch=branch, exist_ok=True)
    except Exception as e:  # an older hub client without `exist_ok`, or a branch that is already there
        print(f"could not create branch '{branch}' ({e}); uploading to it anyway")
    failed = 0
    pairs = files_to_upload(local_dir)
    for i, (local, remote) in enumerate(pairs, 1):
        try:
            api.upload_file(path_or_fileobj=local, path_in_repo=remote, repo_id=repo_id, revision=branch)
            print(f"[{i}/{len(pairs)}] {remote}")
        except Exception as e:
            failed += 1
            print(f"[{i}/{len(pairs)}] {remote}: FAILED ({e})")
    return failed


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--local-checkpoint-dir", "--local_checkpoint_dir", required=True)
    ap.add_argument("--repo-id", "--repo_id", required=True)
    ap.add_argument("--branch", default="main")
    ap.add_argument("--token", default=None)
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    if not os.path.isdir(args.local_checkpoint_dir):
        print(f"not a directory: {args.local_checkpoint_dir}")
        return 1
    if args.dry_run:
        for _, remote in files_to_upload(args.local_checkpoint_dir):
            print(f"would upload {remote} -> {args.repo_id}@{args.branch}")
        return 0
    token = args.token or os.environ.get("HF_TOKEN")
    if not token:
        print("a token is required (--token or $HF_TOKEN)")
        return 1
    return 1 if upload(args.local_checkpoint_dir, args.repo_id, args.branch, token) else 0


if __name__ == "__main__":
    sys.exit(main())
