"""Publish a local model directory (for example a freshly quantised JQ4 model) to a Hugging Face model repository.

    HF_TOKEN=... python -m deliverance_b200.ckpt.upload OWNER/NAME LOCAL_DIR [--private] [--message TEXT] [--dry-run]

Creates the repository when it does not exist and uploads the folder in one commit (reference: scripts/upload_hf_model.py).
``--dry-run`` lists what would be uploaded and needs neither a token nor the network; a directory produced by the quantiser is
refused until its ``.finished`` marker exists.
"""
from __future__ import annotations

import argparse
import os

SKIP = (".finished", ".staging", ".lock", ".tmp")


def plan(local_dir: str) -> list:
    """(relative path, bytes) of every file that would be uploaded, sorted."""
    root = os.path.realpath(os.path.expanduser(local_dir))
    if not os.path.isdir(root):
        raise NotADirectoryError(f"local_dir is not a directory: {root}")
    if os.path.exists(os.path.join(root, "deliverance-quantization.json")) and not os.path.exists(os.path.join(root, ".finished")):
        raise RuntimeError(f"{root} is a quantiser output without its .finished marker: the conversion did not complete")
    out = []
    for d, _, files in os.walk(root):
        for f in files:
            if f.endswith(SKIP) or f.startswith("."):
                continue
            p = os.path.join(d, f)
            out.append((os.path.relpath(p, root), os.path.getsize(p)))
    return sorted(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("repo_id")
    ap.add_argument("local_dir")
    ap.add_argument("--private", action="store_true")
    ap.add_argument("--message", default="Upload Deliverance model")
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    files = plan(a.local_dir)
    total = sum(n for _, n in files)
    print(f"{len(files)} files, {total / 2**20:.1f} MiB -> https://huggingface.co/{a.repo_id}")
    if a.dry_run:
        for rel, n in files:
            print(f"  {n:>12d}  {rel}")
        return 0
    token = os.environ.get("HF_TOKEN")
    if not token:
        raise SystemExit("HF_TOKEN is required")
    try:
        from huggingface_hub import HfApi
    except ImportError as e:
        raise SystemExit(f"huggingface_hub is needed for the upload itself: {e}")
    api = HfApi(token=token)
    api.create_repo(repo_id=a.repo_id, repo_type="model", private=a.private, exist_ok=True)
    api.upload_folder(repo_id=a.repo_id, repo_type="model", folder_path=os.path.realpath(os.path.expanduser(a.local_dir)), commit_message=a.message,
                      ignore_patterns=[".*", "*.tmp"])
    print(f"Uploaded {a.local_dir} to https://huggingface.co/{a.repo_id}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
