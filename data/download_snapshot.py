"""Download a dataset repository from the Hugging Face Hub into ``downloads/<repo_id>``
(data/download_snapshot.py of the reference). Needs network access and ``huggingface_hub``.

    python data/download_snapshot.py --repo_id openai/prm800k [--hf_token ...]
"""
from __future__ import annotations

import argparse
import os
from typing import Optional


def hf_download(repo_id: str, hf_token: Optional[str] = None, root: str = "downloads") -> str:
    from huggingface_hub import snapshot_download
    target = os.path.join(root, repo_id)
    os.makedirs(target, exist_ok=True)
    try:
        snapshot_download(repo_id, local_dir=target, token=hf_token, repo_type="dataset")
    except Exception as e:  # noqa: BLE001
        status = getattr(getattr(e, "response", None), "status_code", None)
        if status == 401:
            print("You need to pass a valid `--hf_token=...` to download private downloads.")
        else:
            raise
    return target


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description="Download data from HuggingFace Hub.")
    ap.add_argument("--repo_id", type=str, required=True)
    ap.add_argument("--hf_token", type=str, default=None)
    a = ap.parse_args()
    hf_download(a.repo_id, a.hf_token)
