"""Download a model repository from the Hugging Face Hub into ``<local_dir>/<repo_id>``
(scripts/download.py of the reference). Needs network access and ``huggingface_hub``.

    python scripts/download.py --repo_id EleutherAI/llemma_7b --local_dir checkpoints
"""
from __future__ import annotations

import argparse
import os
from typing import Optional


def hf_download(repo_id: str, hf_token: Optional[str] = None,
                local_dir: Optional[str] = None) -> str:
    from huggingface_hub import snapshot_download
    target = os.path.join(local_dir or "checkpoints", repo_id)
    os.makedirs(target, exist_ok=True)
    try:
        snapshot_download(repo_id, local_dir=target, token=hf_token)
    except Exception as e:  # noqa: BLE001
        status = getattr(getattr(e, "response", None), "status_code", None)
        if status == 401:
            print("You need to pass a valid `--hf_token=...` to download private checkpoints.")
        else:
            raise
    return target


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description="Download a checkpoint from HuggingFace Hub.")
    ap.add_argument("--repo_id", type=str, default="meta-llama/llama-2-7b-chat-hf")
    ap.add_argument("--local_dir", type=str, default=None)
    ap.add_argument("--hf_token", type=str, default=None)
    a = ap.parse_args()
    hf_download(a.repo_id, a.hf_token, a.local_dir)
