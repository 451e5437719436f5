"""Fetch tokenizer / config / weight files of a Hugging Face repository into ``<local_dir>/<repo name>``.

    python scripts/download_hf_assets.py --repo_id Qwen/Qwen3-1.7B --assets tokenizer config [--all] [--hf_token ...]

Needs network access and the `huggingface_hub` package on the machine where it runs (training hosts are usually
offline: run it where the hub is reachable and copy the folder).  ``--assets`` picks file groups: ``tokenizer``
(tokenizer*.json, vocab / merges, special tokens, chat template), ``config`` (config.json, generation_config.json),
``safetensors`` (weights + index), ``index`` (only model.safetensors.index.json, enough for shard naming on export).

(reference: scripts/download_hf_assets.py)
"""

from __future__ import annotations

import argparse
import fnmatch
import os

GROUPS = {
    "tokenizer": ["tokenizer.json", "tokenizer_config.json", "tokenizer.model", "vocab.json", "vocab.txt", "merges.txt",
                  "special_tokens_map.json", "added_tokens.json", "chat_template.jinja"],
    "config": ["config.json", "generation_config.json"],
    "safetensors": ["*.safetensors", "model.safetensors.index.json"],
    "index": ["model.safetensors.index.json"],
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--repo_id", required=True)
    ap.add_argument("--local_dir", default="assets/hf")
    ap.add_argument("--assets", nargs="+", default=["tokenizer", "config", "index"], choices=sorted(GROUPS))
    ap.add_argument("--all", action="store_true", help="download every file of the repository")
    ap.add_argument("--hf_token", default=os.environ.get("HF_TOKEN"))
    a = ap.parse_args()
    try:
        from huggingface_hub import hf_hub_download, list_repo_files
    except ImportError as e:
        raise SystemExit("huggingface_hub is not installed on this machine") from e
    target = os.path.join(a.local_dir, a.repo_id.split("/")[-1])
    os.makedirs(target, exist_ok=True)
    files = list_repo_files(a.repo_id, token=a.hf_token)
    if not a.all:
        pats = [p for g in a.assets for p in GROUPS[g]]
        files = [f for f in files if any(fnmatch.fnmatch(os.path.basename(f), p) for p in pats)]
    for f in files:
        print("fetching", f)
        hf_hub_download(a.repo_id, f, local_dir=target, token=a.hf_token)
    print(f"{len(files)} file(s) in {target}")


if __name__ == "__main__":
    main()
