"""Fetch tokenizer / weights / index / config files of a Hugging Face repository into ``<local_dir>/<model name>/``.

``python -m torchtitan_b200.scripts.download_hf_assets --repo_id meta-llama/Llama-3.1-8B --assets tokenizer config
[--all] [--hf_token ...] [--additional_patterns "*.txt"]``. Asset types and file patterns follow
scripts/download_hf_assets.py:13-258. Needs network access and ``huggingface_hub``."""

from __future__ import annotations

import argparse
import fnmatch
import os

ASSET_PATTERNS = {
    "tokenizer": ["tokenizer.json", "tokenizer_config.json", "tokenizer.model", "vocab.txt", "vocab.json", "merges.txt",
                  "special_tokens_map.json"],
    "safetensors": ["*.safetensors", "*model.safetensors.index.json"],
    "index": ["*model.safetensors.index.json"],
    "config": ["config.json", "generation_config.json"],
}


def select_files(all_files: list[str], asset_types: list[str], download_all: bool = False,
                 additional_patterns: list[str] | None = None) -> list[str]:
    if download_all:
        return list(all_files)
    patterns: list[str] = []
    for t in asset_types:
        if t not in ASSET_PATTERNS:
            raise ValueError(f"Unknown asset type {t}. Available types: {list(ASSET_PATTERNS)}")
        patterns += ASSET_PATTERNS[t]
    patterns += list(additional_patterns or [])
    return [f for f in all_files if any(fnmatch.fnmatch(os.path.basename(f), p) or fnmatch.fnmatch(f, p) for p in patterns)]


def download_hf_assets(repo_id: str, local_dir: str, asset_types, download_all: bool = False, hf_token: str | None = None,
                       additional_patterns: list | None = None) -> list[str]:
    from huggingface_hub import hf_hub_download, list_repo_files

    if "/" not in repo_id:
        raise ValueError(f"Invalid repo_id format: '{repo_id}'. Expected format: 'organization/model-name'")
    asset_types = [asset_types] if isinstance(asset_types, str) else list(asset_types)
    model_dir = os.path.join(local_dir, repo_id.split("/")[-1].strip())
    files = select_files(list_repo_files(repo_id=repo_id, token=hf_token), asset_types, download_all, additional_patterns)
    if not files:
        print(f"No matching files found in {repo_id}")
        return []
    done = []
    for f in files:
        try:
            hf_hub_download(repo_id=repo_id, filename=f, local_dir=model_dir, token=hf_token)
            print(f"Successfully downloaded {f} to {model_dir}")
            done.append(f)
        except Exception as e:  # one missing optional file must not stop the rest
            print(f"Failed to download {f}: {e}")
    return done


if __name__ == "__main__":
    p = argparse.ArgumentParser(description="Download files from HuggingFace Hub.")
    p.add_argument("--repo_id", type=str, required=True)
    p.add_argument("--local_dir", type=str, default="assets/hf/")
    p.add_argument("--hf_token", type=str, default=os.environ.get("HF_TOKEN"))
    p.add_argument("--additional_patterns", type=str, nargs="*", default=[])
    p.add_argument("--assets", type=str, nargs="+", default=[], choices=list(ASSET_PATTERNS))
    p.add_argument("--all", action="store_true", default=False)
    a = p.parse_args()
    if not a.all and not a.assets:
        p.error("At least one asset type must be specified unless --all is used")
    download_hf_assets(a.repo_id, a.local_dir, a.assets, a.all, a.hf_token, a.additional_patterns)
