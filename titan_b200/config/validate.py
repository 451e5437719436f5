"""Check a training command line without launching anything:

    python -m titan_b200.config.validate --module deepseek_v4 --config debug_deepseek_v4_single_node_1b \\
        --training.seq_len 1152 dataloader:chat_data_loader_config --dataloader.dataset_path parquet

resolves the recipe, applies the overrides exactly as the trainer would and prints the resulting configuration as JSON
(exit status 0), or the parser's complaint (non-zero).  The launch scripts accept it in place of the trainer
(``TRAIN_FILE=titan_b200.config.validate``), which is how the example scripts are tested.
"""

from __future__ import annotations

import dataclasses
import json
import sys

from titan_b200.config.manager import ConfigManager


def _plain(obj):
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        return {"_type": type(obj).__name__, **{f.name: _plain(getattr(obj, f.name)) for f in dataclasses.fields(obj)}}
    if isinstance(obj, (list, tuple)):
        return [_plain(v) for v in obj]
    if isinstance(obj, dict):
        return {str(k): _plain(v) for k, v in obj.items()}
    if isinstance(obj, (str, int, float, bool)) or obj is None:
        return obj
    return repr(obj)


def main(argv: list[str] | None = None) -> int:
    cfg = ConfigManager().parse_args(argv)
    json.dump(_plain(cfg), sys.stdout, indent=1)
    sys.stdout.write("\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
