"""Memory and step-time estimate of a training command line, without a GPU:

    python -m titan_b200.simulator --world 4 --module deepseek_v32 --config deepseek_v32_sparse_cp8 \\
        --training.seq_len 131072 --parallelism.context_parallel_degree 4

``--world N`` is the job size (default: the `NGPU` / `WORLD_SIZE` environment, else 1); everything else is the
trainer's own command line (recipe + dotted overrides).  ``--json`` prints the report as JSON instead of the table.
The exit status is 0 when the estimate fits the HBM budget (`--memory_sim.hbm_budget_gib`), 3 when it does not.
"""

from __future__ import annotations

import os
import sys

from titan_b200.config.manager import ConfigManager
from titan_b200.simulator.memory import estimate


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    world = int(os.environ.get("NGPU", os.environ.get("WORLD_SIZE", "1")))
    as_json = False
    rest = []
    i = 0
    while i < len(argv):
        if argv[i] == "--world":
            world = int(argv[i + 1])
            i += 2
        elif argv[i].startswith("--world="):
            world = int(argv[i].split("=", 1)[1])
            i += 1
        elif argv[i] == "--json":
            as_json = True
            i += 1
        else:
            rest.append(argv[i])
            i += 1
    cfg = ConfigManager().parse_args(rest)
    report = estimate(cfg, world)
    print(report.to_json() if as_json else report.summary())
    return 0 if report.fits else 3


if __name__ == "__main__":
    sys.exit(main())
