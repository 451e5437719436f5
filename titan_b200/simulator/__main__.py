"""Memory and step-time estimate of a training command line, without a GPU:

    python -m titan_b200.simulator --world 4 --module deepseek_v32 --config deepseek_v32_sparse_cp8 \\
        --training.seq_len 131072 --parallelism.context_parallel_degree 4

``--world N`` is the job size (default: the `NGPU` / `WORLD_SIZE` environment, else 1); everything else is the
trainer's own command line (recipe + dotted overrides).  ``--json`` prints the report as JSON instead of the table.
``--worlds 1,2,4,8`` prints one line per job size instead (peak memory, step time, tokens/s and the tokens/s per GPU
relative to the smallest size): sizes the recipe's degrees do not divide are skipped with the reason.
``--checkpointing`` prints one line per activation-checkpoint mode (none, selective, full) at the given job size and
marks the fastest one that fits.
The exit status is 0 when the estimate fits the HBM budget (`--memory_sim.hbm_budget_gib`), 3 when it does not.
"""

from __future__ import annotations

import os
import sys

from titan_b200.config.manager import ConfigManager
from titan_b200.simulator.memory import estimate


def _table(rest: list[str], worlds: list[int]) -> int:
    print(f"{'GPUs':>5} {'peak GiB':>9} {'fits':>5} {'ms/step':>9} {'tokens/s':>12} {'per GPU':>10} {'vs first':>9}")
    first = None
    all_fit = True
    for w in worlds:
        cfg = ConfigManager().parse_args(rest)   # a fresh configuration per size: `estimate` edits nothing, recipes may
        try:
            rep = estimate(cfg, w)
        except ValueError as e:
            print(f"{w:>5} skipped: {e}")
            continue
        per_gpu = rep.tokens_per_second_estimate / w
        first = first or per_gpu
        all_fit &= rep.fits
        print(f"{w:>5} {rep.bytes_total / 2 ** 30:>9.1f} {'yes' if rep.fits else 'NO':>5} "
              f"{rep.step_seconds_estimate * 1e3:>9.1f} {rep.tokens_per_second_estimate:>12,.0f} {per_gpu:>10,.0f} "
              f"{per_gpu / first if first else 0:>9.2f}")
    return 0 if all_fit else 3


def _checkpointing_table(rest: list[str], world: int) -> int:
    rows = []
    for mode in ("none", "selective", "full"):
        cfg = ConfigManager().parse_args(rest)
        cfg.activation_checkpoint.mode = mode
        rep = estimate(cfg, world)
        rows.append((mode, rep))
    fitting = [(rep.step_seconds_estimate, mode) for mode, rep in rows if rep.fits and rep.step_seconds_estimate > 0]
    best = min(fitting)[1] if fitting else None
    print(f"{'checkpointing':>14} {'peak GiB':>9} {'fits':>5} {'ms/step':>9} {'tokens/s':>12}")
    for mode, rep in rows:
        print(f"{mode:>14} {rep.bytes_total / 2 ** 30:>9.1f} {'yes' if rep.fits else 'NO':>5} "
              f"{rep.step_seconds_estimate * 1e3:>9.1f} {rep.tokens_per_second_estimate:>12,.0f}"
              f"{'   <- fastest that fits' if mode == best else ''}")
    return 0 if best else 3


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    world = int(os.environ.get("NGPU", os.environ.get("WORLD_SIZE", "1")))
    as_json = False
    worlds: list[int] = []
    ac_table = False
    rest = []
    i = 0
    while i < len(argv):
        if argv[i] == "--world":
            world = int(argv[i + 1])
            i += 2
        elif argv[i].startswith("--world="):
            world = int(argv[i].split("=", 1)[1])
            i += 1
        elif argv[i] == "--worlds":
            worlds = [int(v) for v in argv[i + 1].split(",") if v]
            i += 2
        elif argv[i] == "--checkpointing":
            ac_table = True
            i += 1
        elif argv[i] == "--json":
            as_json = True
            i += 1
        else:
            rest.append(argv[i])
            i += 1
    if worlds:
        return _table(rest, worlds)
    if ac_table:
        return _checkpointing_table(rest, world)
    cfg = ConfigManager().parse_args(rest)
    report = estimate(cfg, world)
    print(report.to_json() if as_json else report.summary())
    return 0 if report.fits else 3


if __name__ == "__main__":
    sys.exit(main())
