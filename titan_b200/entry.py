"""Command-line entry: ``python -m titan_b200.entry --module M --config C [--section.field value ...]``.

Flow: parse the recipe + overrides → apply global numeric flags → build the trainer →
(seed-checkpoint mode: save step-0 from one process and exit) → train → close and destroy the
process group.  Any exception closes the trainer first (flushes async checkpoints, writers)
and is re-raised so the launcher sees a non-zero exit.

In ``--comm.mode fake_backend`` one process pretends to be ``NGPU`` ranks and runs a single step:
the dry run that feeds the memory simulator.

Parity: torchtitan_npu/entry.py:27-132, scripts/run_train.sh:13-40.
"""

from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

from titan_b200.config.manager import ConfigManager
from titan_b200.utils.logging import init_logger, logger

__all__ = ["main"]


def main(argv: list[str] | None = None):
    init_logger()
    config = ConfigManager().parse_args(argv)
    if config.comm.mode == "fake_backend":
        config.training.steps = min(config.training.steps, 1)
        config.checkpoint.enable = False
    if config.memory_sim.enable:
        from titan_b200.simulator.memory import run_from_config

        report = run_from_config(config)
        logger.info("%s", report.summary())
        return report

    trainer = None
    try:
        trainer = config.build()
        trainer.train()
    except Exception:
        if trainer is not None:
            trainer.close()
        raise
    else:
        trainer.close()
        if dist.is_initialized():
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            dist.destroy_process_group()
        logger.info("process group destroyed")
    return trainer


if __name__ == "__main__":
    main(sys.argv[1:])
