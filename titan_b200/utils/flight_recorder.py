"""NCCL flight-recorder wiring.

Must run before the process group is created: sets the trace ring size, enables
async error handling / the watchdog monitor, and points dump-on-timeout at
``{dump_folder}/{comm.save_traces_folder}/{prefix}<rank>``.  ``trace_buf_size = 0``
leaves everything off.

Parity: torchtitan_npu/tools/flight_recorder.py:15-43 (the same wiring for the
HCCL variables), docs/feature_guides/metrics_and_debugging.md:13-71.
"""

from __future__ import annotations

import os

__all__ = ["setup_flight_recorder", "FLIGHT_RECORDER_ENV"]

FLIGHT_RECORDER_ENV = (
    "TORCH_NCCL_TRACE_BUFFER_SIZE",
    "TORCH_FR_BUFFER_SIZE",
    "TORCH_NCCL_ASYNC_ERROR_HANDLING",
    "TORCH_NCCL_ENABLE_MONITORING",
    "TORCH_NCCL_DUMP_ON_TIMEOUT",
    "TORCH_NCCL_DEBUG_INFO_TEMP_FILE",
    "TORCH_FR_DUMP_TEMP_FILE",
)


def setup_flight_recorder(comm_config, base_folder: str = "", env: dict | None = None) -> dict[str, str]:
    """Populate the environment (or `env`, for tests) and return what was set."""
    env = os.environ if env is None else env
    size = int(getattr(comm_config, "trace_buf_size", 0) or 0)
    if size <= 0:
        return {}
    dump_dir = os.path.join(base_folder, comm_config.save_traces_folder)
    prefix = os.path.join(dump_dir, comm_config.save_traces_file_prefix)
    values = {
        "TORCH_NCCL_TRACE_BUFFER_SIZE": str(size),
        "TORCH_FR_BUFFER_SIZE": str(size),
        # 3 = tear down the communicator and raise on the host instead of hanging
        "TORCH_NCCL_ASYNC_ERROR_HANDLING": "3",
        "TORCH_NCCL_ENABLE_MONITORING": "1",
        "TORCH_NCCL_DUMP_ON_TIMEOUT": "1",
        "TORCH_NCCL_DEBUG_INFO_TEMP_FILE": prefix,
        "TORCH_FR_DUMP_TEMP_FILE": prefix,
    }
    set_now = {}
    for k, v in values.items():
        if k not in env:  # a user's explicit setting wins
            env[k] = v
            set_now[k] = v
    try:
        os.makedirs(dump_dir, exist_ok=True)
    except OSError:
        pass
    return set_now
