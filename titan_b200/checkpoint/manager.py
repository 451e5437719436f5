"""Checkpoint manager: DCP save / load / resume, HF safetensors import/export.

Layout: ``{dump_folder}/{checkpoint.folder}/step-N/{.metadata, *.distcp}`` (full
train state: model, optimizer, lr_scheduler, dataloader, train_state) or HF
safetensors (model only).  Resume precedence: an existing ``step-*`` in the
output folder beats ``initial_load_path``, which beats the model's HF assets.
DCP reshards on load, so a checkpoint written under one parallel layout loads
under another.

Writer knobs: ``sync_files`` (fsync before returning), ``drop_page_cache_after_save``
(``posix_fadvise(DONTNEED)`` on written files to relieve host memory),
``empty_cache_after_save`` (release staging buffers of the caching allocator).
Async modes: ``async`` (background thread, no pinned stager), and
``async_with_pinned_mem`` (separate process fed from a pinned staging buffer).

Parity: torchtitan_npu/patches/torch/checkpoint.py:30-220,
docs/feature_guides/checkpoint.md:8-73,195-225, entry.py:115-121 (seed checkpoint).
"""

from __future__ import annotations

import enum
import gc
import glob
import os
import re
import shutil
import time
from typing import Any

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
import torch.nn as nn
from torch.distributed.checkpoint import FileSystemWriter
from torch.distributed.checkpoint.state_dict import (
    StateDictOptions,
    get_model_state_dict,
    set_model_state_dict,
)
from torch.distributed.checkpoint.stateful import Stateful

from titan_b200.utils.logging import logger

__all__ = ["CheckpointManager", "AsyncMode", "ModelWrapper", "drop_page_cache_for_path", "MODEL", "OPTIMIZER"]

MODEL, OPTIMIZER, LR_SCHEDULER, DATALOADER, TRAIN_STATE = "model", "optimizer", "lr_scheduler", "dataloader", "train_state"


class AsyncMode(str, enum.Enum):
    DISABLED = "disabled"
    ASYNC = "async"
    ASYNC_WITH_PINNED_MEM = "async_with_pinned_mem"


class ModelWrapper(Stateful):
    """Flat state dict over all model parts (pipeline stages hold disjoint FQNs)."""

    def __init__(self, model: nn.Module | list[nn.Module]):
        self.model = [model] if isinstance(model, nn.Module) else model

    def state_dict(self) -> dict[str, Any]:
        sd: dict[str, Any] = {}
        for part in self.model:
            sd.update(get_model_state_dict(part))
        return sd

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        for part in self.model:
            set_model_state_dict(part, model_state_dict=state_dict, options=StateDictOptions(strict=False))


def drop_page_cache_for_path(path: str) -> None:
    """Ask Linux to evict the page-cache pages of every file under `path`."""
    if not hasattr(os, "posix_fadvise"):
        return
    candidates = [path] if os.path.isfile(path) else [
        os.path.join(r, f) for r, _, fs in os.walk(path) for f in fs
    ]
    for cand in candidates:
        fd = None
        try:
            fd = os.open(cand, os.O_RDONLY)
            os.posix_fadvise(fd, 0, 0, os.POSIX_FADV_DONTNEED)
        except OSError as exc:
            logger.debug("page-cache drop failed for %s: %s", cand, exc)
        finally:
            if fd is not None:
                os.close(fd)


class _Writer(FileSystemWriter):
    """`FileSystemWriter` that can evict what it wrote from the host page cache."""

    def __init__(self, path, *, sync_files: bool = True, drop_page_cache: bool = False, **kw):
        super().__init__(path, sync_files=sync_files, **kw)
        self._drop_page_cache = drop_page_cache

    def write_data(self, plan, planner):
        fut = super().write_data(plan, planner)
        if self._drop_page_cache:
            fut.wait()
            drop_page_cache_for_path(str(self.path))
        return fut


class CheckpointManager:
    def __init__(self, *, dataloader, model_parts: list[nn.Module], optimizers, lr_schedulers,
                 states: dict[str, Any], config, sd_adapter=None, base_folder: str = "", ft_manager=None):
        self.config = config
        self.enable = config.enable
        self.sd_adapter = sd_adapter
        self.states = dict(states)
        self.states.update({
            MODEL: ModelWrapper(model_parts),
            OPTIMIZER: optimizers,
            DATALOADER: dataloader,
            LR_SCHEDULER: lr_schedulers,
        })
        self.folder = os.path.join(base_folder, config.folder)
        self.interval = config.interval
        self.keep_latest_k = config.keep_latest_k
        if 0 < self.keep_latest_k < 2:
            raise ValueError("keep_latest_k must be 0 (keep all) or >= 2")
        self.async_mode = AsyncMode(config.async_mode.lower())
        if self.async_mode == AsyncMode.ASYNC_WITH_PINNED_MEM and not torch.cuda.is_available():
            # pinned staging needs a device; a host-only run still overlaps the write with training
            logger.warning("checkpoint.async_mode async_with_pinned_mem needs a GPU; using 'async'")
            self.async_mode = AsyncMode.ASYNC
        self.export_dtype = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}[
            config.export_dtype
        ]
        self.exclude_from_loading = list(config.exclude_from_loading)
        self.pg = None
        self.stager = None
        self._async_future = None
        if self.enable and self.async_mode != AsyncMode.DISABLED and dist.is_initialized():
            # a CPU group so background saves never contend with training collectives
            self.pg = dist.new_group(backend="gloo")
        self.begin_time = time.monotonic()

    # ------------------------------------------------------------------ paths
    def _step_dir(self, step: int) -> str:
        return os.path.join(self.folder, f"step-{step}")

    def _find_load_step(self, folder: str | None = None) -> int:
        folder = folder or self.folder
        steps = []
        for path in glob.glob(os.path.join(folder, "step-*")):
            m = re.search(r"step-(\d+)$", path)
            if m and (os.path.exists(os.path.join(path, ".metadata"))
                      or glob.glob(os.path.join(path, "*.safetensors"))):
                steps.append(int(m.group(1)))
        return max(steps) if steps else -1

    # ------------------------------------------------------------------ save
    def _should_save(self, curr_step: int, last_step: bool = False) -> bool:
        if not self.enable or self.config.load_only:
            return False
        if curr_step == 1 and self.config.enable_first_step_checkpoint:
            return True
        return last_step or curr_step % self.interval == 0

    def _flattened_state(self) -> dict[str, Any]:
        return {k: v for k, v in self.states.items()}

    def _export_model_state(self) -> dict[str, Any]:
        sd = self.states[MODEL].state_dict()
        if self.export_dtype != torch.float32:
            sd = {k: (v.to(self.export_dtype) if torch.is_floating_point(v) else v) for k, v in sd.items()}
        return sd

    @torch.no_grad()
    def dcp_save(self, state_dict: dict[str, Any], checkpoint_id: str, async_mode: AsyncMode, *,
                 to_hf: bool = False):
        cfg = self.config
        consolidate_from = None
        if to_hf:
            if self.sd_adapter is None:
                raise ValueError("HF export requested but the model has no state-dict adapter")
            from torch.distributed.checkpoint import HuggingFaceStorageWriter

            state_dict = self.sd_adapter.to_hf(state_dict)
            mapping = self.sd_adapter.fqn_to_index_mapping
            if mapping:
                mapping = {k: v for k, v in mapping.items() if k in state_dict}
                consolidate_from = os.path.join(checkpoint_id, "sharded")
                writer = HuggingFaceStorageWriter(path=consolidate_from, save_distributed=True,
                                                  fqn_to_index_mapping=mapping, enable_consolidation=False)
            else:
                writer = HuggingFaceStorageWriter(path=checkpoint_id, save_distributed=True,
                                                  enable_consolidation=True)
            writer.sync_files = cfg.sync_files
            save_id = None
        else:
            writer = _Writer(checkpoint_id, sync_files=cfg.sync_files, drop_page_cache=cfg.drop_page_cache_after_save)
            save_id = checkpoint_id

        if async_mode == AsyncMode.ASYNC:
            if hasattr(writer, "per_thread_copy_ahead"):
                writer.per_thread_copy_ahead = 0
            ret = dcp.async_save(state_dict, storage_writer=writer, checkpoint_id=save_id, process_group=self.pg)
        elif async_mode == AsyncMode.ASYNC_WITH_PINNED_MEM:
            from torch.distributed.checkpoint.state_dict_saver import AsyncCheckpointerType
            from torch.distributed.checkpoint.staging import DefaultStager, StagingOptions

            if self.stager is None:
                self.stager = DefaultStager(StagingOptions(True, True, True, True))
            if hasattr(writer, "per_thread_copy_ahead"):
                writer.per_thread_copy_ahead = 0
            ret = dcp.async_save(state_dict, storage_writer=writer, checkpoint_id=save_id, process_group=self.pg,
                                 async_checkpointer_type=AsyncCheckpointerType.PROCESS, async_stager=self.stager)
        else:
            ret = dcp.save(state_dict, storage_writer=writer, checkpoint_id=save_id)

        if consolidate_from is not None:
            from torch.distributed.checkpoint._consolidate_hf_safetensors import (
                consolidate_safetensors_files_on_every_rank,
            )

            consolidate_safetensors_files_on_every_rank(
                input_dir=consolidate_from, output_dir=checkpoint_id,
                fqn_to_index_mapping=mapping, num_threads=5)
        return ret

    def maybe_wait_for_staging(self) -> None:
        fut = self._async_future
        if fut is not None and hasattr(fut, "staging_completion"):
            fut.staging_completion.result()

    def _wait_async(self) -> None:
        fut = self._async_future
        if fut is None:
            return
        done = getattr(fut, "upload_completion", fut)
        done.result()
        self._async_future = None

    def save(self, curr_step: int, last_step: bool = False):
        if not self._should_save(curr_step, last_step):
            return None
        begin = time.monotonic()
        self._wait_async()
        cid = self._step_dir(curr_step)
        if last_step and self.config.last_save_model_only:
            sd = self._export_model_state()
            ret = self.dcp_save(sd, cid, AsyncMode.DISABLED, to_hf=self.config.last_save_in_hf)
        else:
            if hasattr(self.states[OPTIMIZER], "init_cache_state_dict"):
                self.states[OPTIMIZER].init_cache_state_dict()
            ret = self.dcp_save(self._flattened_state(), cid, self.async_mode)
            if self.async_mode != AsyncMode.DISABLED:
                self._async_future = ret
        self._purge_stale()
        if self.config.empty_cache_after_save:
            gc.collect()
            if torch.cuda.is_available():
                torch.cuda.empty_cache()
        logger.info("saved checkpoint step-%d in %.2f s", curr_step, time.monotonic() - begin)
        return ret

    def _purge_stale(self) -> None:
        if self.keep_latest_k <= 0 or (dist.is_initialized() and dist.get_rank() != 0):
            return
        found = []
        for path in glob.glob(os.path.join(self.folder, "step-*")):
            m = re.search(r"step-(\d+)$", path)
            if m:
                found.append((int(m.group(1)), path))
        found.sort()
        for _, path in found[: -self.keep_latest_k]:
            shutil.rmtree(path, ignore_errors=True)

    # ------------------------------------------------------------------ load
    def _states_to_load(self, model_only: bool) -> dict[str, Any]:
        if model_only:
            return self.states[MODEL].state_dict()
        return {k: v for k, v in self.states.items() if k not in self.exclude_from_loading}

    def dcp_load(self, state_dict: dict[str, Any], checkpoint_id: str, *, from_hf: bool = False,
                 from_quantized: bool = False) -> None:
        if from_hf:
            if self.sd_adapter is None:
                raise ValueError("HF load requested but the model has no state-dict adapter")
            hf_sd = self.sd_adapter.to_hf(state_dict)
            reader = self.sd_adapter.get_hf_storage_reader(checkpoint_id, from_quantized)
            dcp.load(hf_sd, storage_reader=reader)
            native = self.sd_adapter.from_hf(hf_sd)
            self.states[MODEL].load_state_dict(native)
        else:
            dcp.load(state_dict, checkpoint_id=checkpoint_id)
            if MODEL not in state_dict:  # model-only flat dict
                self.states[MODEL].load_state_dict(state_dict)

    def load(self, step: int = -1) -> bool:
        """Load per the precedence rules; returns whether anything was loaded."""
        cfg = self.config
        if not self.enable:
            return False
        model_only = False
        from_hf = False
        if os.path.isdir(self.folder) and self._find_load_step() >= 0:
            # an existing run in the output folder always wins
            step = self._find_load_step() if step == -1 else step
            cid = self._step_dir(step)
            if not os.path.isdir(cid):
                raise FileNotFoundError(f"--checkpoint.load_step={step} but {cid} does not exist")
        elif cfg.initial_load_path:
            cid = cfg.initial_load_path
            if not os.path.isdir(cid):
                raise FileNotFoundError(f"checkpoint.initial_load_path {cid} is not a directory")
            model_only = cfg.initial_load_model_only
            from_hf = cfg.initial_load_in_hf
        elif cfg.initial_load_in_hf:
            cid = getattr(self.sd_adapter, "hf_assets_path", None)
            if not cid or not os.path.isdir(cid):
                raise FileNotFoundError("initial_load_in_hf is set but no HF assets path is available")
            model_only, from_hf = True, True
        else:
            return False
        begin = time.monotonic()
        if from_hf:
            self.dcp_load(self.states[MODEL].state_dict(), cid, from_hf=True,
                          from_quantized=cfg.initial_load_in_hf_quantized)
        else:
            self.dcp_load(self._states_to_load(model_only), cid)
        gc.collect()
        logger.info("loaded checkpoint %s in %.2f s", cid, time.monotonic() - begin)
        return True

    def close(self) -> None:
        self._wait_async()
        if self.stager is not None and hasattr(self.stager, "close"):
            self.stager.close()
