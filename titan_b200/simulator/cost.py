"""Step-time estimate for the meta-device run of the memory simulator.

While `MetaMemoryTracker` follows storages, `StepCost` prices every operator of the same forward + backward:

* contractions (library matmuls, the tcgen05 GEMM operators, grouped GEMMs, block-scaled FP8 GEMMs, dense attention)
  by their FLOPs at a fraction of the measured tensor-core rate, never below the time their bytes need;
* everything else by the bytes of its tensor arguments and results at a fraction of the measured copy rate (views and
  allocations are free), never below a per-launch floor;
* the hand-written kernels whose speed is set by latency rather than by a roofline (sparse attention on gathered
  tiles, the indexer's scoring and its selected-key backward) by rates measured on B200s
  (the summaries under `profiles/` give the numbers).

Kernels that are launched through `ctypes` never reach the dispatcher; inside `ops._lib.no_launch()` the stand-in
library hands their names and integer arguments to `StepCost.on_library_call`.  The optimizer step and the exposed
part of the collectives are added from closed forms.  The result is an ESTIMATE with calibrated constants: the
tests pin it to measured steps (Llama-3 8B dense / MXFP8, DeepSeek-V3.2 sparse attention, DeepSeek-V4,
DeepSeek-V3 16B with expert parallelism) within a stated band.

The reference publishes throughput tables but has no step-time model; its estimation notes cover memory only
(.agents/skills/oom-analysis/references/memory-estimation-templates.md:7-107).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field

import torch
from torch.utils._pytree import tree_flatten

__all__ = ["Peaks", "StepCost"]


@dataclass
class Peaks:
    """Device rates the estimate divides by.  Defaults are measured on B200s of one pool (a copy and a library bf16
    GEMM running for seconds under the power cap); `Peaks.load()` prefers a `MEASURED_PEAKS.json` beside the
    package's repository root when one exists."""

    bf16_tflops: float = 1387.5          # sustained library GEMM
    hbm_gbs: float = 6530.0              # copy rate, read + write
    fp8_factor: float = 1.55             # block-scaled FP8 GEMM over bf16 (2.2-2.5 PFLOP/s burst vs 1.65 burst)
    gemm_efficiency: float = 0.95        # large products inside a training step vs the back-to-back GEMM loop
                                         # (280 ms for the 369 TFLOP of a Llama-3 8B step: the clocks sit higher)
    small_gemm_efficiency: float = 0.45  # below `small_gemm_flops`
    small_gemm_flops: float = 2.0e10
    memory_efficiency: float = 0.62      # element-wise / normalisation kernels vs the copy rate
    optimizer_efficiency: float = 0.78   # fused AdamW: 22 bytes per parameter in 34.4 ms for 8.03 G parameters
    launch_floor_s: float = 4.5e-6       # an operator cannot cost less than its launch
    attention_fwd_tflops: float = 1300.0  # library fused attention (causal FLOPs), forward: 13.5 ms per 17.6 TFLOP
    attention_bwd_tflops: float = 1000.0  # backward (2.5x the forward FLOPs): 43.9 ms
    flash_fwd_tflops: float = 534.0      # the framework's tcgen05 attention: 1.03 ms at 8192 x 32 heads x 128
    flash_bwd_tflops: float = 312.0      # 4.40 ms
    # latency-bound kernels: seconds per (query x selected key x head), measured at 16 heads / top-2048
    sparse_fwd_s: float = 3.8e-3 / (4096 * 2048 * 16)
    sparse_bwd_s: float = 7.6e-3 / (4096 * 2048 * 16)
    sparse_bwd_large_stream: float = 1.17    # gradient buffer of the latent no longer fits in L2
    indexer_score_s: float = 5.11e-3 / (8192 * 32768 * 64)   # per (query x key x head), 128-dim keys, resident form
    indexer_sel_bwd_s: float = 1.35e-3 / (2048 * 2048 * 64)  # per (query x selected key x head)
    host_s_per_operator: float = 10e-6   # eager dispatch + autograd bookkeeping per operator: a step cannot be shorter
                                         # than the host needs to issue it (DeepSeek-V4 mini: 26 k operators, 259 ms)
    exposed_fsdp: float = 1.0            # the FSDP traffic time at link rate shows up in full, partly as waits and
                                         # partly as GEMMs that slow down beside the collectives: Llama-3 8B goes
                                         # from 438 ms on one GPU to 444 / 452 ms on 4 / 8 although the optimizer
                                         # step shrinks by 31 ms
    exposed_tp: float = 1.0
    pcie_gbs: float = 50.0               # pinned host <-> device, per direction (Swap optimizer streams its state)
    exposed_ep: float = 1.5              # dispatch / combine run inside the layer at about two thirds of the link rate,
                                         # plus the staging copies on either side

    @classmethod
    def load(cls) -> "Peaks":
        here = os.path.dirname(os.path.abspath(__file__))
        path = os.path.join(os.path.dirname(os.path.dirname(here)), "MEASURED_PEAKS.json")
        p = cls()
        try:
            with open(path) as f:
                d = json.load(f)
            p.bf16_tflops = float(d.get("bf16_tflops_sustained", p.bf16_tflops))
            p.hbm_gbs = float(d.get("hbm_gbs", p.hbm_gbs))
        except (OSError, ValueError):
            pass
        return p


def _nbytes(t) -> int:
    return t.numel() * t.element_size() if isinstance(t, torch.Tensor) else 0


def _tensors(tree) -> list[torch.Tensor]:
    """Tensors of a (nested) argument structure, in argument order."""
    return [x for x in tree_flatten(tree)[0] if isinstance(x, torch.Tensor)]


@dataclass
class StepCost:
    peaks: Peaks = field(default_factory=Peaks.load)
    seconds: float = 0.0
    flops: float = 0.0
    bytes: float = 0.0
    launches: int = 0
    by_kind: dict = field(default_factory=dict)
    unpriced: int = 0                 # operators whose pricing rule failed (counted, not fatal)
    free_ops: int = 0                 # views and allocations: no device time, but the host still dispatches them
    grouped_rows_scale: float = 1.0   # rows in use / rows the expert-major buffers are sized for

    # ------------------------------------------------------------------ bookkeeping
    def _add(self, kind: str, seconds: float, flops: float = 0.0, nbytes: float = 0.0) -> None:
        seconds = max(seconds, self.peaks.launch_floor_s)
        self.seconds += seconds
        self.flops += flops
        self.bytes += nbytes
        self.launches += 1
        self.by_kind[kind] = self.by_kind.get(kind, 0.0) + seconds

    def _contraction(self, kind: str, flops: float, nbytes: float, rate_factor: float = 1.0) -> None:
        p = self.peaks
        eff = p.gemm_efficiency if flops >= p.small_gemm_flops else p.small_gemm_efficiency
        t = flops / (p.bf16_tflops * 1e12 * eff * rate_factor)
        self._add(kind, max(t, nbytes / (p.hbm_gbs * 1e9)), flops, nbytes)

    def _memory(self, kind: str, nbytes: float) -> None:
        self._add(kind, nbytes / (self.peaks.hbm_gbs * 1e9 * self.peaks.memory_efficiency), 0.0, nbytes)

    # ------------------------------------------------------------------ dispatcher operators
    def on_op(self, func, args, kwargs, out) -> None:
        name = str(func)                      # e.g. "aten.mm.default", "titan_b200.gemm.default"
        ns, _, rest = name.partition(".")
        base = rest.split(".")[0]
        ins, outs = _tensors((args, kwargs)), _tensors(out)
        if not outs:
            return
        if ns == "aten" and base.startswith(("empty", "new_empty")):
            self.free_ops += 1
            return                            # an allocation moves no bytes
        if not base.endswith("_"):            # in-place operators alias their argument and still do the work
            try:
                in_keys = {id(t.untyped_storage()) for t in ins}
                if ins and all(id(t.untyped_storage()) in in_keys for t in outs):
                    self.free_ops += 1
                    return                    # every result aliases an argument: a view
            except Exception:
                pass
        nbytes = sum(_nbytes(t) for t in ins) + sum(_nbytes(t) for t in outs)
        a = ins[0] if ins else None
        if ns == "aten":
            if base in ("mm", "addmm", "bmm", "baddbmm", "matmul", "linear"):
                x, y = (ins[-2], ins[-1]) if len(ins) >= 2 else (a, a)
                k = x.shape[-1]
                self._contraction("matmul", 2.0 * outs[0].numel() * k, nbytes)
                return
            if base == "_grouped_mm":
                x, w = ins[0], ins[1]
                if w.dim() == 3:              # rows x [groups, K, N]
                    fl = 2.0 * x.shape[0] * w.shape[-2] * w.shape[-1]
                else:                          # per-group weight gradient: contraction over the rows
                    fl = 2.0 * x.shape[0] * x.shape[1] * w.shape[-1]
                self._contraction("grouped_mm", fl, nbytes)
                return
            if base in ("zeros", "zeros_like", "zero_", "fill_", "full", "full_like", "ones", "ones_like"):
                self._memory("fill", sum(_nbytes(t) for t in outs))
                return
            self._memory("elementwise", nbytes)
            return
        if ns == "titan_b200":
            if base == "gemm":
                a_mn = bool(args[2]) if len(args) > 2 else bool(kwargs.get("a_mn", False))
                k = ins[0].shape[0] if a_mn else ins[0].shape[1]
                self._contraction("gemm_tcgen05", 2.0 * outs[0].numel() * k, nbytes)
                return
            if base == "grouped_gemm_m":
                g = self.grouped_rows_scale
                self._contraction("grouped_gemm", 2.0 * outs[0].numel() * ins[0].shape[1] * g, nbytes * g)
                return
            if base == "grouped_gemm_k":
                g = self.grouped_rows_scale
                self._contraction("grouped_gemm", 2.0 * ins[0].shape[0] * ins[0].shape[1] * ins[1].shape[1] * g,
                                  nbytes * g)
                return
            if base == "mx_linear_fwd":
                x, w = ins[0], ins[1]
                self._contraction("mxfp8_gemm", 2.0 * x.shape[0] * x.shape[1] * w.shape[0], nbytes,
                                  self.peaks.fp8_factor)
                self._memory("mx_quantize", 2.0 * (_nbytes(x) + _nbytes(w)))
                return
            if base in ("flash_attention_fwd", "flash_attention_bwd"):
                q, k = ins[0], ins[1]          # [B, S, H, D]
                fl = 4.0 * q.shape[0] * q.shape[2] * q.shape[1] * k.shape[1] * q.shape[3] * 0.5
                if base.endswith("bwd"):
                    self._add("flash_attention", 2.5 * fl / (self.peaks.flash_bwd_tflops * 1e12), 2.5 * fl, nbytes)
                else:
                    self._add("flash_attention", fl / (self.peaks.flash_fwd_tflops * 1e12), fl, nbytes)
                return
            if base == "sparse_mla_fwd":
                q, idx = ins[0], ins[2]        # [S, H, Dq], [S, K]
                pairs = q.shape[0] * idx.shape[1] * q.shape[1]
                self._add("sparse_attention", pairs * self.peaks.sparse_fwd_s,
                          2.0 * pairs * (q.shape[2] + int(args[4])), nbytes)
                return
            if base == "indexer_topk":
                q, k = ins[0], ins[2]          # [B, S, H, D], [B, T, 1, D]
                pairs = q.shape[0] * q.shape[1] * k.shape[1] * q.shape[2]
                score_bytes = q.shape[0] * q.shape[1] * k.shape[1] * 4.0
                self._add("indexer scoring", pairs * self.peaks.indexer_score_s * 0.5     # causal: half the pairs
                          + 3.0 * score_bytes / (self.peaks.hbm_gbs * 1e9), 2.0 * pairs * q.shape[3], nbytes)
                return
            self._memory("fused_elementwise", nbytes)
            return
        self._memory("other", nbytes)

    def on_dense_attention(self, q, k, backward: bool) -> None:
        """Library fused attention (the stand-in of the meta run): q [B, H, S, D], k [B, Hkv, T, D], causal."""
        fl = 4.0 * q.shape[0] * q.shape[1] * q.shape[2] * k.shape[2] * q.shape[3] * 0.5
        nbytes = 2.0 * (_nbytes(q) + 2 * _nbytes(k))
        if backward:
            self._add("attention", 2.5 * fl / (self.peaks.attention_bwd_tflops * 1e12), 2.5 * fl, 2 * nbytes)
        else:
            self._add("attention", fl / (self.peaks.attention_fwd_tflops * 1e12), fl, nbytes)

    # ------------------------------------------------------------------ kernels launched through ctypes
    def on_library_call(self, name: str, args: tuple) -> None:
        try:
            self._price_library_call(name, args)
        except Exception:
            self.unpriced += 1

    def _price_library_call(self, name: str, args: tuple) -> None:
        ints = [a for a in args if isinstance(a, int) and not isinstance(a, bool)]
        p = self.peaks
        if name == "tb_gemm_auto" and len(args) >= 6:
            m, n, k = (int(v) for v in args[3:6])
            self._contraction("gemm_tcgen05", 2.0 * m * n * k, 2.0 * (m * k + n * k + m * n))
        elif name in ("tb_mxfp8_gemm", "tb_mxfp8_grouped_gemm") and len(args) >= 8:
            m, n, k = (int(v) for v in args[5:8])
            g = self.grouped_rows_scale if name == "tb_mxfp8_grouped_gemm" else 1.0   # rows in use, not capacity
            self._contraction("mxfp8_gemm", 2.0 * m * n * k * g, (1.0 * (m * k + n * k) + 2.0 * m * n) * g,
                              p.fp8_factor)
        elif name == "tb_sparse_mla_bwd" and len(args) >= 14:
            s, h, t, kk, dq = (int(v) for v in args[8:13])
            big = p.sparse_bwd_large_stream if t * dq * 4 > 100e6 else 1.0
            self._add("sparse_attention", s * kk * h * p.sparse_bwd_s * big, 4.0 * s * kk * h * dq * 2, 0.0)
        elif name == "tb_indexer_sel_bwd" and len(args) >= 13:
            s, h, _t, kk = (int(v) for v in args[8:12])
            self._add("indexer backward", s * kk * h * p.indexer_sel_bwd_s, 0.0, 0.0)
        elif name in ("tb_mx_quantize", "tb_mx_quantize_dual", "tb_mx_dequantize"):
            rows_cols = [v for v in ints if v > 8][:2]
            if len(rows_cols) == 2:
                self._memory("mx_quantize", 4.0 * rows_cols[0] * rows_cols[1])
        elif name.startswith("tb_") and not name.endswith(("_blocks", "_bytes", "_count", "bind_device")):
            self._add("library_kernel", p.launch_floor_s)   # small kernels: routing plans, pads, flags

    # ------------------------------------------------------------------ closed forms outside the traced step
    def add_optimizer_step(self, local_params: float, param_bytes: int, moment_bytes: int) -> None:
        p = self.peaks
        # read + write parameters and two moments, read the gradients; one more read of the gradients for their norm
        step = local_params * (2 * param_bytes + 4 * moment_bytes + param_bytes)
        self._add("optimizer", step / (p.hbm_gbs * 1e9 * p.optimizer_efficiency), 0.0, step)
        norm = local_params * param_bytes
        self._add("gradient norm", norm / (p.hbm_gbs * 1e9 * 0.4), 0.0, norm)

    def add_optimizer_swap(self, host_state_bytes: float) -> None:
        """Swap optimizer: every step the state travels to the device and back; the two directions overlap."""
        if host_state_bytes > 0:
            t = host_state_bytes / (self.peaks.pcie_gbs * 1e9)
            self.seconds += t
            self.by_kind["optimizer state swap"] = self.by_kind.get("optimizer state swap", 0.0) + t

    def exposed_collectives(self, comm_bytes: dict, link_gbs: float) -> float:
        share = {"fsdp_all_gather": self.peaks.exposed_fsdp, "fsdp_reduce_scatter": self.peaks.exposed_fsdp,
                 "tp_sp_collectives": self.peaks.exposed_tp, "ep_all_to_all": self.peaks.exposed_ep}
        t = sum(v / (link_gbs * 1e9) * share.get(k, 1.0) for k, v in comm_bytes.items())
        if t:
            self.seconds += t
            self.by_kind["collectives (exposed)"] = self.by_kind.get("collectives (exposed)", 0.0) + t
        return t
