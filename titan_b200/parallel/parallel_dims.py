"""`ParallelDims`: degrees of every parallelism axis and the device meshes built from them.

World layout (slowest → fastest varying rank index):

    dense  view: [pp, dp_replicate, dp_shard, cp, tp]
    sparse view: [pp, dp_replicate, efsdp, ep, etp]          (same ranks, regrouped for MoE)

Named meshes: ``pp, dp_replicate, dp_shard, cp, tp`` (dense axes), ``fsdp`` =
flatten(dp_shard, cp), ``dp`` = flatten(dp_replicate, dp_shard) (batch axis),
``loss`` = flatten(dp_replicate, dp_shard, cp), and ``efsdp, ep, etp`` from
the sparse view.  The sparse view is its own `DeviceMesh`, so expert-parallel
all-to-all traffic runs on communicators that FSDP all-gather / reduce-scatter
never touch and the two overlap on NVLink.

Parity: `ParallelDims(dp_replicate, dp_shard, cp, tp, pp, ep, etp, world_size)`
with meshes ``pp, dp_replicate, fsdp, efsdp, ep, etp, tp, cp, loss``
(tests/testing/parallel_dims.py:9-29), the dedicated EP process group
(torchtitan_npu/train.py:136-175), `seq_len_divisor`,
`fsdp_gradient_divide_factor`, `non_data_parallel_size`
(models/deepseek_v32/parallelize.py:141-144,255-276).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
from torch.distributed.device_mesh import DeviceMesh

__all__ = ["ParallelDims"]


@dataclass
class ParallelDims:
    dp_replicate: int = 1
    dp_shard: int = -1
    cp: int = 1
    tp: int = 1
    pp: int = 1
    ep: int = 1
    etp: int = 1
    world_size: int = 1
    dedicated_ep_group: bool = True

    _meshes: dict[str, DeviceMesh] = field(default_factory=dict, init=False, repr=False)
    _dense: DeviceMesh | None = field(default=None, init=False, repr=False)
    _sparse: DeviceMesh | None = field(default=None, init=False, repr=False)
    _device_type: str = field(default="cpu", init=False, repr=False)

    def __post_init__(self):
        self._validate()

    # ------------------------------------------------------------------ validation
    def _validate(self):
        for name in ("dp_replicate", "cp", "tp", "pp", "ep", "etp"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be >= 1, got {getattr(self, name)}")
        if self.dp_shard != -1 and self.dp_shard < 1:
            raise ValueError("dp_shard must be -1 (auto) or >= 1")
        rest = self.dp_replicate * self.cp * self.tp * self.pp
        if self.dp_shard == -1:
            if self.world_size % rest != 0:
                raise ValueError(f"world_size {self.world_size} not divisible by dp_replicate*cp*tp*pp = {rest}")
            self.dp_shard = self.world_size // rest
        if rest * self.dp_shard != self.world_size:
            raise ValueError(
                f"dp_replicate({self.dp_replicate}) * dp_shard({self.dp_shard}) * cp({self.cp}) * tp({self.tp}) "
                f"* pp({self.pp}) != world_size({self.world_size})"
            )
        if self.ep > 1:
            if self.etp not in (1, self.tp):
                raise ValueError("etp must be 1 or equal to tp")
            pool = self.dp_shard * self.cp * (self.tp if self.etp == 1 else 1)
            if pool % self.ep != 0:
                raise ValueError(f"ep({self.ep}) must divide dp_shard*cp{'*tp' if self.etp == 1 else ''} = {pool}")
            if self.etp == self.tp and self.ep % self.cp != 0 and self.cp % self.ep != 0:
                raise ValueError("ep and cp must divide one another")

    # ------------------------------------------------------------------ derived sizes
    @property
    def efsdp(self) -> int:
        if self.ep == 1:
            return self.dp_shard * self.cp
        pool = self.dp_shard * self.cp * (self.tp if self.etp == 1 else 1)
        return pool // self.ep

    @property
    def dp_enabled(self) -> bool:
        return self.dp_replicate > 1 or self.dp_shard > 1

    @property
    def dp_replicate_enabled(self) -> bool:
        return self.dp_replicate > 1

    @property
    def dp_shard_enabled(self) -> bool:
        return self.dp_shard > 1

    @property
    def fsdp_enabled(self) -> bool:
        return self.dp_shard > 1 or self.cp > 1

    @property
    def cp_enabled(self) -> bool:
        return self.cp > 1

    @property
    def tp_enabled(self) -> bool:
        return self.tp > 1

    @property
    def pp_enabled(self) -> bool:
        return self.pp > 1

    @property
    def ep_enabled(self) -> bool:
        return self.ep > 1

    @property
    def etp_enabled(self) -> bool:
        return self.etp > 1

    @property
    def fsdp_gradient_divide_factor(self) -> int:
        """Every FSDP group (dense and expert) divides by the same factor so grads are consistent."""
        return self.dp_replicate * self.dp_shard * self.cp

    @property
    def non_data_parallel_size(self) -> int:
        return self.cp * self.tp * self.pp

    @property
    def seq_len_divisor(self) -> int:
        # SP shards the sequence by tp; CP by 2*cp (room for a head-tail balancer even when unused)
        return self.tp * (self.cp * 2)

    @property
    def dp_degree(self) -> int:
        return self.dp_replicate * self.dp_shard

    # ------------------------------------------------------------------ mesh construction
    def build_mesh(self, device_type: str | None = None) -> DeviceMesh:
        if device_type is None:
            device_type = "cuda" if torch.cuda.is_available() else "cpu"
        self._device_type = device_type
        ranks = torch.arange(self.world_size, dtype=torch.int)
        dense = ranks.view(self.pp, self.dp_replicate, self.dp_shard, self.cp, self.tp)
        self._dense = DeviceMesh(
            device_type, dense, mesh_dim_names=("pp", "dp_replicate", "dp_shard", "cp", "tp")
        )
        m = self._meshes
        for n in ("pp", "dp_replicate", "dp_shard", "cp", "tp"):
            m[n] = self._dense[n]
        m["fsdp"] = self._dense["dp_shard", "cp"]._flatten("fsdp")
        m["dp"] = self._dense["dp_replicate", "dp_shard"]._flatten("dp")
        m["loss"] = self._dense["dp_replicate", "dp_shard", "cp"]._flatten("loss")

        # ep == 1: experts (if any) are sharded like dense params; the last axis is tp.
        # ep > 1, etp == tp: efsdp * ep == dp_shard * cp, last axis is tp.
        # ep > 1, etp == 1 : tp ranks are borrowed by ep: efsdp * ep == dp_shard * cp * tp, last axis is 1.
        last = self.tp if (self.ep == 1 or self.etp == self.tp) else 1
        sparse = ranks.view(self.pp, self.dp_replicate, self.efsdp, self.ep, last)
        if self.ep > 1:
            self._sparse = DeviceMesh(
                device_type, sparse.contiguous(), mesh_dim_names=("pp_s", "dp_replicate_s", "efsdp", "ep", "etp")
            )
            for n in ("efsdp", "ep", "etp"):
                m[n] = self._sparse[n]
        else:
            m["efsdp"], m["ep"], m["etp"] = m["fsdp"], None, None
        return self._dense

    @property
    def world_mesh(self) -> DeviceMesh:
        if self._dense is None:
            self.build_mesh()
        return self._dense

    def _enabled(self, name: str) -> bool:
        size = {
            "pp": self.pp,
            "dp_replicate": self.dp_replicate,
            "dp_shard": self.dp_shard,
            "cp": self.cp,
            "tp": self.tp,
            "ep": self.ep,
            "etp": self.etp,
            "efsdp": self.efsdp,
            "fsdp": self.dp_shard * self.cp,
            "dp": self.dp_replicate * self.dp_shard,
            "loss": self.dp_replicate * self.dp_shard * self.cp,
        }[name]
        return size > 1

    def get_mesh(self, name: str | tuple[str, ...]) -> DeviceMesh:
        """Mesh for an axis (or a tuple of dense axes); raises if the axis has degree 1."""
        if self._dense is None:
            self.build_mesh()
        if isinstance(name, (tuple, list)):
            names = tuple(name)
            if set(names) <= {"dp_replicate", "fsdp"}:
                # HSDP 2-D mesh: (replicate, shard)
                return self._hsdp_mesh()
            if set(names) <= {"dp_replicate", "efsdp"}:
                return self._hsdp_mesh(expert=True)
            return self._dense[names]
        if not self._enabled(name):
            raise ValueError(f"mesh {name!r} has degree 1; use get_optional_mesh")
        return self._meshes[name]

    def get_optional_mesh(self, name: str) -> DeviceMesh | None:
        if self._dense is None:
            if self.world_size == 1 and not torch.distributed.is_initialized():
                return None   # a single process without a process group: every degree is 1, no mesh to hand out
            self.build_mesh()
        if name not in self._meshes or self._meshes[name] is None or not self._enabled(name):
            return None
        return self._meshes[name]

    def mesh_even_if_trivial(self, name: str) -> DeviceMesh | None:
        """Like `get_optional_mesh` but also returns meshes of degree 1 (None only if never built)."""
        if self._dense is None:
            if self.world_size == 1 and not torch.distributed.is_initialized():
                return None
            self.build_mesh()
        return self._meshes.get(name)

    def _hsdp_mesh(self, expert: bool = False) -> DeviceMesh:
        key = "hsdp_e" if expert else "hsdp"
        if key not in self._meshes:
            ranks = torch.arange(self.world_size, dtype=torch.int)
            if expert:
                t = ranks.view(self.pp, self.dp_replicate, self.efsdp, -1).permute(0, 3, 1, 2)
                names = ("pp_h", "rest_h", "dp_replicate", "efsdp")
            else:
                t = ranks.view(self.pp, self.dp_replicate, self.dp_shard * self.cp, self.tp).permute(0, 3, 1, 2)
                names = ("pp_h", "rest_h", "dp_replicate", "fsdp")
            full = DeviceMesh(self._device_type, t.contiguous(), mesh_dim_names=names)
            self._meshes[key] = full[names[2], names[3]]
        return self._meshes[key]

    # ------------------------------------------------------------------ coordinates
    def coordinate(self, rank: int) -> dict[str, int]:
        """Index of `rank` along each dense axis (pure arithmetic; no process group needed)."""
        out = {}
        r = rank
        for name, size in (("tp", self.tp), ("cp", self.cp), ("dp_shard", self.dp_shard),
                           ("dp_replicate", self.dp_replicate), ("pp", self.pp)):
            out[name] = r % size
            r //= size
        return out
